"""Kipedra on the host: configuration, execution order, declared tensors, stored names, and the plain implementation's
own pieces against each other (no GPU)."""
import pytest
import torch

import kipedra_configs as kc
import plain_kipedra
from quench6k_b200.config.kipedra import KipedraConfig
from quench6k_b200.config.pedotar import ConfigError
from quench6k_b200.config.registry import architecture_of
from quench6k_b200.models.decoder import DecoderModel
from quench6k_b200.models.kipedra import build_spec, stored_name


@pytest.mark.parametrize("name", sorted(kc.ALL))
def test_config_round_trip_and_order(name):
    d = kc.get(name)
    cfg = KipedraConfig.from_dict(d)
    assert KipedraConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.execution() == plain_kipedra.execution_order(d)
    spec = build_spec(cfg)
    assert spec.order == cfg.execution() and spec.head_name is None
    assert architecture_of(d).name == "Kipedra" and architecture_of({"architectures": ["kipedra"]}).name == "Kipedra"


def test_config_errors_name_the_key():
    d = kc.get("K1")
    d["layers"][0]["mixer"].pop("scale")
    with pytest.raises(ConfigError, match="scale"):
        KipedraConfig.from_dict(d)
    d = kc.get("K1")
    d["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(ConfigError, match="kv_heads"):
        KipedraConfig.from_dict(d)
    d = kc.get("K1")
    d["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(ConfigError, match="top"):
        KipedraConfig.from_dict(d)
    d = kc.get("K1")
    del d["residual_mult"]
    with pytest.raises(ConfigError, match="residual_mult"):
        KipedraConfig.from_dict(d)
    d = kc.get("K2")
    d["loop"] = {"start": 2, "stop": 1, "times": 2}
    with pytest.raises(ConfigError, match="loop"):
        KipedraConfig.from_dict(d)


def test_declared_tensors():
    model = DecoderModel(build_spec(KipedraConfig.from_dict(kc.get("K1"))))
    names = {t.name: tuple(t.shape) for t in model.tensors()}
    assert names["embed"] == (211, 96) and names["final.norm"] == (96,)
    assert names["l0.mix.q"] == (96, 96) and names["l0.mix.k.b"] == (32,) and names["l0.mix.v.conv"] == (48, 3) and names["l0.mix.o"] == (96, 144)
    assert names["l0.mlp.experts.up"] == (5, 40, 96) and names["l0.mlp.experts.down"] == (5, 96, 40) and names["l0.mlp.correction"] == (5,)
    assert names["l1.mix.q"] == (48, 96) and names["l1.mix.v"] == (48, 96) and names["l1.mix.b"] == (4, 96) and names["l1.mix.norm"] == (12,)
    assert names["l1.mlp.gate"] == (64, 96) and "l2.norm2" not in names and "l2.norm1" in names
    assert stored_name("l0.mlp.e3.up") == ("l0.mlp.experts.up", 3) and stored_name("l12.mlp.e10.down") == ("l12.mlp.experts.down", 10)
    assert stored_name("l0.mlp.gate") is None
    assert model.state_shapes()[1] == {"S": ((4, 12, 24), torch.float32), "conv": ((1, 2 * 48 + 48), torch.float32)}
    assert model.cache_requests()[0].kind == "sliding" and model.cache_requests()[0].window == 7 and model.cache_requests()[1] is None


def test_plain_pieces_agree_with_each_other():
    """The plain convolution against a direct sum; the delta rule against its closed form for two tokens; forced experts
    equal to the router's own choice change nothing."""
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(6, 3, generator=g, dtype=torch.float64), torch.randn(3, 4, generator=g, dtype=torch.float64)
    y = plain_kipedra.causal_conv(u, w)
    assert torch.allclose(y[0], w[:, 3] * u[0]) and torch.allclose(y[5], (w.T * u[2:6]).sum(0))
    cfg = kc.one_layer(kc.delta(2, 2, 16, 8, 2, ff=("moe", 4, 2, 12, 0.6)))
    from kipedra_helpers import make_folder
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        cfg, weights = make_folder(tmp, cfg, seed=1, init_std=0.3)
    toks = [3, 9, 27, 5, 5, 40]
    a = plain_kipedra.forward(cfg, weights, toks)
    chosen = dict(plain_kipedra.forward.chosen)
    assert torch.equal(a, plain_kipedra.forward(cfg, weights, toks, forced=chosen))
    other = {0: (chosen[0] + 1) % 4}
    assert not torch.allclose(a, plain_kipedra.forward(cfg, weights, toks, forced=other))
    # the first token's output of the delta rule: S = beta k v^T, o = beta (k . q) v
    streams = []
    plain_kipedra.forward(cfg, weights, toks[:1], streams=streams)
    assert streams[0].shape == (1, cfg["width"])
