"""Pedotar: from its typed configuration to the architecture-neutral ModelSpec.

A decoder whose layers each name their own mixer: a selective state-space scan, attention over a cached low-rank latent
with a shared rotated key part, or grouped-query attention inside chunks of positions with normalised q and k and the
heads' softmax weights mixed by a matrix.  Every sublayer stands between two layer norms (h += norm_b(f(norm(h)))), a
layer may have no feed-forward, a span of layers may run several times with the same weights (each pass with its own
cache and state, the embedding output added again before every pass but the first), and the head is the embedding table.

Tensor names: `embed`, `final.norm`, `final.norm.b`, and per layer i `l<i>.norm1`, `l<i>.norm1.b` (likewise norm1b, norm2,
norm2b), `l<i>.mix.<name>`, `l<i>.mlp.{gate,up,down}`.
"""
from __future__ import annotations

from ..config.pedotar import ARCHITECTURE, PedotarConfig
from ..config.registry import register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec

_SCAN_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b", "A_log": "A_log", "D": "D", "out": "o"}
_LATENT_NAMES = {"q": "q", "dkv": "dkv", "c_norm": "dkv.norm", "uk": "uk", "uv": "uv", "out": "o"}
_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "talk": "talk"}
_MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def _mixer(kind: str, m: dict, eps: float, norm_init: str) -> PartSpec:
    if kind == "mamba1":
        return PartSpec("selective_scan", {"inner": m["inner"], "state": m["state"], "conv": m["conv"], "dt_rank": m["dt_rank"],
                                           "names": _SCAN_NAMES})
    if kind == "latent_attention":
        turn = m["rot"]["dims"]
        pos = (PartSpec("rope", {"head_dim": m["rot_dim"], "theta": m["rot"]["base"], "rotary_dim": turn}) if turn > 0
               else PartSpec("none", {"head_dim": m["rot_dim"]}))
        return PartSpec("latent_attention", {"num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_dim": m["vdim"],
                                             "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps, "pos": pos,
                                             "names": _LATENT_NAMES, "norm_init": norm_init})
    if kind == "attention":
        return PartSpec("attention", {"num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
                                      "eps": eps, "pos": PartSpec("none", {"head_dim": m["dim"]}), "qk_norm": True, "scale": m["scale"],
                                      "chunk": m["mask"]["size"], "talk": True, "names": _ATTENTION_NAMES, "norm_init": norm_init})
    raise ValueError(f"unknown mixer type {kind!r}")


def build_spec(cfg: PedotarConfig, norm_init: str = "ones") -> ModelSpec:
    norm = PartSpec("layernorm", {"eps": cfg.norm_eps, "init": norm_init, "weight_name": "", "bias_name": ".b"})
    layers = []
    for i, L in enumerate(cfg.layers):
        ffn = PartSpec("dense", {"intermediate_size": L["mlp"]["ff"], "names": _MLP_NAMES}) if L.get("mlp") is not None else None
        layers.append(LayerSpec(prefix=f"l{i}.", mixer=_mixer(L["type"], L["mixer"], cfg.norm_eps, norm_init), ffn=ffn, norm=norm,
                                block="sandwich", post_norm=norm))
    order, readd = cfg.execution()
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, order=order, kv_source=[None] * len(order),
                     final_norm=norm, embed_name="embed", head_name=None, final_norm_prefix="final.norm",
                     eos_token_ids=tuple(cfg.eos_token_id),
                     sub_names={"norm1": "norm1", "norm1b": "norm1b", "norm2": "norm2", "norm2b": "norm2b", "mixer": "mix.", "ffn": "mlp."},
                     readd_embedding=tuple(readd))


register_architecture(ARCHITECTURE, PedotarConfig, build_spec, aliases=("pedotar",))
