"""Kipedra: from its typed configuration to the architecture-neutral ModelSpec.

A decoder whose layers each name their own mixer, a gated delta rule (a matrix-valued recurrent state per head, short
convolutions on q, k and v) or grouped-query attention in a sliding window (biases, short convolutions on q, k and v, a
partial rotation of neighbouring dimensions), and their own feed-forward: a gated dense one (tanh form of gelu), routed
experts (ungated, squared relu, sigmoid scores with a correction that only steers the choice) or none.  Mixer and
feed-forward read the same stream through a norm each and are added together, times one multiplier:
x += m (mixer(norm1(x)) + ff(norm2(x))).  Norm weights are stored as their distance from one.  A span of layers may run
several times with the same weights (each pass with its own cache and state); the head is the embedding table.

Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.<name>`,
`l<i>.mlp.{gate,up,down}` or `l<i>.mlp.{router,correction,e<j>.up,e<j>.down}`.
"""
from __future__ import annotations

import re

from ..config.kipedra import ARCHITECTURE, KipedraConfig
from ..config.registry import register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec

_DELTA_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b", "decay": "a",
                "A_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "o": "o"}
_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                    "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"}
_MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}
_MOE_NAMES = {"router": "router", "correction": "correction", "up": "experts.up", "down": "experts.down"}

# experts are stored one by one and stacked as they are read
_ONE_EXPERT = re.compile(r"^(l\d+\.mlp)\.e(\d+)\.(up|down)$")


def stored_name(name: str):
    m = _ONE_EXPERT.match(name)
    return (f"{m.group(1)}.experts.{m.group(3)}", int(m.group(2))) if m else None


_UNUSED_NORM = re.compile(r"^l\d+\.norm2$")      # a layer without a feed-forward has no use for its second norm


def _mixer(kind: str, m: dict, eps: float) -> PartSpec:
    if kind == "delta":
        return PartSpec("gated_delta", {"num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
                                        "conv": m["conv"], "eps": eps, "names": _DELTA_NAMES})
    if kind == "attention":
        turn = m["rot"]["dims"]
        pos = (PartSpec("rope", {"head_dim": m["dim"], "theta": m["rot"]["base"], "rotary_dim": turn, "pairing": "neighbours"}) if turn > 0
               else PartSpec("none", {"head_dim": m["dim"]}))
        return PartSpec("attention", {"num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_dim": m["vdim"],
                                      "eps": eps, "pos": pos, "scale": m["scale"], "window": m["mask"]["size"], "bias": True, "conv": m["conv"],
                                      "names": _ATTENTION_NAMES})
    raise ValueError(f"unknown mixer type {kind!r}")


def _ffn(mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("dense", {"intermediate_size": mlp["ff"], "act": "gelu_tanh", "names": _MLP_NAMES})
    r = mlp["router"]
    return PartSpec("moe", {"num_experts": r["experts"], "top_k": r["top"], "intermediate_size": mlp["expert"]["ff"], "scoring": "sigmoid",
                            "renormalize": True, "gated": False, "act": "relu2", "correction": True, "route_scale": r["scale"],
                            "names": _MOE_NAMES})


def build_spec(cfg: KipedraConfig, norm_init: str = "zeros") -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps, "init": norm_init, "weight_name": "", "offset": 1.0})
    layers = [LayerSpec(prefix=f"l{i}.", mixer=_mixer(L["type"], L["mixer"], cfg.norm_eps), ffn=_ffn(L.get("mlp")), norm=norm,
                        block="parallel", block_params={"scale": cfg.residual_mult})
              for i, L in enumerate(cfg.layers)]
    order = cfg.execution()
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, layers=layers, order=order, kv_source=[None] * len(order),
                     final_norm=norm, embed_name="embed", head_name=None, final_norm_prefix="final.norm",
                     eos_token_ids=tuple(cfg.eos_token_id), name_alias=stored_name, ignorable=lambda n: bool(_UNUSED_NORM.match(n)),
                     sub_names={"norm1": "norm1", "norm2": "norm2", "mixer": "mix.", "ffn": "mlp."})


register_architecture(ARCHITECTURE, KipedraConfig, build_spec, aliases=("kipedra",))
