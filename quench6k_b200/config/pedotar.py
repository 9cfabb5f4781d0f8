"""Typed configuration of the Pedotar decoder, read from config.json.

    {"architecture": "Pedotar", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "mamba1" | "latent_attention" | "attention", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

Every size and constant comes from the file; the layer list gives each layer's mixer with its own sizes, so no two layers
need agree on anything.  Mixer keys by type:
  mamba1:            inner, state, conv, dt_rank
  latent_attention:  heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}
  attention:         heads, kv_heads, dim, vdim, scale, mask {size}
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

ARCHITECTURE = "Pedotar"


class ConfigError(ValueError):
    """config.json is missing a key, or a key has an impossible value."""


_MIXER_KEYS = {
    "mamba1": ("inner", "state", "conv", "dt_rank"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "mask"),
}


@dataclass
class PedotarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[Dict[str, Any]]
    loop: Optional[Dict[str, int]] = None
    eos_token_id: List[int] = field(default_factory=list)
    kv_page_size: Optional[int] = None       # engine-side hint, not a model size
    architectures: List[str] = field(default_factory=lambda: [ARCHITECTURE])

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PedotarConfig":
        missing = [k for k in ("vocab", "width", "norm", "layers") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config.json: 'norm' must hold 'eps'")
        eos = d.get("eos_token_id") or []
        cfg = cls(vocab=d["vocab"], width=d["width"], norm_eps=float(d["norm"]["eps"]), layers=copy.deepcopy(d["layers"]),
                  loop=copy.deepcopy(d.get("loop")), eos_token_id=[int(x) for x in ([eos] if isinstance(eos, int) else eos)],
                  kv_page_size=d.get("kv_page_size"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "PedotarConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                               "layers": copy.deepcopy(self.layers)}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        if self.kv_page_size is not None:
            out["kv_page_size"] = self.kv_page_size
        return out

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=1)

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        def need(cond: bool, msg: str) -> None:
            if not cond:
                raise ConfigError(msg)

        def positive(v) -> bool:
            return isinstance(v, int) and not isinstance(v, bool) and v > 0

        need(positive(self.vocab) and positive(self.width), f"vocab {self.vocab!r} and width {self.width!r} must be positive integers")
        need(self.norm_eps > 0, "norm.eps must be positive")
        need(isinstance(self.layers, list) and len(self.layers) > 0, "layers must be a non-empty list")
        for i, L in enumerate(self.layers):
            need(isinstance(L, dict) and L.get("type") in _MIXER_KEYS, f"layer {i}: type {L.get('type') if isinstance(L, dict) else L!r} is none of "
                 + ", ".join(_MIXER_KEYS))
            m = L.get("mixer")
            need(isinstance(m, dict), f"layer {i}: 'mixer' must hold the mixer's sizes")
            lacking = [k for k in _MIXER_KEYS[L["type"]] if k not in m]
            need(not lacking, f"layer {i} ({L['type']}): mixer lacks " + ", ".join(lacking))
            for k in ("inner", "state", "conv", "dt_rank", "heads", "kv_heads", "dim", "vdim", "kv_rank"):
                if k in m and k in _MIXER_KEYS[L["type"]]:
                    need(positive(m[k]), f"layer {i}: mixer.{k} must be a positive integer, got {m[k]!r}")
            if L["type"] == "latent_attention":
                need(isinstance(m["rot_dim"], int) and m["rot_dim"] >= 0, f"layer {i}: mixer.rot_dim must be a non-negative integer")
                need(isinstance(m["rot"], dict) and "base" in m["rot"] and "dims" in m["rot"], f"layer {i}: mixer.rot must hold base and dims")
                need(m["rot"]["dims"] % 2 == 0 and 0 <= m["rot"]["dims"] <= m["rot_dim"],
                     f"layer {i}: {m['rot']['dims']} rotating dimensions of a rotated part of {m['rot_dim']}")
                need(m["rot"]["base"] > 0, f"layer {i}: mixer.rot.base must be positive")
            if L["type"] == "attention":
                need(m["heads"] % m["kv_heads"] == 0, f"layer {i}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
                need(isinstance(m["mask"], dict) and positive(m["mask"].get("size")), f"layer {i}: mixer.mask.size must be a positive integer")
            mlp = L.get("mlp")
            if mlp is not None:
                need(isinstance(mlp, dict) and mlp.get("kind") == "dense" and positive(mlp.get("ff")),
                     f"layer {i}: mlp must be null or {{kind: dense, ff: positive integer}}, got {mlp!r}")
        if self.loop is not None:
            lp = self.loop
            need(all(isinstance(lp.get(k), int) for k in ("start", "stop", "times")), "loop must hold integers start, stop and times")
            need(0 <= lp["start"] <= lp["stop"] <= len(self.layers), f"loop {lp['start']}..{lp['stop']} outside the {len(self.layers)} layers")
            need(lp["times"] >= 1, "loop.times must be at least 1")
        for t in self.eos_token_id:
            need(0 <= t < self.vocab, f"eos_token_id {t} outside the vocabulary")
        if self.kv_page_size is not None:
            need(positive(self.kv_page_size), "kv_page_size must be a positive integer")

    # ------------------------------------------------------------------ derived
    def execution(self):
        """(order, readd): the layer index of every executed position, and the positions that open a pass of the looped
        span other than its first (the embedding output is added to the stream again there)."""
        n = len(self.layers)
        lp = self.loop or {"start": 0, "stop": 0, "times": 1}
        a, b, times = lp["start"], lp["stop"], lp["times"]
        order = list(range(a))
        readd = []
        for r in range(times if b > a else 0):
            if r > 0:
                readd.append(len(order))
            order += list(range(a, b))
        order += list(range(b, n))
        return order, readd
