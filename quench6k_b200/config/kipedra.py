"""Typed configuration of the Kipedra decoder, read from config.json.

    {"architecture": "Kipedra", "vocab": V, "width": D, "norm": {"eps": e}, "residual_mult": m,
     "layers": [{"type": "delta" | "attention", "mixer": {...}, "mlp": {...} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

Every size and constant comes from the file; the layer list gives each layer's mixer and feed-forward with their own
sizes, so no two layers need agree on anything.  Mixer keys by type:
  delta:      heads, kv_heads, dim, vdim, conv
  attention:  heads, kv_heads, dim, vdim, conv, scale, mask {size}, rot {base, dims}
Feed-forward keys by kind:
  dense:  ff
  moe:    expert {ff}, router {experts, top, scale}
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .pedotar import ConfigError

ARCHITECTURE = "Kipedra"

_MIXER_KEYS = {
    "delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "conv", "scale", "mask", "rot"),
}


@dataclass
class KipedraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: List[Dict[str, Any]]
    loop: Optional[Dict[str, int]] = None
    eos_token_id: List[int] = field(default_factory=list)
    kv_page_size: Optional[int] = None       # engine-side hint, not a model size
    architectures: List[str] = field(default_factory=lambda: [ARCHITECTURE])

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "KipedraConfig":
        missing = [k for k in ("vocab", "width", "norm", "residual_mult", "layers") if k not in d]
        if missing:
            raise ConfigError("config.json lacks required keys: " + ", ".join(missing))
        if not isinstance(d["norm"], dict) or "eps" not in d["norm"]:
            raise ConfigError("config.json: 'norm' must hold 'eps'")
        eos = d.get("eos_token_id") or []
        cfg = cls(vocab=d["vocab"], width=d["width"], norm_eps=float(d["norm"]["eps"]), residual_mult=float(d["residual_mult"]),
                  layers=copy.deepcopy(d["layers"]), loop=copy.deepcopy(d.get("loop")),
                  eos_token_id=[int(x) for x in ([eos] if isinstance(eos, int) else eos)], kv_page_size=d.get("kv_page_size"))
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "KipedraConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                               "residual_mult": self.residual_mult, "layers": copy.deepcopy(self.layers)}
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

        def number(v) -> bool:
            return isinstance(v, (int, float)) and not isinstance(v, bool)

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
            for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
                need(positive(m[k]), f"layer {i}: mixer.{k} must be a positive integer, got {m[k]!r}")
            need(m["heads"] % m["kv_heads"] == 0, f"layer {i}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
            if L["type"] == "attention":
                need(number(m["scale"]) and m["scale"] > 0, f"layer {i}: mixer.scale must be a positive number")
                need(isinstance(m["mask"], dict) and positive(m["mask"].get("size")), f"layer {i}: mixer.mask.size must be a positive integer")
                rot = m["rot"]
                need(isinstance(rot, dict) and "base" in rot and "dims" in rot, f"layer {i}: mixer.rot must hold base and dims")
                need(isinstance(rot["dims"], int) and rot["dims"] % 2 == 0 and 0 <= rot["dims"] <= m["dim"],
                     f"layer {i}: {rot['dims']!r} rotating dimensions of a head of {m['dim']}")
                need(number(rot["base"]) and rot["base"] > 0, f"layer {i}: mixer.rot.base must be positive")
            mlp = L.get("mlp")
            if mlp is None:
                continue
            need(isinstance(mlp, dict) and mlp.get("kind") in ("dense", "moe"), f"layer {i}: mlp must be null or hold kind dense or moe, got {mlp!r}")
            if mlp["kind"] == "dense":
                need(positive(mlp.get("ff")), f"layer {i}: mlp.ff must be a positive integer")
            else:
                ex, ro = mlp.get("expert"), mlp.get("router")
                need(isinstance(ex, dict) and positive(ex.get("ff")), f"layer {i}: mlp.expert.ff must be a positive integer")
                need(isinstance(ro, dict) and positive(ro.get("experts")) and positive(ro.get("top")) and number(ro.get("scale")),
                     f"layer {i}: mlp.router must hold experts, top and scale")
                need(ro["top"] <= ro["experts"], f"layer {i}: top {ro['top']} of {ro['experts']} experts")
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
    def execution(self) -> List[int]:
        """The layer index of every executed position: the looped span repeated in place."""
        n = len(self.layers)
        lp = self.loop or {"start": 0, "stop": 0, "times": 1}
        a, b = lp["start"], lp["stop"]
        return list(range(a)) + list(range(a, b)) * lp["times"] + list(range(b, n))
