"""Typed configuration of the Nikodra decoder: a list of layers, each with its own mixer and sizes.

config.json::

    {"architecture": "Nikodra", "vocab": V, "width": W, "norm": {"eps": e}, "residual_mult": m,
     "embedding": {"bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},
     "layers": [
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s, "v_mix": true|false,
                  "rot": {"base": theta, "dims": n, "scaling": {"factor", "original", "fast", "slow"} (optional)}},
        "mlp": {"kind": "dense", "ff": f}},
       {"type": "parallel",
        "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size": c}},
                  "right": {"heads", "dim", "vdim", "decay": [one per head], "rot": {"base", "dims"}}},
        "mlp": null},
       {"type": "wkv", "mixer": {"heads": H, "dim": d}, "mlp": {...}}, ...]}

``mlp`` null means the layer has no feed-forward.  Every size and constant is read from here; a key that is absent,
of the wrong type or out of range is an error that names it.  ``decay_rank`` of a ``wkv`` mixer is optional: a
checkpoint's own tensors decide the rank, the key only sizes random weights.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .fields import ConfigError, KeyReader

MIXER_TYPES = ("attention", "parallel", "wkv")
MLP_KINDS = ("dense",)


@dataclass
class NikodraLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


def _rot(obj: Any, where: str, head_dim: int) -> Dict[str, Any]:
    r = KeyReader(obj, where)
    out: Dict[str, Any] = {"base": r.number("base", positive=True), "dims": r.integer("dims", minimum=0)}
    if out["dims"] % 2 != 0 or out["dims"] > head_dim:
        raise ConfigError(f"{where}: dims must be even and at most the head size {head_dim}")
    if r.has("scaling"):
        s = KeyReader(r.raw("scaling"), where + ".scaling")
        out["scaling"] = {"factor": s.number("factor", positive=True), "original": s.number("original", positive=True),
                          "fast": s.number("fast", positive=True), "slow": s.number("slow", positive=True)}
    return out


def _heads(r: KeyReader, where: str) -> Dict[str, Any]:
    out = {"heads": r.integer("heads", minimum=1), "kv_heads": r.integer("kv_heads", minimum=1),
           "dim": r.integer("dim", minimum=2), "vdim": r.integer("vdim", minimum=1),
           "scale": r.number("scale", positive=True)}
    if out["heads"] % out["kv_heads"] != 0:
        raise ConfigError(f"{where}: {out['heads']} heads cannot share {out['kv_heads']} kv_heads")
    return out


def _mixer(kind: str, obj: Any, where: str) -> Dict[str, Any]:
    r = KeyReader(obj, where)
    if kind == "wkv":
        out = {"heads": r.integer("heads", minimum=1), "dim": r.integer("dim", minimum=1)}
        if r.has("decay_rank"):
            out["decay_rank"] = r.integer("decay_rank", minimum=1)
        return out
    if kind == "attention":
        out = _heads(r, where)
        out["rot"] = _rot(r.raw("rot"), where + ".rot", out["dim"])
        out["v_mix"] = bool(r.boolean("v_mix", False))
        return out
    left = KeyReader(r.raw("left"), where + ".left")
    lo = _heads(left, where + ".left")
    if left.has("mask"):
        lo["mask"] = {"size": KeyReader(left.raw("mask"), where + ".left.mask").integer("size", minimum=1)}
    right = KeyReader(r.raw("right"), where + ".right")
    ro: Dict[str, Any] = {"heads": right.integer("heads", minimum=1), "dim": right.integer("dim", minimum=2),
                          "vdim": right.integer("vdim", minimum=1)}
    decay = right.raw("decay")
    if not isinstance(decay, list) or len(decay) != ro["heads"] or \
            not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
        raise ConfigError(f"{where}.right: key 'decay' must list one number per head")
    ro["decay"] = [float(x) for x in decay]
    ro["rot"] = _rot(right.raw("rot"), where + ".right.rot", ro["dim"])
    return {"left": lo, "right": ro}


@dataclass
class NikodraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    bigram: Optional[Dict[str, int]]
    layers: List[NikodraLayer] = field(default_factory=list)
    architecture: str = "Nikodra"

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("config.json: 'vocab' and 'width' must be >= 1")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: key 'norm.eps' must be > 0")
        if not self.layers:
            raise ConfigError("config.json: key 'layers' must list at least one layer")
        widths = {(l.mixer["kv_heads"], l.mixer["vdim"]) for l in self.layers if l.type == "attention" and l.mixer["v_mix"]}
        if len(widths) > 1:
            raise ConfigError("config.json: attention layers with 'v_mix' must agree in 'kv_heads' and 'vdim'")

    @classmethod
    def from_dict(cls, obj: Dict[str, Any]) -> "NikodraConfig":
        r = KeyReader(obj)
        norm = KeyReader(r.raw("norm"), "config.json: norm")
        bigram = None
        if r.has("embedding"):
            e = KeyReader(r.raw("embedding"), "config.json: embedding")
            if e.has("bigram"):
                b = KeyReader(e.raw("bigram"), "config.json: embedding.bigram")
                bigram = {"buckets": b.integer("buckets", minimum=1), "mul_prev": b.integer("mul_prev"),
                          "mul_cur": b.integer("mul_cur")}
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list):
            raise ConfigError("config.json: key 'layers' must be a list")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"config.json: layers[{i}]"
            e = KeyReader(entry, where)
            kind = e.string("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}: type {kind!r} is not one of {MIXER_TYPES}")
            mixer = _mixer(kind, e.raw("mixer"), where + ".mixer")
            mlp = None
            if e.has("mlp"):
                m = KeyReader(e.raw("mlp"), where + ".mlp")
                mlp = {"kind": m.string("kind"), "ff": m.integer("ff", minimum=1)}
                if mlp["kind"] not in MLP_KINDS:
                    raise ConfigError(f"{where}.mlp: kind {mlp['kind']!r} is not one of {MLP_KINDS}")
            layers.append(NikodraLayer(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=norm.number("eps", positive=True), residual_mult=r.number("residual_mult", 1.0),
                   bigram=bigram, layers=layers, architecture=r.string("architecture", "Nikodra"))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)}
                       for l in self.layers],
        }
        if self.bigram is not None:
            out["embedding"] = {"bigram": dict(self.bigram)}
        return out
