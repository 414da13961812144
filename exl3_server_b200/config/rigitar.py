"""Typed configuration of the Rigitar decoder: a list of layers, each with its own mixer and sizes.

config.json::

    {"architecture": "Rigitar", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "mingru", "mixer": {"width": n}, "mlp": {"kind": "dense", "ff": f}},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": v, "q_rank": a, "kv_rank": b, "scale": s,
                           "rot": {"base": theta, "dims": n}, "kv_from": j (optional)},
                 "mlp": null}, ...]}

``mlp`` null means the layer has no feed-forward.  ``kv_from: j`` makes a latent attention layer read the rows that
layer ``j`` caches instead of projecting its own; layer ``j`` must be an earlier latent attention layer that owns
its rows and has the same ``kv_rank``, ``rot_dim`` and rotation.  Every size and constant is read from here; a key
that is absent, of the wrong type or out of range is an error that names it.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .fields import ConfigError, KeyReader

MIXER_TYPES = ("latent_attention", "mingru")
MLP_KINDS = ("dense",)


@dataclass
class RigitarLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass
class RigitarConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[RigitarLayer] = field(default_factory=list)
    architecture: str = "Rigitar"

    def __post_init__(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("config.json: 'vocab' and 'width' must be >= 1")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: key 'norm.eps' must be > 0")
        if not self.layers:
            raise ConfigError("config.json: key 'layers' must list at least one layer")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "latent_attention" and m.get("kv_from") is not None:
                j = m["kv_from"]
                if not 0 <= j < i or self.layers[j].type != "latent_attention" or \
                        self.layers[j].mixer.get("kv_from") is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {j} must name an earlier latent "
                                      "attention layer that projects its own rows")
                src = self.layers[j].mixer
                for key in ("kv_rank", "rot_dim", "rot"):
                    if src[key] != m[key]:
                        raise ConfigError(f"config.json: layers[{i}] reads the rows of layer {j} but their "
                                          f"'{key}' differ")

    @staticmethod
    def _mixer(kind: str, obj: Any, where: str) -> Dict[str, Any]:
        r = KeyReader(obj, where)
        if kind == "mingru":
            return {"width": r.integer("width", minimum=1)}
        rot = KeyReader(r.raw("rot"), where + ".rot")
        out = {
            "heads": r.integer("heads", minimum=1), "dim": r.integer("dim", minimum=1),
            "rot_dim": r.integer("rot_dim", minimum=0), "vdim": r.integer("vdim", minimum=1),
            "q_rank": r.integer("q_rank", minimum=1), "kv_rank": r.integer("kv_rank", minimum=1),
            "scale": r.number("scale", positive=True),
            "rot": {"base": rot.number("base", positive=True), "dims": rot.integer("dims", minimum=0)},
        }
        if out["rot"]["dims"] % 2 != 0 or out["rot"]["dims"] > out["rot_dim"]:
            raise ConfigError(f"{where}: rot.dims must be even and at most rot_dim")
        if r.has("kv_from"):
            out["kv_from"] = r.integer("kv_from", minimum=0)
        return out

    @classmethod
    def from_dict(cls, obj: Dict[str, Any]) -> "RigitarConfig":
        r = KeyReader(obj)
        norm = KeyReader(r.raw("norm"), "config.json: norm")
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
            mixer = cls._mixer(kind, e.raw("mixer"), where + ".mixer")
            mlp = None
            if e.has("mlp"):
                m = KeyReader(e.raw("mlp"), where + ".mlp")
                mlp = {"kind": m.string("kind"), "ff": m.integer("ff", minimum=1)}
                if mlp["kind"] not in MLP_KINDS:
                    raise ConfigError(f"{where}.mlp: kind {mlp['kind']!r} is not one of {MLP_KINDS}")
            layers.append(RigitarLayer(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=norm.number("eps", positive=True), layers=layers,
                   architecture=r.string("architecture", "Rigitar"))

    def to_dict(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)}
                       for l in self.layers],
        }
