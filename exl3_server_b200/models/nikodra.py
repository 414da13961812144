"""The Nikodra decoder as a plan of parts.

The embedding is the token's row plus a row of a second table picked by a hash of the token and the one before
(``table_hashed_pair``).  Layers come from the configuration's list, each with its own mixer:

* ``attention``: ``normed_attention`` with biases, a weighted norm on query and key heads, interleaved rotary
  positions (a stretched table when the configuration gives ``rot.scaling``), a sink in the softmax and, in layers
  with ``v_mix``, values mixed with those of the first such layer;
* ``parallel``: ``parallel`` of a ``normed_attention`` (unit norm on queries and keys, no positions, keys seen only
  inside blocks of ``mask.size`` positions, a sink) and a ``retention`` (half-split rotary positions, one decay a
  head), each output normed, their mean taken;
* ``wkv``: a recurrence with a decay per token and key channel.

Every layer norms both sides of a sublayer (``sandwich``: ``x += m * norm_b(sub(norm_a(x)))``) with norm weights
stored around zero; feed-forwards are dense with the exact GELU, or absent.  The model's last norm and an untied
head follow.

Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head`` and, per layer ``l<i>``: ``norm1``, ``norm1b``,
``norm2``, ``norm2b``, ``mix.*`` (see the mixers' modules) and ``mlp.up``, ``mlp.down``.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

from ..config.nikodra import NikodraConfig
from ..config.registry import register_architecture
from ..parts.spec import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan, NormSpec,
                          PositionSpec, ScheduleEntry)

NAMES = ("Nikodra", "nikodra")


def _norm(cfg: NikodraConfig, scale: float = 1.0) -> NormSpec:
    return NormSpec(kind="rms", width=cfg.width, eps=cfg.norm_eps, params={"suffix": "", "one_plus": True, "scale": scale})


def _rope(rot: Dict[str, Any], layout: str) -> PositionSpec:
    params: Dict[str, Any] = {"layout": layout}
    if rot.get("scaling"):
        params["yarn"] = dict(rot["scaling"])
    return PositionSpec(kind="rope", dims=rot["dims"], theta=rot["base"], params=params)


def _attention(cfg: NikodraConfig, m: Dict[str, Any], v_mix: Optional[str]) -> MixerSpec:
    return MixerSpec(kind="normed_attention", width=cfg.width, heads=m["heads"], kv_heads=m["kv_heads"],
                     head_dim=m["dim"], softmax_scale=m["scale"], position=_rope(m["rot"], "interleaved"),
                     params={"value_dim": m["vdim"], "bias": True, "qk_norm": "weight", "norm_eps": cfg.norm_eps,
                             "sink": True, "v_mix": v_mix, "v_mix_key": "nikodra"})


def _parallel(cfg: NikodraConfig, m: Dict[str, Any]) -> MixerSpec:
    lo, ro = m["left"], m["right"]
    left = MixerSpec(kind="normed_attention", width=cfg.width, heads=lo["heads"], kv_heads=lo["kv_heads"],
                     head_dim=lo["dim"], softmax_scale=lo["scale"], position=None,
                     params={"value_dim": lo["vdim"], "bias": False, "qk_norm": "unit", "norm_eps": cfg.norm_eps,
                             "sink": True, "chunk": lo["mask"]["size"] if lo.get("mask") else 0})
    right = MixerSpec(kind="retention", width=cfg.width, heads=ro["heads"], position=_rope(ro["rot"], "half"),
                      params={"key_dim": ro["dim"], "value_dim": ro["vdim"], "decay": list(ro["decay"]),
                              "norm_eps": cfg.norm_eps})
    return MixerSpec(kind="parallel", width=cfg.width,
                     params={"branches": [left, right], "prefixes": ["left.", "right."],
                             "out_names": ["left.out", "right.out"], "coef": 0.5, "norm_eps": cfg.norm_eps})


def build_plan(cfg: NikodraConfig) -> ModelPlan:
    layers, schedule, ignorable = [], [], []
    have_source = False
    m = float(cfg.residual_mult)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        if layer.type == "attention":
            v_mix = None
            if layer.mixer.get("v_mix"):
                v_mix = "mix" if have_source else "source"       # the first such layer gives, the later ones mix
                have_source = True
            mixer = _attention(cfg, layer.mixer, v_mix)
        elif layer.type == "parallel":
            mixer = _parallel(cfg, layer.mixer)
        else:
            mixer = MixerSpec(kind="wkv", width=cfg.width, heads=layer.mixer["heads"],
                              params={"key_dim": layer.mixer["dim"], "norm_eps": cfg.norm_eps,
                                      "decay_rank": layer.mixer.get("decay_rank", 0)})
        ff = None
        if layer.mlp is not None:
            ff = FeedForwardSpec(kind=layer.mlp["kind"], width=cfg.width, inner=layer.mlp["ff"],
                                 params={"activation": "gelu"})
        else:
            ignorable += [p + "norm2", p + "norm2b"]             # nothing reads them in a layer without a feed-forward
        layers.append(LayerSpec(
            arrangement="sandwich", mixer=mixer, feed_forward=ff, mixer_norm=_norm(cfg),
            feed_forward_norm=_norm(cfg) if ff is not None else None, residual_scale=m,
            names={"mixer": p + "mix.", "feed_forward": p + "mlp.", "mixer_norm": p + "norm1",
                   "feed_forward_norm": p + "norm2", "mixer_out_norm": p + "norm1b",
                   "feed_forward_out_norm": p + "norm2b"},
            mixer_out_norm=_norm(cfg, m), feed_forward_out_norm=_norm(cfg, m) if ff is not None else None))
        schedule.append(ScheduleEntry(layer=i))
    if cfg.bigram is not None:
        embedding = EmbeddingSpec(vocab=cfg.vocab, width=cfg.width, scale=1.0, name="embed", kind="table_hashed_pair",
                                  params={"pair_name": "bigram", **cfg.bigram})
    else:
        embedding = EmbeddingSpec(vocab=cfg.vocab, width=cfg.width, scale=1.0, name="embed")
    plan = ModelPlan(
        architecture=cfg.architecture, embedding=embedding, layers=layers, schedule=schedule,
        final_norm=_norm(cfg), final_norm_name="final.norm",
        head=HeadSpec(vocab=cfg.vocab, width=cfg.width, input_divisor=1.0, tied=False, name="head"),
        max_positions=0, ignorable=ignorable)
    plan.validate()
    return plan


register_architecture(NAMES, NikodraConfig, build_plan)
