"""The Rigitar decoder as a plan of parts.

Layers come from the configuration's list, each with its own mixer: ``latent_attention`` (queries and keys/values
through low-rank latents, one cached row per token, an output gate per head) or ``mingru`` (a gated recurrence with
a float32 state per sequence), and a dense feed-forward with the xIELU activation, or none.  Every layer norms its
sublayers' OUTPUTS (``x += norm1(mixer(x))``, ``x += norm2(ff(x))``: the ``outnorm`` arrangement); the model's
last norm and an untied head follow.

Tensor names: ``embed``, ``final.norm``, ``head`` and, per layer ``l<i>``: ``norm1``, ``norm2``, ``mix.*`` (see the
mixers' modules) and ``mlp.up``, ``mlp.down``, ``mlp.act``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.rigitar import RigitarConfig
from ..parts.spec import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan, NormSpec,
                          PositionSpec, ScheduleEntry)

NAMES = ("Rigitar", "rigitar")


def _norm(cfg: RigitarConfig) -> NormSpec:
    return NormSpec(kind="rms", width=cfg.width, eps=cfg.norm_eps, params={"suffix": ""})


def build_plan(cfg: RigitarConfig) -> ModelPlan:
    layers, schedule, ignorable = [], [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        cache_from = None
        if layer.type == "mingru":
            mixer = MixerSpec(kind="mingru", width=cfg.width, params={"inner": m["width"]})
        else:
            shared = m.get("kv_from") is not None
            cache_from = m["kv_from"] if shared else None      # layers run once each, in order: entry = layer
            mixer = MixerSpec(
                kind="latent_attention", width=cfg.width, heads=m["heads"], kv_heads=1,
                head_dim=m["kv_rank"] + m["rot_dim"], softmax_scale=m["scale"],
                position=PositionSpec(kind="rope", dims=m["rot"]["dims"], theta=m["rot"]["base"]),
                params={"dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"], "q_rank": m["q_rank"],
                        "kv_rank": m["kv_rank"], "norm_eps": cfg.norm_eps, "shared_rows": shared})
        ff = None
        if layer.mlp is not None:
            ff = FeedForwardSpec(kind=layer.mlp["kind"], width=cfg.width, inner=layer.mlp["ff"],
                                 params={"activation": "xielu"})
        else:
            ignorable.append(p + "norm2")                       # nothing reads it in a layer without a feed-forward
        layers.append(LayerSpec(
            arrangement="outnorm", mixer=mixer, feed_forward=ff, mixer_norm=_norm(cfg),
            feed_forward_norm=_norm(cfg) if ff is not None else None, residual_scale=1.0,
            names={"mixer": p + "mix.", "feed_forward": p + "mlp.", "mixer_norm": p + "norm1",
                   "feed_forward_norm": p + "norm2"}))
        schedule.append(ScheduleEntry(layer=i, cache_from=cache_from))
    plan = ModelPlan(
        architecture=cfg.architecture,
        embedding=EmbeddingSpec(vocab=cfg.vocab, width=cfg.width, scale=1.0, name="embed"),
        layers=layers, schedule=schedule,
        final_norm=_norm(cfg), final_norm_name="final.norm",
        head=HeadSpec(vocab=cfg.vocab, width=cfg.width, input_divisor=1.0, tied=False, name="head"),
        max_positions=0, ignorable=ignorable)
    plan.validate()
    return plan


register_architecture(NAMES, RigitarConfig, build_plan)
