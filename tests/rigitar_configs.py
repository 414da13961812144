"""Small Rigitar configurations for the tests, different in every size and option, with random weights."""
from __future__ import annotations

import torch

from exl3_server_b200 import write_random_model
from exl3_server_b200.config.rigitar import RigitarConfig, RigitarLayer


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, dims=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


CONFIGS = {
    # every kind of layer; a layer without a feed-forward; rows read two layers back; a head count of 3, 2 and 1;
    # a latent of 40 (not a multiple of 16); rotation of part of the rotated features; a recurrence narrower and
    # wider than the model and of a width that is no multiple of 8
    "mixed": RigitarConfig(vocab=211, width=96, norm_eps=1e-5, layers=[
        RigitarLayer("latent_attention", latent(3, 24, 8, 20, 40, 40, 0.2), dense(160)),
        RigitarLayer("mingru", {"width": 72}, None),
        RigitarLayer("latent_attention", latent(2, 16, 8, 32, 24, 40, 0.25, kv_from=0), dense(104)),
        RigitarLayer("latent_attention", latent(1, 32, 16, 16, 48, 64, 0.15, base=500.0, dims=8), None),
        RigitarLayer("mingru", {"width": 130}, dense(56)),
    ]),
    # eight heads on one row (several passes of the attention kernel), a rotated part wider than the rest of the
    # query, two layers reading the same rows, recurrences first and last
    "heads8": RigitarConfig(vocab=300, width=128, norm_eps=1e-6, layers=[
        RigitarLayer("mingru", {"width": 128}, dense(192)),
        RigitarLayer("latent_attention", latent(8, 16, 32, 16, 64, 96, 0.14, base=40000.0), dense(256)),
        RigitarLayer("latent_attention", latent(8, 16, 32, 24, 32, 96, 0.14, base=40000.0, kv_from=1), None),
        RigitarLayer("latent_attention", latent(4, 48, 32, 8, 64, 96, 0.1, base=40000.0, kv_from=1), dense(64)),
        RigitarLayer("mingru", {"width": 40}, None),
    ]),
    # wide latents (the attention kernel's widest rows), no rotated part at all in one layer, nothing but attention
    "wide": RigitarConfig(vocab=97, width=64, norm_eps=1e-5, layers=[
        RigitarLayer("latent_attention", latent(2, 32, 64, 16, 32, 512, 0.12), dense(96)),
        RigitarLayer("latent_attention", latent(5, 8, 0, 8, 16, 272, 0.3, dims=0), None),
    ]),
    # sizes that are multiples of nothing: no vector access, no tensor-core projection fits
    "odd": RigitarConfig(vocab=77, width=100, norm_eps=2e-6, layers=[
        RigitarLayer("latent_attention", latent(3, 10, 6, 12, 20, 36, 0.3, base=300.0), dense(70)),
        RigitarLayer("mingru", {"width": 50}, dense(30)),
        RigitarLayer("latent_attention", latent(2, 14, 6, 9, 12, 36, 0.2, base=300.0, kv_from=0), None),
    ]),
    # one mechanism alone
    "only_latent": RigitarConfig(vocab=128, width=80, norm_eps=1e-6, layers=[
        RigitarLayer("latent_attention", latent(4, 32, 16, 24, 48, 80, 0.18), None)]),
    "only_mingru": RigitarConfig(vocab=128, width=80, norm_eps=1e-6, layers=[
        RigitarLayer("mingru", {"width": 96}, None)]),
    "only_ff": RigitarConfig(vocab=128, width=80, norm_eps=1e-6, layers=[
        RigitarLayer("mingru", {"width": 8}, dense(200))]),
}


def make_rigitar(name: str, folder: str, std: float = 0.08) -> str:
    """std 0.08: scores of order one, so that a wrong key, position or slot shows far above rounding."""
    return write_random_model(CONFIGS[name], folder, seed=4321 + sum(map(ord, name)), std=std, norm_std=0.1,
                              dtype=torch.bfloat16)
