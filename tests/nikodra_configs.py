"""Small Nikodra configurations for the tests, different in every size and option, with random weights."""
from __future__ import annotations

import os

import torch
from safetensors import safe_open

from exl3_server_b200 import write_random_model
from exl3_server_b200.config.nikodra import NikodraConfig, NikodraLayer
from exl3_server_b200.weights.safetensors_io import write_safetensors


def attn(heads, kv_heads, dim, vdim, scale, base=10000.0, dims=None, scaling=None, v_mix=False):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot, "v_mix": v_mix}


def par(left, block, right_heads, dk, dv, decay, base=10000.0, dims=None):
    lo = {k: left[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale")}
    if block:
        lo["mask"] = {"size": block}
    return {"left": lo, "right": {"heads": right_heads, "dim": dk, "vdim": dv, "decay": list(decay),
                                  "rot": {"base": base, "dims": dk if dims is None else dims}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


BIGRAM = {"buckets": 97, "mul_prev": 31, "mul_cur": 7}

CONFIGS = {
    # every kind of layer; three layers that mix values with a layer between them that does not; values narrower and
    # wider than keys; part of a head rotated; stretched and plain frequency tables; two and three kv heads; blocks
    # of 50 positions (no multiple of a page); a layer without a feed-forward; a multiplier that is not 1/2
    "mixed": NikodraConfig(vocab=211, width=96, norm_eps=1e-5, residual_mult=0.7, bigram=BIGRAM, layers=[
        NikodraLayer("attention", attn(4, 2, 24, 16, 0.21, scaling=(4.0, 64, 16.0, 1.0), v_mix=True), dense(160)),
        NikodraLayer("wkv", {"heads": 3, "dim": 16, "decay_rank": 8}, None),
        NikodraLayer("attention", attn(6, 3, 16, 40, 0.3, base=500.0, dims=8), dense(64)),
        NikodraLayer("attention", attn(2, 2, 32, 16, 0.18, dims=16, scaling=(8.0, 32, 8.0, 2.0), v_mix=True), None),
        NikodraLayer("parallel", par(attn(6, 2, 16, 24, 0.25), 50, 3, 16, 24, (0.9, 0.97, 0.995), dims=8), dense(104)),
        NikodraLayer("attention", attn(4, 2, 16, 16, 0.25, base=100000.0, v_mix=True), dense(72)),
    ]),
    # sizes that are multiples of nothing: heads of 10 and 6 features, a width of 100, a state of 12 x 20
    "odd": NikodraConfig(vocab=77, width=100, norm_eps=2e-6, residual_mult=0.5, bigram={"buckets": 13, "mul_prev": 5, "mul_cur": 3}, layers=[
        NikodraLayer("parallel", par(attn(3, 1, 10, 6, 0.3), 7, 2, 12, 20, (0.8, 0.99), base=300.0), dense(70)),
        NikodraLayer("wkv", {"heads": 2, "dim": 14, "decay_rank": 5}, dense(30)),
        NikodraLayer("attention", attn(5, 5, 10, 12, 0.3, base=300.0, dims=6, v_mix=True), None),
    ]),
    # heads of 64 and 128, a state of 64 x 128, blocks of exactly two pages, long decays
    "wide": NikodraConfig(vocab=300, width=128, norm_eps=1e-6, residual_mult=1.0, bigram=BIGRAM, layers=[
        NikodraLayer("attention", attn(4, 2, 64, 128, 0.125, base=250000.0, scaling=(2.0, 256, 24.0, 2.0), v_mix=True), dense(320)),
        NikodraLayer("parallel", par(attn(2, 1, 128, 64, 0.09), 128, 2, 64, 128, (0.95, 0.998), base=250000.0), None),
        NikodraLayer("wkv", {"heads": 2, "dim": 64, "decay_rank": 16}, dense(192)),
        NikodraLayer("attention", attn(8, 2, 64, 128, 0.125, v_mix=True), None),
    ]),
    # keys and values of 64 and of 128 features: the sizes of the tensor-core attention kernels, with the sink, blocks of
    # 100 positions (edges inside pages), eight query heads on a kv head, part of a head rotated, mixed values
    "tensor": NikodraConfig(vocab=200, width=128, norm_eps=1e-6, residual_mult=0.5, bigram=BIGRAM, layers=[
        NikodraLayer("attention", attn(4, 2, 64, 64, 0.125, dims=32, scaling=(4.0, 256, 32.0, 1.0), v_mix=True), dense(128)),
        NikodraLayer("parallel", par(attn(4, 2, 128, 128, 0.09), 100, 2, 32, 32, (0.9, 0.99)), None),
        NikodraLayer("attention", attn(8, 1, 128, 128, 0.09, base=800000.0), None),
        NikodraLayer("attention", attn(6, 2, 64, 64, 0.125, v_mix=True), dense(96)),
    ]),
    # one mechanism alone
    "only_attention": NikodraConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, bigram=None, layers=[
        NikodraLayer("attention", attn(4, 2, 32, 24, 0.18, scaling=(4.0, 128, 32.0, 1.0)), None)]),
    "only_parallel": NikodraConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, bigram=None, layers=[
        NikodraLayer("parallel", par(attn(4, 4, 16, 16, 0.25), 70, 4, 16, 32, (0.5, 0.9, 0.99, 0.999)), None)]),
    "only_attention_64": NikodraConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, bigram=None, layers=[
        NikodraLayer("attention", attn(4, 2, 64, 64, 0.09, dims=32, scaling=(4.0, 128, 32.0, 1.0)), None)]),
    "only_parallel_64": NikodraConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, bigram=None, layers=[
        NikodraLayer("parallel", par(attn(4, 2, 64, 64, 0.09), 70, 2, 16, 16, (0.9, 0.99)), None)]),
    "only_wkv": NikodraConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, bigram=None, layers=[
        NikodraLayer("wkv", {"heads": 4, "dim": 24}, None)]),
    "only_embedding": NikodraConfig(vocab=128, width=80, norm_eps=1e-6, residual_mult=0.5, bigram=BIGRAM, layers=[
        NikodraLayer("wkv", {"heads": 1, "dim": 8}, dense(200))]),
}


def make_nikodra(name: str, folder: str, std: float = 0.08) -> str:
    """std 0.08: scores of order one, so that a wrong key, position or slot shows far above rounding.  The scalars
    that weigh another layer's values are set to 0.2 to 0.6 (random ones would be near zero and hide the mixing),
    and the decay offsets are spread over -3 .. 1 so that the recurrence forgets at every rate."""
    write_random_model(CONFIGS[name], folder, seed=977 + sum(map(ord, name)), std=std, norm_std=0.1,
                       dtype=torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    with safe_open(path, framework="pt") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    g = torch.Generator().manual_seed(5)
    for k in sorted(tensors):
        if k.endswith(".vmix"):
            tensors[k] = (0.2 + 0.4 * torch.rand((), generator=g)).to(torch.bfloat16)
        elif k.endswith(".mix.w0"):
            tensors[k] = (-3.0 + 4.0 * torch.rand(tensors[k].shape, generator=g)).to(torch.bfloat16)
        elif ".mix.mu." in k:
            tensors[k] = torch.rand(tensors[k].shape, generator=g).to(torch.bfloat16)
        elif k.endswith(".mix.u"):
            tensors[k] = (tensors[k].float() * 5.0).to(torch.bfloat16)
    write_safetensors(path, tensors.items(), metadata={"format": "pt"})
    return folder
