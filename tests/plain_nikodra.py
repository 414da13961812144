"""A plain, slow implementation of the Nikodra decoder: whole sequences, no cache, no state carried between calls,
float64, one function per mechanism.  It shares no code with the package: config.json is read with ``json``, the
weights with the ``safetensors`` library, and everything is plain torch arithmetic on the CPU.  Attention builds the
full score matrix with its mask; the recurrences are Python loops over tokens.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch
from safetensors import safe_open

F = torch.float64


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(F)
    return out


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the stored weight lies around zero, the factor is 1 + w."""
    return unit_rms(x, eps) * (1.0 + w)


def pair_rows(tokens: List[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the second embedding table for every token: a hash of (token before, token); the last row first."""
    return [buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets for i, t in enumerate(tokens)]


def rotary_frequencies(rot: dict) -> (torch.Tensor, float):
    """Frequencies of the dims/2 pairs and the factor on sines and cosines (1 without ``scaling``)."""
    dims, base = rot["dims"], rot["base"]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    turns = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(turns(sc["fast"])), 0), min(math.ceil(turns(sc["slow"])), dims - 1)
    ramp = torch.tensor([min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001))) for i in range(dims // 2)], dtype=F)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x: torch.Tensor, rot: dict, interleaved: bool) -> torch.Tensor:
    """x [T, heads, d] at positions 0 .. T-1: the first ``dims`` features rotated pair by pair, the rest as they are.
    Pairs are (2i, 2i + 1) when ``interleaved``, else (i, i + dims / 2)."""
    dims = rot["dims"]
    if dims == 0:
        return x
    f, factor = rotary_frequencies(rot)
    a = torch.arange(x.shape[0], dtype=F)[:, None] * f[None, :]
    c, s = (a.cos() * factor)[:, None, :], (a.sin() * factor)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = u * c - v * s, v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = u * c - v * s, v * c + u * s
    return out


def sink_softmax(s: torch.Tensor) -> torch.Tensor:
    """Rows of exp(s) / (1 + sum exp(s)); masked places hold -inf."""
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(dim=-1, keepdim=True))


def grouped_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, block: int) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv]; causal, inside blocks of ``block`` positions when > 0."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    i = torch.arange(T)
    seen = i[:, None] >= i[None, :]
    if block > 0:
        seen = seen & ((i[:, None] // block) == (i[None, :] // block))
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T * scale).masked_fill(~seen, -math.inf)
        heads.append(sink_softmax(s) @ v[:, g])
    return torch.cat(heads, dim=-1)


def attention_mixer(h, w, p, m, eps, first_values):
    """Returns (output, values as computed here before mixing)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q = rotate(unit_rms(q, eps) * w[p + "q.norm"], m["rot"], True)
    k = rotate(unit_rms(k, eps) * w[p + "k.norm"], m["rot"], True)
    own = v
    if first_values is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * first_values
    return grouped_attention(q, k, v, m["scale"], 0) @ w[p + "o"].T + w[p + "o.b"], own


def retention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: List[float]) -> torch.Tensor:
    """q, k [T, H, dk], v [T, H, dv] -> o [T, H, dv]: S = decay S + k v^T, o = S^T q, token by token."""
    T, H, dv = v.shape
    o = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(q.shape[2], dv, dtype=F)
        for t in range(T):
            S = decay[hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    return o


def parallel_mixer(h, w, p, m, eps):
    T = h.shape[0]
    a = m["left"]
    H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    q = unit_rms((h @ w[p + "left.q"].T).view(T, H, d), eps)
    k = unit_rms((h @ w[p + "left.k"].T).view(T, G, d), eps)
    v = (h @ w[p + "left.v"].T).view(T, G, dv)
    left = grouped_attention(q, k, v, a["scale"], a["mask"]["size"] if a.get("mask") else 0) @ w[p + "left.o"].T
    b = m["right"]
    H, d, dv = b["heads"], b["dim"], b["vdim"]
    q = rotate((h @ w[p + "right.q"].T).view(T, H, d), b["rot"], False)
    k = rotate((h @ w[p + "right.k"].T).view(T, H, d), b["rot"], False) * d ** -0.5
    o = unit_rms(retention(q, k, (h @ w[p + "right.v"].T).view(T, H, dv), b["decay"]), eps).reshape(T, H * dv)
    g = h @ w[p + "right.g"].T
    right = (o * g * torch.sigmoid(g)) @ w[p + "right.o"].T
    return 0.5 * (unit_rms(left, eps) * w[p + "left.out"] + unit_rms(right, eps) * w[p + "right.out"])


def wkv(r, k, v, decay, bonus):
    """r, k, v, decay [T, H, d], bonus [H, d] -> o [T, H, d]: o = (S + diag(u) k v^T)^T r, then S = diag(w) S + k v^T."""
    T, H, d = r.shape
    o = torch.zeros(T, H, d, dtype=F)
    for hd in range(H):
        S = torch.zeros(d, d, dtype=F)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S + bonus[hd][:, None] * kv).T @ r[t, hd]
            S = decay[t, hd][:, None] * S + kv
    return o


def wkv_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    before = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]])
    blend = {s: h + (before - h) * w[p + "mu." + s] for s in "rkvgw"}
    r, k, v = ((blend[s] @ w[p + s].T).view(T, H, d) for s in "rkv")
    g = blend["g"] @ w[p + "g"].T
    decay = torch.exp(-torch.exp(torch.tanh(blend["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    o = unit_rms(wkv(r, k, v, decay, w[p + "u"]), eps).reshape(T, H * d)
    return (o * w[p + "norm"] * g * torch.sigmoid(g)) @ w[p + "o"].T


def dense_gelu(h, w, p):
    z = h @ w[p + "up"].T
    return (0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))) @ w[p + "down"].T


class PlainNikodra:
    def __init__(self, model_dir: str):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_weights(model_dir)
        self.eps = self.cfg["norm"]["eps"]

    def residuals(self, tokens: List[int]) -> List[torch.Tensor]:
        """The residual stream after the embedding and after every layer."""
        cfg, w, eps = self.cfg, self.w, self.eps
        x = w["embed"][torch.tensor(tokens)]
        bg = (cfg.get("embedding") or {}).get("bigram")
        if bg:
            x = x + w["bigram"][torch.tensor(pair_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"]))]
        mult = cfg.get("residual_mult", 1.0)
        out = [x]
        first_values = None
        for i, layer in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = norm_around_zero(x, w[p + "norm1"], eps)
            if layer["type"] == "attention":
                mixes = bool(layer["mixer"].get("v_mix"))
                y, own = attention_mixer(h, w, p + "mix.", layer["mixer"], eps, first_values if mixes else None)
                if mixes and first_values is None:
                    first_values = own
            elif layer["type"] == "parallel":
                y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
            else:
                y = wkv_mixer(h, w, p + "mix.", layer["mixer"], eps)
            x = x + mult * norm_around_zero(y, w[p + "norm1b"], eps)
            if layer.get("mlp"):
                y = dense_gelu(norm_around_zero(x, w[p + "norm2"], eps), w, p + "mlp.")
                x = x + mult * norm_around_zero(y, w[p + "norm2b"], eps)
            out.append(x)
        return out

    def logits(self, tokens: List[int]) -> torch.Tensor:
        x = self.residuals(tokens)[-1]
        return norm_around_zero(x, self.w["final.norm"], self.eps) @ self.w["head"].T

    def greedy(self, prompt: List[int], n: int) -> List[int]:
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(torch.argmax(self.logits(toks)[-1])))
        return toks[len(prompt):]
