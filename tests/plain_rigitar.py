"""A plain, slow implementation of the Rigitar decoder: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the package: config.json is read with ``json``, the weights with the
``safetensors`` library, and everything is plain torch arithmetic on the CPU.

Unlike the package's latent attention, which never forms a head's keys or values, this one expands them
(``k_h = Wuk_h c``, ``v_h = Wuv_h c``) and runs ordinary attention per head; the recurrence is a Python loop.
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


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def rotate(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [..., T, d]: feature i < dims / 2 is paired with i + dims / 2; features from dims on pass."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = positions.to(F)[:, None] * f[None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * a.cos() - v * a.sin(), v * a.cos() + u * a.sin(), x[..., dims:]], dim=-1)


def softmax_rows(s: torch.Tensor) -> torch.Tensor:
    e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


def latent_rows(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """What a layer caches per token: the normed latent and the rotated shared key part."""
    T, r = h.shape[0], m["kv_rank"]
    ckv = h @ w[p + "dkv"].T
    c = rms_norm(ckv[:, :r], w[p + "dkv.norm"], eps)
    kr = rotate(ckv[:, r:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, rows) -> torch.Tensor:
    """``rows``: (c, kr) of the layer whose rows this layer reads (its own, or another's)."""
    T, H, d, rd, vd = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = rows
    q = (rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps) @ w[p + "uq"].T).view(T, H, d + rd)
    gate = torch.sigmoid(h @ w[p + "g"].T)                       # [T, H]
    out = torch.zeros(T, H, vd, dtype=F)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hd in range(H):
        k_n = c @ w[p + "uk"][hd * d:(hd + 1) * d].T             # [T, d]
        v = c @ w[p + "uv"][hd * vd:(hd + 1) * vd].T             # [T, vd]
        q_n = q[:, hd, :d]
        q_r = rotate(q[:, hd, d:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
        s = (q_n @ k_n.T + q_r @ kr.T) * m["scale"]
        s = s.masked_fill(~causal, -math.inf)
        out[:, hd] = (softmax_rows(s) @ v) * gate[:, hd:hd + 1]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def mingru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = h @ w[p + "g"].T
    S = torch.zeros(z.shape[1], dtype=F)
    ys = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        ys.append(S * g[t] * torch.sigmoid(g[t]))
    return torch.stack(ys) @ w[p + "o"].T


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(x))


def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    pos = softplus(pq[0]) * z * z + z / 2
    neg = (0.5 + softplus(pq[1])) * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return xielu(h @ w[p + "up"].T, w[p + "act"]) @ w[p + "down"].T


class PlainRigitar:
    def __init__(self, model_dir: str):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_weights(model_dir)
        self.eps = self.cfg["norm"]["eps"]

    def residuals(self, ids: List[int]) -> List[torch.Tensor]:
        """The residual stream after the embedding and after every layer."""
        w, eps = self.w, self.eps
        x = w["embed"][torch.tensor(ids, dtype=torch.long)]
        out, rows = [x], {}
        for i, layer in enumerate(self.cfg["layers"]):
            p, m = f"l{i}.mix.", layer["mixer"]
            if layer["type"] == "mingru":
                y = mingru(x, w, p)
            else:
                src = m.get("kv_from")
                if src is None:
                    rows[i] = latent_rows(x, w, p, m, eps)
                y = latent_attention(x, w, p, m, eps, rows[i if src is None else src])
            x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
            if layer.get("mlp") is not None:
                x = x + rms_norm(dense_ff(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
            out.append(x)
        return out

    def logits(self, ids: List[int]) -> torch.Tensor:
        x = self.residuals(ids)[-1]
        return rms_norm(x, self.w["final.norm"], self.eps) @ self.w["head"].T

    def greedy(self, prompt: List[int], n: int) -> List[int]:
        ids, out = list(prompt), []
        for _ in range(n):
            tok = int(torch.argmax(self.logits(ids)[-1]))
            out.append(tok)
            ids.append(tok)
        return out
