"""The latent attention mixer: queries and keys/values through low-rank latents, one cached row per token.

With ``H`` heads of ``dim`` unrotated and ``rot_dim`` rotated query/key features, values of ``vdim`` and latents of
``q_rank`` and ``kv_rank`` features (``params`` of the spec):

    c_q = rmsnorm(x Wdq^T) * w_dq                     q = c_q Wuq^T, per head [ q^n (dim) | q^r (rot_dim) ]
    [c' | k'] = x Wdkv^T                              c = rmsnorm(c') * w_dkv,   k^r = rope(k')  (shared by all heads)
    k^n_h = Wuk_h c,  v_h = Wuv_h c
    s_h(i, j) = (q^n_h(i) . k^n_h(j) + rope(q^r_h(i)) . k^r(j)) * scale,   j <= i,   softmax over j
    y = concat_h( sigmoid(x wg_h) * sum_j p_h(i, j) v_h(j) ) Wo^T

The cache keeps ``[c | k^r]`` per token and nothing per head.  The per-head keys and values are never formed: the
query is carried into the latent space (``q^n_h Wuk_h``, a product per head), attention runs over the cached rows
as keys whose leading ``kv_rank`` features are also the values, and ``Wuv_h`` is applied to what comes out.  That
is the same arithmetic for prompts, portions of prompts and single tokens, so their results differ by rounding only.

A layer with ``kv_from`` has no ``dkv`` projection: it reads the rows that an earlier layer of the same latent
shape wrote (the plan's ``cache_from``) through its own ``uk`` and ``uv``.

The three projections of the input (``dq``, ``dkv``, ``g``) are one matrix; both norms, the rotation of the shared key
part, the cache write and the gate are one kernel (``csrc/latent.cu``); the rotation of the queries rides on the
kernel that carries them into the latent space.  Norms, angles, scores, softmax and gates are float32.

Tensor names under the mixer's prefix: ``dq``, ``dq.norm``, ``uq``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``g``, ``o``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, KVRequest, StateRequest
from .linear import Linear
from .position import RotaryPosition
from .registry import register_mixer
from .spec import MixerSpec, PositionSpec

# Keys per work item of the CUDA-core attention kernel; a multiple of the cache's page size.
SPLIT_KEYS = 256
# Tokens in a step beyond which the bfloat16 products per head (queries into the latent space, values out of it) are
# the library's batched product; up to here this library's kernel, which reads the weights once.
MANY_ROWS = 64


def _up16(n: int) -> int:
    return (n + 15) // 16 * 16


class LatentAttention:
    @staticmethod
    def _sizes(spec: MixerSpec):
        p = spec.params
        try:
            sizes = {k: int(p[k]) for k in ("dim", "rot_dim", "vdim", "q_rank", "kv_rank")}
        except KeyError as e:
            raise ValueError(f"latent attention: the spec's params lack {e.args[0]!r}") from None
        if min(sizes["dim"], sizes["vdim"], sizes["q_rank"], sizes["kv_rank"]) < 1 or sizes["rot_dim"] < 0 or spec.heads < 1:
            raise ValueError(f"latent attention: sizes must be positive, got {sizes} with {spec.heads} heads")
        return sizes

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        z = cls._sizes(spec)
        H = spec.heads
        out = [
            TensorSpec(prefix + "dq", (z["q_rank"], spec.width)),
            TensorSpec(prefix + "dq.norm", (z["q_rank"],), init="ones"),
            TensorSpec(prefix + "uq", (H * (z["dim"] + z["rot_dim"]), z["q_rank"])),
            TensorSpec(prefix + "uk", (H * z["dim"], z["kv_rank"])),
            TensorSpec(prefix + "uv", (H * z["vdim"], z["kv_rank"])),
            TensorSpec(prefix + "g", (H, spec.width)),
            TensorSpec(prefix + "o", (spec.width, H * z["vdim"])),
        ]
        if not spec.params.get("shared_rows", False):
            out += [TensorSpec(prefix + "dkv", (z["kv_rank"] + z["rot_dim"], spec.width)),
                    TensorSpec(prefix + "dkv.norm", (z["kv_rank"],), init="ones")]
        return out

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        z = self._sizes(spec)
        self.spec, self.ctx = spec, ctx
        self.H = H = spec.heads
        self.dim, self.rot_dim, self.vdim = z["dim"], z["rot_dim"], z["vdim"]
        self.q_rank, self.kv_rank = z["q_rank"], z["kv_rank"]
        self.owner = not spec.params.get("shared_rows", False)
        self.eps = float(spec.params["norm_eps"])
        # a cached row: [c | zeros to a multiple of 16 | k^r | zeros to a multiple of 16]
        self.rank_pad = _up16(self.kv_rank)
        self.row = _up16(self.rank_pad + self.rot_dim)
        pos = spec.position or PositionSpec(kind="rope", dims=0)
        if pos.dims % 2 != 0 or not 0 <= pos.dims <= self.rot_dim:
            raise ValueError(f"latent attention: {pos.dims} rotated features must be even and at most rot_dim {self.rot_dim}")
        self.rot = pos.dims
        self.inv_freq = (K.rotary_table(RotaryPosition.frequencies(pos) * float(pos.scale)).to(ctx.device)
                         if self.rot > 0 else None)
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else (self.dim + self.rot_dim) ** -0.5
        # the joint input projection: [dq | dkv (owners) | g], rows padded to a multiple of 16
        names = ["dq"] + (["dkv"] if self.owner else []) + ["g"]
        w = torch.cat([tensors[prefix + n].to(ctx.dtype) for n in names], dim=0)
        self.q_off, self.kv_off = 0, self.q_rank
        self.g_off = self.q_rank + (self.kv_rank + self.rot_dim if self.owner else 0)
        pad = _up16(w.shape[0]) - w.shape[0]
        if pad:
            w = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0)
        self.inp = Linear(w, None, ctx.dtype)
        self.w_dq_norm = tensors[prefix + "dq.norm"].contiguous()
        self.w_dkv_norm = tensors[prefix + "dkv.norm"].contiguous() if self.owner else None
        self.uq = Linear(tensors[prefix + "uq"], None, ctx.dtype)
        # per head: [dim, kv_rank] as stored (a head's rows of uk), and uv turned to [kv_rank, vdim]
        self.w_uk = tensors[prefix + "uk"].to(ctx.dtype).view(H, self.dim, self.kv_rank).contiguous()
        self.w_uv = tensors[prefix + "uv"].to(ctx.dtype).view(H, self.vdim, self.kv_rank).transpose(1, 2).contiguous()
        self.o = Linear(tensors[prefix + "o"], None, ctx.dtype)

    def cache_request(self) -> Optional[KVRequest]:
        return KVRequest(kv_heads=1, head_dim=self.row, window=0, value_dim=0, values_in_keys=True)

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if kv is None:
            raise RuntimeError("latent attention needs a cache view")
        if kv.owns != self.owner:
            raise RuntimeError("latent attention: the plan's cache_from and the layer's own rows disagree")
        T, H, dt = x.shape[0], self.H, self.ctx.dtype
        a = self.inp(x, out_dtype=self.inp.wide_dtype(T))
        cq, gate = K.latent_prep(a, self.q_off, self.q_rank, self.w_dq_norm, self.kv_off, self.kv_rank, self.rot_dim,
                                 self.w_dkv_norm, self.g_off, H, self.eps, self.inv_freq, self.rot, batch.tok_pos,
                                 batch.tok_seq, kv.block_table, kv.page_size, kv.k if self.owner else None, self.row,
                                 self.rank_pad, dt)
        q = self.uq(cq)                                                   # [T, H * (dim + rot_dim)]
        hq = self.dim + self.rot_dim
        many = dt == torch.bfloat16 and T > MANY_ROWS                     # the per-head products go to the library
        ql = torch.empty((T, H * self.row), dtype=dt, device=x.device)    # per head [q^n Wuk | 0 | rope(q^r) | 0]
        K.head_gemm(q, H * hq, hq, None if many else self.w_uk, ql, H * self.row, self.row, T, H, self.dim,
                    self.kv_rank, rot_dim=self.rot_dim, rot=self.rot, inv_freq=self.inv_freq, tok_pos=batch.tok_pos,
                    tail_off=self.rank_pad)
        if many:
            # a product per head, written where the head's row of ql has its place (a strided view: no copy afterwards)
            torch.bmm(q.view(T, H, hq)[:, :, :self.dim].transpose(0, 1), self.w_uk,
                      out=ql.view(T, H, self.row)[:, :, :self.kv_rank].transpose(0, 1))
        ol = torch.empty((T, H * self.rank_pad), dtype=dt, device=x.device)
        gated = self.attend(ql, ol, batch, kv, gate)
        o = torch.empty((T, H * self.vdim), dtype=dt, device=x.device)
        if many:
            torch.bmm(ol.view(T, H, self.rank_pad)[:, :, :self.kv_rank].transpose(0, 1), self.w_uv,
                      out=o.view(T, H, self.vdim).transpose(0, 1))
            if not gated:
                o = (o.view(T, H, self.vdim) * gate[:, :, None]).to(dt).view(T, H * self.vdim)
        else:
            K.head_gemm(ol, H * self.rank_pad, self.rank_pad, self.w_uv, o, H * self.vdim, self.vdim, T, H,
                        self.kv_rank, self.vdim, mul=None if gated else gate)
        return self.o(o, out_dtype=self.o.wide_dtype(T))

    def attend(self, ql: torch.Tensor, ol: torch.Tensor, batch, kv, gate: torch.Tensor) -> bool:
        """Attention of the step's tokens over the cached rows: ``H`` query heads on one row per key.  Returns
        whether the gate is already in ``ol`` (a factor per (token, head) commutes with the head's value projection,
        and the tensor-core kernel applies it as it writes)."""
        T = ql.shape[0]
        if K.attn_latent_supported(ql.dtype, self.row, self.rank_pad, kv.page_size):
            # bfloat16: both products on the tensor cores, a block per tile of a sequence's (token, head) rows
            per, n = self._chunks(batch, kv.page_size, ql.device)
            scratch = None
            if n > 1:
                scratch = batch.workspace.plain(K.attn_latent_scratch_bytes(T, self.H, self.rank_pad, n) // 4)
            K.attn_latent(ql, ol, kv.k, kv.block_table, batch.row_start, batch.row_pos0, batch.n_rows, T, batch.max_new,
                          self.H, self.row, self.rank_pad, kv.page_size, self.scale, per, n, scratch, gate)
            return True
        split = max(SPLIT_KEYS, kv.page_size)
        if split % kv.page_size:
            split = kv.page_size * (split // kv.page_size + 1)
        n = max(1, (batch.max_kv_len + split - 1) // split)
        scratch = None
        if n > 1:
            scratch = batch.workspace.floats(K.attn_tokens_scratch_bytes(T, self.H, self.rank_pad, n) // 4)
        K.attn_tokens_kv(ql, ql.stride(0), ol, kv.k, kv.k, kv.block_table, batch.tok_pos, batch.tok_seq, T, self.H, 1,
                         self.row, self.rank_pad, self.row, kv.page_size, 0, self.scale, split, n, scratch)
        return False

    def _chunks(self, batch, page: int, device):
        """``(pages per chunk, chunks)`` for the tensor-core kernel: one chunk when the step's tiles of rows already
        give every SM a block (prompts, large batches); else the keys are cut into as many chunks of whole pages as
        it takes to get there, none shorter than two pages.  The choice depends on the step's size, not on a token's
        position: results differ between batch sizes by rounding."""
        pages = max(1, (batch.max_kv_len + page - 1) // page)
        tile = K.attn_latent_row_tile(self.row, batch.max_new * self.H)
        blocks = batch.n_rows * ((batch.max_new * self.H + tile - 1) // tile)
        want = max(1, K.sm_count(device) // max(1, blocks))
        n = max(1, min(want, pages // 2))
        per = (pages + n - 1) // n
        return per, (pages + per - 1) // per

    def weight_bytes(self) -> int:
        own = sum(t.numel() * t.element_size() for t in (self.w_uk, self.w_uv))
        return self.inp.weight_bytes() + self.uq.weight_bytes() + self.o.weight_bytes() + own


register_mixer("latent_attention", LatentAttention)
