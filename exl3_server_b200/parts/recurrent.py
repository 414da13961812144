"""Recurrent mixers: a state of fixed size per sequence instead of keys and values.

``mingru``: a gated recurrence whose gates read only the current token.  With
``a = x Wz^T + bz``, ``u = x Wx^T + bx`` and ``g = x Wg^T`` (``width`` features each):

    z_t = sigmoid(a_t)
    c_t = u_t + 1/2 where u_t >= 0, sigmoid(u_t) where u_t < 0
    S_t = (1 - z_t) S_(t-1) + z_t c_t                (element by element)
    y_t = (S_t * silu(g_t)) Wo^T

The state starts at zero (the cache zeroes a slot's row when it is opened), is
float32 and is carried from step to step in the cache's per-sequence state, so a
prompt cut into steps in any way, and token-by-token decoding, walk the same
chain of sums (rows of many tokens are cut into chunks that run side by side and
are joined through the recurrence's linearity, which changes roundings only).  The three input projections are one matrix; the gates, the
candidate and the recurrence are float32 (``csrc/recurrent.cu``).

Tensor names under the mixer's prefix: ``z``, ``z.b``, ``x``, ``x.b``, ``g``, ``o``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import kernels as K
from ..weights.loader import TensorSpec
from .base import BuildContext, KVRequest, StateRequest
from .linear import Linear
from .registry import register_mixer
from .spec import MixerSpec


class MinGRU:
    @staticmethod
    def _inner(spec: MixerSpec) -> int:
        n = int(spec.params.get("inner", 0))
        if n < 1:
            raise ValueError("mingru: the spec's params must give 'inner', the width of the recurrence")
        return n

    @classmethod
    def tensor_specs(cls, spec: MixerSpec, prefix: str) -> List[TensorSpec]:
        n = cls._inner(spec)
        return [
            TensorSpec(prefix + "z", (n, spec.width)), TensorSpec(prefix + "z.b", (n,), init="zeros"),
            TensorSpec(prefix + "x", (n, spec.width)), TensorSpec(prefix + "x.b", (n,), init="zeros"),
            TensorSpec(prefix + "g", (n, spec.width)),
            TensorSpec(prefix + "o", (spec.width, n)),
        ]

    def __init__(self, spec: MixerSpec, tensors: Dict[str, torch.Tensor], prefix: str, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        self.inner = self._inner(spec)
        w = torch.cat([tensors[prefix + n].to(ctx.dtype) for n in ("z", "x", "g")], dim=0)
        b = torch.cat([tensors[prefix + "z.b"].to(ctx.dtype), tensors[prefix + "x.b"].to(ctx.dtype),
                       torch.zeros(self.inner, dtype=ctx.dtype, device=w.device)])
        self.zug = Linear(w, b, ctx.dtype)
        self.o = Linear(tensors[prefix + "o"], None, ctx.dtype)

    def cache_request(self) -> Optional[KVRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.inner,), torch.float32)

    def forward(self, x: torch.Tensor, batch, kv, state) -> torch.Tensor:
        if state is None:
            raise RuntimeError("mingru needs its per-sequence state")
        zug = self.zug(x, out_dtype=self.zug.wide_dtype(x.shape[0]))
        need = K.mingru_scratch_bytes(batch.n_rows, x.shape[0], self.inner, batch.max_new)
        scratch = batch.workspace.plain(need // 4) if need else None      # prompts: chunks side by side
        y = K.mingru_scan(zug, state, batch.slot_ids, batch.row_start, batch.n_rows, self.inner, batch.max_new,
                          self.ctx.dtype, scratch)
        return self.o(y, out_dtype=self.o.wide_dtype(x.shape[0]))

    def weight_bytes(self) -> int:
        return self.zug.weight_bytes() + self.o.weight_bytes()


register_mixer("mingru", MinGRU)
