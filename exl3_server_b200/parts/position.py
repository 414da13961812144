"""Position encodings applied to queries and keys.

``rope``: half-split rotary embedding over the first ``dims`` features of each
head: for d < dims/2, ``f_d = theta^(-2d/dims)``, angle ``a = pos * scale * f_d``,
``x'[d] = x[d] cos a - x[d + dims/2] sin a``,
``x'[d + dims/2] = x[d + dims/2] cos a + x[d] sin a`` — the reference's
``mx::fast::rope(x, hd, traditional=false, theta, 1.0, offset)``
(src/model.cpp:566-567).  The frequency table (times ``scale``) is computed once in float64
and kept as two float32 rows, the rounded frequencies and what the rounding lost
(``kernels.rotary_table``): the kernels' float32 angles then stay right at large positions,
where ``pos * f`` with a rounded ``f`` is off by ``pos * 6e-8`` radians.  A scaled or extended
variant only needs another table.

Parameters of a ``rope`` spec (``PositionSpec.params``), for mixers that apply the encoding through
``kernels.qk_prep`` (``table``, ``layout_code``, ``mscale``):

* ``layout``: ``"half"`` (feature d with d + dims/2, the default) or ``"interleaved"`` (feature 2d with 2d + 1);
* ``yarn``: ``{"factor", "original", "fast", "slow"}``, a frequency table stretched for contexts beyond
  ``original`` positions: with ``n(t) = dims ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(n(fast)), 0)``,
  ``hi = min(ceil(n(slow)), dims - 1)`` and ``ramp_d = clamp((d - lo) / max(hi - lo, 0.001), 0, 1)``, the frequency is
  ``f_d / factor * ramp_d + f_d (1 - ramp_d)``, and sines and cosines are multiplied by ``0.1 ln(factor) + 1``.

The Llama-family kernels (``rotate_and_store``, ``fused_rotation``) know the half layout without that factor only.

``none``: no rotation; keys and values are still written to the cache.

A position part has ``rotate_and_store(qkv, batch, kv, heads, kv_heads, head_dim)``; it may also offer
``fused_rotation(head_dim)`` (see below), which lets the decode attention kernel do both jobs itself.
"""
from __future__ import annotations

import math

import torch

from ..ops import kernels as K
from .base import BuildContext
from .registry import register_position
from .spec import PositionSpec


class RotaryPosition:
    def __init__(self, spec: PositionSpec, head_dim: int, ctx: BuildContext):
        if spec.dims % 2 != 0 or not 0 <= spec.dims <= head_dim:
            raise ValueError(f"rope: dims {spec.dims} must be even and at most head_dim {head_dim}")
        self.spec = spec
        layout = spec.params.get("layout", "half")
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rope: layout must be 'half' or 'interleaved', got {layout!r}")
        self.layout_code = 1 if layout == "interleaved" else 0
        yarn = spec.params.get("yarn")
        self.mscale = 0.1 * math.log(float(yarn["factor"])) + 1.0 if yarn else 1.0
        self.plain = self.layout_code == 0 and self.mscale == 1.0       # what the Llama-family kernels apply
        self.inv_freq = K.rotary_table(self.frequencies(spec) * float(spec.scale)).to(ctx.device)

    @staticmethod
    def frequencies(spec: PositionSpec) -> torch.Tensor:
        """float64 ``theta^(-2d/dims)`` for d < dims / 2, stretched when the spec has ``yarn`` parameters."""
        d = torch.arange(0, spec.dims // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * d / max(1, spec.dims))
        yarn = spec.params.get("yarn")
        if yarn and spec.dims:
            factor, original = float(yarn["factor"]), float(yarn["original"])

            def turns(t: float) -> float:
                return spec.dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(float(spec.theta)))

            lo = max(math.floor(turns(float(yarn["fast"]))), 0)
            hi = min(math.ceil(turns(float(yarn["slow"]))), spec.dims - 1)
            ramp = torch.clamp((d - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
        return f

    @property
    def table(self) -> torch.Tensor:
        """The frequency table as ``kernels.rotary_table`` lays it out."""
        return self.inv_freq

    def rotate_and_store(self, qkv: torch.Tensor, batch, kv, heads: int, kv_heads: int, head_dim: int) -> None:
        if not self.plain:
            raise ValueError("rope: this kernel applies the half layout without a factor on sines and cosines")
        write = kv is not None and kv.owns
        K.rope_kv_write(qkv, self.inv_freq, self.spec.dims, 1.0, batch.tok_pos,
                        batch.tok_seq, kv.block_table, kv.k if write else None, kv.v if write else None,
                        heads, kv_heads, head_dim, kv.page_size, write)


    def fused_rotation(self, head_dim: int):
        """``(frequency table, dims, position scale)`` when an attention kernel can apply this encoding itself (all of a head's
        features rotated, or none), else None: then ``rotate_and_store`` runs as a step of its own."""
        if self.spec.dims == 0:
            return None, 0, 1.0
        if not self.plain:
            return None
        if self.spec.dims == head_dim:
            return self.inv_freq, self.spec.dims, 1.0                # the scale is in the table
        return None


class NoPosition(RotaryPosition):
    def __init__(self, spec: PositionSpec, head_dim: int, ctx: BuildContext):
        super().__init__(PositionSpec(kind="none", dims=0), head_dim, ctx)


register_position("rope", RotaryPosition)
register_position("none", NoPosition)
