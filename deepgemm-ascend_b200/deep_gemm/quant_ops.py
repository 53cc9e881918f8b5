"""Producers of block-scaled FP8 operands whose scale factors come out in the layout the GEMM reads.

`swiglu_apply_weight_to_fp8` mirrors the reference's third-party/tilelang_ops/swiglu_apply_weight_to_fp8.py:411-449
(same arguments, same return pair); `cast_to_fp8` is the same kernel without the SwiGLU step and has no counterpart in
the reference. Both return `(out, out_sf)` with `out` E4M3 [tokens, hidden] and `out_sf` int16 [tokens, hidden / 64]
whose stride(0) == 1: pass them to `fp8_gemm_*` / `m_grouped_fp8_gemm_*` as `(out, out_sf)` with `recipe_a=(1, 32)`
and no scale-factor transform runs.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib as L
from ._api import _host_assert, _stream_ptr


def _launch(x, hidden, swiglu, topk_weights, psum, clamp_value, expert_alignment):
    tokens = x.size(0)
    out = torch.empty((tokens, hidden), dtype=torch.float8_e4m3fn, device=x.device)
    cols = (hidden // 32 + 1) // 2
    storage = torch.empty((cols, tokens), dtype=torch.int16, device=x.device)
    if tokens:
        if topk_weights is not None:
            _host_assert(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous() and topk_weights.numel() == tokens,
                         'topk_weights must be a contiguous float32 tensor with one weight per token')
        if psum is not None:
            _host_assert(psum.dtype == torch.int32 and psum.dim() == 1 and psum.is_contiguous() and psum.device == x.device,
                         'psum_num_tokens_per_expert must be a contiguous int32 vector on the device of x')
        L.check(L.lib().dg_quant_fp8_launch(
            x.data_ptr(), x.stride(0), tokens, hidden, int(swiglu),
            topk_weights.data_ptr() if topk_weights is not None else None,
            psum.data_ptr() if psum is not None else None, psum.numel() if psum is not None else 0, int(expert_alignment),
            int(clamp_value is not None), float(clamp_value or 0.0), out.data_ptr(), out.stride(0),
            storage.data_ptr(), tokens, _stream_ptr(x.device)))
    return out, storage.T


def swiglu_apply_weight_to_fp8(x: torch.Tensor, topk_weights: Optional[torch.Tensor] = None,
                               psum_num_tokens_per_expert: Optional[torch.Tensor] = None,
                               clamp_value: Optional[float] = None, expert_alignment: int = 128):
    """x [tokens, 2 * hidden] BF16 -> (E4M3 [tokens, hidden], packed UE8M0 scales) of
    silu(min(x_l, clamp)) * clamp(x_r, -clamp, clamp) * weight. Rows in the padding of the psum layout are not written."""
    _host_assert(x.dim() == 2 and x.is_contiguous() and x.dtype == torch.bfloat16, 'x must be a contiguous 2-D BF16 tensor')
    _host_assert(x.size(1) % 256 == 0, 'the row length of x must be a multiple of 256')
    return _launch(x, x.size(1) // 2, True, topk_weights, psum_num_tokens_per_expert, clamp_value, expert_alignment)


def cast_to_fp8(x: torch.Tensor, psum_num_tokens_per_expert: Optional[torch.Tensor] = None, expert_alignment: int = 128):
    """x [tokens, hidden] BF16 -> (E4M3 [tokens, hidden], packed UE8M0 scales per 1x32)."""
    _host_assert(x.dim() == 2 and x.stride(1) == 1 and x.dtype == torch.bfloat16, 'x must be a row-major 2-D BF16 tensor')
    _host_assert(x.size(1) % 32 == 0, 'the row length of x must be a multiple of 32')
    return _launch(x, x.size(1), False, None, psum_num_tokens_per_expert, None, expert_alignment)
