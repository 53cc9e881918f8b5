"""CPU restatement of the SwiGLU / cast -> FP8 producer (test infrastructure, never shipped).

Follows third-party/tilelang_ops/swiglu_apply_weight_to_fp8.py of the reference: clamp (:156-161), SiLU by division
(:162-165), weight (:166), per-32-channel scale from the bit pattern of max(amax, 1e-4) * (1 / 448) rounded up to a
power of two (:80-90), value times the inverse scale rounded to E4M3 (:250-252), scale bytes packed two per int16
with consecutive tokens contiguous (:104-125, 446-449), tokens in psum padding skipped (:263-268).

Parity unpinned by the reference for this function: the reference's own test of the operator (tests/test_mega_moe.py)
needs the NPU kernel itself as ground truth and holds no fixture, so this restatement is checked against the formulas
above only. The GPU test compares with a tolerance because exp() differs in the last bit between implementations.
"""

from __future__ import annotations

import torch


def swiglu_quant_ref(x: torch.Tensor, topk_weights=None, psum=None, clamp_value=None, alignment: int = 128,
                     swiglu: bool = True):
    """Returns (codes uint8 [T, H], sf int16 [T, ceil(H/64)], valid bool [T], dequantised fp32 [T, H])."""
    t = x.size(0)
    xf = x.float()
    if swiglu:
        h = x.size(1) // 2
        xl, xr = xf[:, :h], xf[:, h:]
        if clamp_value is not None:
            xl = torch.clamp(xl, max=clamp_value)
            xr = torch.clamp(xr, min=-clamp_value, max=clamp_value)
        y = xl / (1.0 + torch.exp(-xl)) * xr
        if topk_weights is not None:
            y = y * topk_weights.float().reshape(-1, 1)
    else:
        h = x.size(1)
        y = xf
    groups = h // 32
    amax = y.reshape(t, groups, 32).abs().amax(dim=-1)
    scaled = (torch.clamp(amax, min=1e-4) * torch.tensor(1.0 / 448.0, dtype=torch.float32)).contiguous()
    bits = scaled.view(torch.int32)
    exponent = ((bits - 1) >> 23) + 1                                   # UE8M0 byte
    inverse = ((254 - exponent) << 23).view(torch.float32)
    q = (y.reshape(t, groups, 32) * inverse.unsqueeze(-1)).reshape(t, h).to(torch.float8_e4m3fn)
    scale = (exponent << 23).view(torch.float32)
    deq = (q.float().reshape(t, groups, 32) * scale.unsqueeze(-1)).reshape(t, h)
    e8 = exponent.to(torch.uint8)
    if groups % 2:
        e8 = torch.nn.functional.pad(e8, (0, 1))
    sf = e8.contiguous().view(torch.int16)                                # low byte = even 32-block
    valid = torch.ones(t, dtype=torch.bool)
    if psum is not None:
        valid[:] = False
        start = 0
        for p in psum:
            valid[start:min(int(p), t)] = True
            start = (int(p) + alignment - 1) // alignment * alignment
    return q.view(torch.uint8), sf, valid, deq
