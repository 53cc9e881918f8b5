"""Scale-factor layout oracle and psum-layout helpers (test infrastructure).

Restates:
  * the required scale-factor layout: tests/test_layout.py:39-58 (``reference``
    and ``check_layout``), csrc/apis/layout.hpp:19-36, and the byte order of a
    packed pair, deep_gemm/include/deep_gemm/transform_sf.hpp:276-279;
  * group-padding zeroing: tests/test_layout.py:61-63,91-97;
  * the psum layout: tests/generators.py:212-235,
    deep_gemm/include/deep_gemm/scheduler.hpp:17-23,147-162.

Required layout: int16 [..., MN, ceil(ceil(K/32)/2)], MN-major (stride(-2)==1,
stride(-1)==MN); each int16 packs the UE8M0 bytes of two consecutive 32-wide K
blocks, low byte = even block; an odd block count leaves the last high byte 0.
``gran_k = 128`` (an extension the reference rejects) repeats each scale over
the four 32-wide blocks it covers.
"""

from __future__ import annotations

import torch


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def align(a: int, b: int) -> int:
    return ceil_div(a, b) * b


def make_psum_layout(sizes: list[int], alignment: int = 256) -> tuple[int, list[int]]:
    """sizes per group -> (total rows incl. padding, psum list of END rows)."""
    psum, out = 0, []
    for s in sizes:
        out.append(psum + s)
        psum = align(psum + s, alignment)
    return psum, out


def psum_valid_spans(psum: list[int], alignment: int = 256):
    last = 0
    for p in psum:
        yield slice(last, p)
        last = align(p, alignment)


def psum_padding_spans(psum: list[int], alignment: int = 256, gran: int = 1):
    for p in psum:
        s0, s1 = ceil_div(p, gran), align(p, alignment) // gran
        if s0 < s1:
            yield slice(s0, s1)


def _ue8m0_bytes(sf: torch.Tensor) -> torch.Tensor:
    """fp32 -> exponent byte (bits >> 23) & 0xff."""
    return ((sf.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)


def required_sf_layout(sf: torch.Tensor, mn: int, k: int, gran_mn: int, gran_k: int = 32,
                       psum: list[int] | None = None, alignment: int = 256,
                       k_psum: list[int] | None = None) -> torch.Tensor:
    """Any accepted SF input -> the required int16 MN-major layout.

    ``sf`` is fp32 [..., ceil(MN/gran_mn), ceil(K/gran_k)] or int16
    [..., ceil(MN/gran_mn), ceil(K/(2*gran_k))] in any major. ``psum`` zeroes the
    padding rows of an m-grouped operand; ``k_psum`` zeroes the padding K units of
    a k-grouped operand (32-blocks of an fp32 source, whole packed columns of an
    int16 source: tests/test_layout.py:95-97)."""
    assert gran_k in (32, 128)
    if k_psum is not None:
        assert gran_k == 32 and psum is None
        sf = sf.clone()
        for span in psum_padding_spans(k_psum, alignment, 32 if sf.dtype == torch.float32 else 64):
            sf[..., span] = 0
    k32 = ceil_div(k, 32)
    if sf.dtype == torch.float32:
        b = _ue8m0_bytes(sf)
    else:
        assert sf.dtype == torch.int16
        b = sf.contiguous().view(torch.uint8)           # [..., rows, 2*cols], low byte first
    if gran_k == 128:
        b = b.repeat_interleave(4, dim=-1)
    # Keep exactly the blocks that exist, then pad to an even count with 0.
    if b.shape[-1] >= k32:
        b = b[..., :k32]
    if psum is not None:
        b = b.clone()
        for span in psum_padding_spans(psum, alignment, gran_mn):
            b[..., span, :] = 0
    if int16_pad := (b.shape[-1] % 2):
        b = torch.nn.functional.pad(b, (0, int16_pad))
    packed = b.contiguous().view(torch.int16)            # [..., rows, ceil(k32/2)]
    if sf.dtype == torch.int16 and gran_k == 32:
        # int16 input keeps whatever its last high byte holds (tests/test_layout.py:39-50).
        src = sf
        if psum is not None:
            src = sf.clone()
            for span in psum_padding_spans(psum, alignment, gran_mn):
                src[..., span, :] = 0
        packed = src
    out = packed.transpose(-2, -1).repeat_interleave(gran_mn, -1)[..., :mn]
    return out.contiguous().transpose(-2, -1)


def unpack_required_sf(sf16: torch.Tensor, k: int) -> torch.Tensor:
    """Required-layout int16 [..., MN, K64] -> fp32 scales [..., MN, ceil(K/32)]."""
    b = sf16.contiguous().view(torch.uint8)              # [..., MN, 2*K64]
    b = b[..., :ceil_div(k, 32)]
    return (b.to(torch.int32) << 23).view(torch.float32)
