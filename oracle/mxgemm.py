"""Dequantise-then-matmul oracle (test infrastructure, never shipped).

Restates the ground truth used by the reference's tests:
  * value decode and scale application: tests/generators.py:98-121 (FP4 value
    table and ``_scale_quantized_reference``), :137-166 (uniform-code operands);
  * UE8M0 rounding of a float scale: tests/generators.py:27-31;
  * N(0,1) block quantisation: tests/generators.py:34-58 (FP4 rounding
    boundaries, nibble packing), :61-95 (``quantize_with_major``);
  * expected outputs: tests/generators.py:300-322 (dense, alpha/bias/acc),
    :324-359 (m-grouped psum layout), :361-398 (k-grouped psum layout);
  * metric: tests/utils.py:36-43 (``calc_diff``);
  * FP4 -> E4M3 byte map: deep_gemm/include/deep_gemm/fp8_dequant_gemm.hpp:24-38.

Arithmetic contract: D[m,n] = sum over 32-wide K blocks kb of
(sum_{k in kb} A[m,k] B[n,k]) * 2^(eA[m,kb]-127) * 2^(eB[n,kb]-127), FP32
accumulation, one round-to-nearest cast at the end.
"""

from __future__ import annotations

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
               -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def decode_e4m3(t: torch.Tensor) -> torch.Tensor:
    """E4M3 bytes (uint8 / int8 / float8_e4m3fn storage) -> fp32 values."""
    if t.dtype != torch.float8_e4m3fn:
        t = t.view(torch.uint8).view(torch.float8_e4m3fn)
    return t.float()


def decode_e2m1_packed(packed: torch.Tensor, axis: int = -1) -> torch.Tensor:
    """Packed E2M1 (two codes per byte along ``axis``, low nibble = even index)
    -> fp32 values with ``axis`` doubled (tests/generators.py:45-49,98-102)."""
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    u = packed.contiguous().view(torch.uint8).transpose(axis, -1)
    lo = lut[(u & 0x0F).long()]
    hi = lut[(u >> 4).long()]
    out = torch.stack((lo, hi), dim=-1).reshape(*u.shape[:-1], u.shape[-1] * 2)
    return out.transpose(axis, -1)


def e2m1_to_e4m3_byte(code: int) -> int:
    """Exact E2M1 code -> E4M3 byte (fp8_dequant_gemm.hpp:24-38)."""
    mag = code & 7
    byte = 0x00 if mag == 0 else 0x30 if mag == 1 else 0x30 + (mag << 2)
    return byte | ((code & 8) << 4)


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """Round a positive float up to a power of two (tests/generators.py:27-31)."""
    bits = x.abs().float().contiguous().view(torch.int32)
    exp = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).int()
    return (exp.clamp(1, 254) << 23).view(torch.float32)


def _block_amax(x: torch.Tensor, gran: tuple[int, int]) -> torch.Tensor:
    mn, k = x.shape
    gm, gk = gran
    pm, pk = _ceil_div(mn, gm) * gm, _ceil_div(k, gk) * gk
    padded = torch.zeros(pm, pk, dtype=torch.float32)
    padded[:mn, :k] = x
    return padded.reshape(pm // gm, gm, pk // gk, gk).abs().amax(dim=(1, 3))


def _expand_sf(sf: torch.Tensor, shape: tuple[int, ...], gran: tuple[int, int]) -> torch.Tensor:
    full = sf.repeat_interleave(gran[0], dim=-2).repeat_interleave(gran[1], dim=-1)
    return full[..., :shape[-2], :shape[-1]]


def quantize_e4m3(x: torch.Tensor, gran: tuple[int, int]):
    """N(0,1)-style block quantisation to E4M3 (tests/generators.py:61-95).

    Returns (data float8 [MN,K], sf fp32 [ceil(MN/gm), ceil(K/gk)], dequantised fp32)."""
    sf = ceil_to_ue8m0(_block_amax(x, gran).clamp(1e-4) / 448.0)
    full = _expand_sf(sf, x.shape, gran)
    q = (x.float() / full).to(torch.float8_e4m3fn)
    return q, sf.contiguous(), (q.float() * full).contiguous()


def quantize_e2m1(x: torch.Tensor, gran: tuple[int, int], pack_axis: int = -1):
    """Block quantisation to packed E2M1 (tests/generators.py:34-50,61-95).

    Returns (packed int8 with ``pack_axis`` halved, sf fp32, dequantised fp32)."""
    sf = ceil_to_ue8m0(_block_amax(x, gran).clamp(1e-4) / 6.0)
    full = _expand_sf(sf, x.shape, gran)
    y = x.float() / full
    ay = y.abs()
    code = torch.zeros_like(y, dtype=torch.uint8)
    for boundary in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        code += (ay > boundary).to(torch.uint8)
    sign = (y < 0) & (code != 0)
    values = torch.tensor(E2M1_VALUES[:8], dtype=torch.float32)[code.long()]
    values = torch.where(sign, -values, values)
    code = code | (sign.to(torch.uint8) << 3)
    c = code.transpose(pack_axis, -1).contiguous()
    packed = ((c[..., 0::2] & 0x0F) | ((c[..., 1::2] & 0x0F) << 4)).view(torch.int8)
    return packed.transpose(pack_axis, -1), sf.contiguous(), (values * full).contiguous()


def dequantize(values: torch.Tensor, sf: torch.Tensor, gran_mn: int, gran_k: int) -> torch.Tensor:
    """values fp32 [..., MN, K] times sf fp32 [..., ceil(MN/gran_mn), ceil(K/gran_k)]."""
    return (values.float() * _expand_sf(sf.float(), values.shape, (gran_mn, gran_k))).contiguous()


def gemm_ref(a_deq: torch.Tensor, b_deq: torch.Tensor, out_dtype: torch.dtype,
             c: torch.Tensor | None = None, bias: torch.Tensor | None = None,
             alpha: float | None = None) -> torch.Tensor:
    """D = alpha * A @ B^T (+ C | + bias), one cast (tests/generators.py:316-322).

    ``a_deq`` is [M,K], ``b_deq`` is [N,K], both already dequantised fp32."""
    d = a_deq.float() @ b_deq.float().T
    if alpha is not None:
        d = alpha * d
    if c is not None:
        d = d + c.float()
    if bias is not None:
        d = d + bias.float().reshape(1, -1)
    return d.to(out_dtype)


def m_grouped_psum_ref(a_deq: torch.Tensor, b_deq: torch.Tensor, psum: list[int],
                       out_dtype: torch.dtype, alignment: int = 256) -> torch.Tensor:
    """Rows [align(psum[g-1]), psum[g]) of A use B[g]; all other rows of D are 0
    (tests/generators.py:346-353)."""
    from .sf_layout import psum_valid_spans, align
    total_m = align(psum[-1], alignment) if psum else 0
    assert a_deq.shape[0] == total_m
    d = torch.zeros(total_m, b_deq.shape[1], dtype=out_dtype)
    for g, span in enumerate(psum_valid_spans(psum, alignment)):
        d[span] = (a_deq[span].float() @ b_deq[g].float().T).to(out_dtype)
    return d


def k_grouped_psum_ref(a_deq: torch.Tensor, b_deq: torch.Tensor, psum: list[int], out_dtype: torch.dtype,
                       c: torch.Tensor | None = None, alignment: int = 256) -> torch.Tensor:
    """D[g] = A[span g]^T @ B[span g] (+ C[g]) with ``a_deq`` [K, M] and ``b_deq`` [K, N]; span g is
    [align(psum[g-1]), psum[g]) along K; an empty span gives 0 (+ C[g]) (tests/generators.py:392-396).
    With ``c`` the sum is formed in FP32 before the one cast, as the accumulating kernel does."""
    from .sf_layout import psum_valid_spans
    d = torch.zeros(len(psum), a_deq.shape[1], b_deq.shape[1], dtype=torch.float32)
    for g, span in enumerate(psum_valid_spans(psum, alignment)):
        d[g] = a_deq[span].float().T @ b_deq[span].float()
        if c is not None:
            d[g] += c[g].float()
    return d.to(out_dtype)


def m_grouped_masked_ref(a_deq: torch.Tensor, b_deq: torch.Tensor, masked_m: list[int],
                         out_dtype: torch.dtype) -> torch.Tensor:
    """D[g, :masked_m[g]] = A[g, :masked_m[g]] @ B[g]^T; other rows are returned
    as zero and must be ignored by the comparison (no reference test exists for
    this entry point: parity unpinned by the reference)."""
    g_, max_m, _ = a_deq.shape
    d = torch.zeros(g_, max_m, b_deq.shape[1], dtype=out_dtype)
    for g in range(g_):
        mg = int(masked_m[g])
        d[g, :mg] = (a_deq[g, :mg].float() @ b_deq[g].float().T).to(out_dtype)
    return d


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y>/(|x|^2+|y|^2) (tests/utils.py:36-43)."""
    x, y = x.double(), y.double()
    den = (x * x + y * y).sum()
    if den == 0:
        return 0.0
    return float(1 - 2 * (x * y).sum() / den)


def max_rel_err(x: torch.Tensor, y: torch.Tensor, floor_frac: float = 1.0 / 64) -> float:
    """max |x-y| / max(|y|, floor_frac * max|y|): element-wise relative error with
    a floor so that outputs that cancel to ~0 do not dominate."""
    x, y = x.double(), y.double()
    if y.numel() == 0:
        return 0.0
    scale = y.abs().max()
    if scale == 0:
        return float((x - y).abs().max())
    den = torch.maximum(y.abs(), scale * floor_frac)
    return float(((x - y).abs() / den).max())


def stochastic_round_bf16(fp32: torch.Tensor) -> torch.Tensor:
    """BF16 stochastic rounding model of the reference (tests/utils.py:70-92): per row, each aligned quartet of
    FP32 bit patterns (columns past N count as zero) and its index seed a hash; a value rounds up when its discarded
    16 bits exceed 0xffff minus its 16 random bits; NaN becomes 0x7fc0. Returns a bfloat16 tensor."""
    import numpy as np
    values = fp32.detach().cpu().contiguous().numpy().view(np.uint32)
    n = values.shape[-1]
    values = np.pad(values, [(0, 0)] * (values.ndim - 1) + [(0, -n % 4)])
    values = values.reshape(*values.shape[:-1], -1, 4)
    with np.errstate(over='ignore'):
        h = (values[..., 0] * np.uint32(0x5671d42b) + values[..., 1] * np.uint32(0x9995e499) +
             values[..., 2] * np.uint32(0xace1b8a5) + values[..., 3] * np.uint32(0xe153538d) +
             np.arange(values.shape[-2], dtype=np.uint32))
        h = (h ^ (h >> np.uint32(23))) * np.uint32(0x7feb352d)
        h ^= h >> np.uint32(16)
        h1, h2 = h * np.uint32(0x846ca68b), h * np.uint32(0xd35a2d97)
    h1 ^= h1 >> np.uint32(11)
    h2 ^= h2 >> np.uint32(11)
    random_bits = np.stack((h1 & 0xffff, h1 >> np.uint32(16), h2 & 0xffff, h2 >> np.uint32(16)), axis=-1)
    rounded = (values >> np.uint32(16)) + ((values & 0xffff) > (0xffff - random_bits))
    rounded = np.where((values & 0x7fffffff) > 0x7f800000, 0x7fc0, rounded).astype(np.uint16)
    out = rounded.reshape(*fp32.shape[:-1], -1)[..., :n].copy()
    return torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)
