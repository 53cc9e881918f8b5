"""Checkers the benchmark hangs on its timed cases: sampled rows of an output against the oracle.

TEST INFRASTRUCTURE, like the rest of this package: `bench.py` imports these functions and hands them to the workloads
of `deep_gemm.testing` as callables, so that nothing inside the shipped package refers to the oracle. A case object only
has to expose its device tensors (`a`, `b`, `sfa`, `sfb` in the required int16 layout, `d`) and its sizes.
Tolerance as in tests/helpers.py: 1 - cosine <= 1e-3, max relative error <= 2e-2.
"""

from __future__ import annotations

import torch

from .mxgemm import calc_diff, decode_e2m1_packed, decode_e4m3, dequantize, gemm_ref, max_rel_err
from .sf_layout import unpack_required_sf


def close(out: torch.Tensor, ref: torch.Tensor) -> bool:
    out, ref = out.cpu(), ref.cpu()
    return bool(torch.isfinite(out.float()).all()) and calc_diff(out, ref) <= 1e-3 and max_rel_err(out, ref) <= 2e-2


def _scales(sf16: torch.Tensor, k: int) -> torch.Tensor:
    """Required-layout int16 scales [..., MN, K64] (any strides) -> FP32 scales [..., MN, ceil(K/32)] on the host."""
    return unpack_required_sf(sf16.cpu().contiguous(), k)


def _values(kind: str, t: torch.Tensor) -> torch.Tensor:
    return decode_e4m3(t.cpu()) if kind == 'fp8' else decode_e2m1_packed(t.cpu(), axis=-1)


def mixed_case(case, rows: int = 16) -> bool:
    """FP8 x packed-FP4 "NN": a [M, K] E4M3, b [K, N / 2] packed E2M1."""
    idx = torch.randperm(case.m, generator=torch.Generator().manual_seed(3))[:rows].sort().values
    a_deq = dequantize(decode_e4m3(case.a[idx.to(case.a.device)].cpu()), _scales(case.sfa, case.k)[idx], 1, 32)
    b_vals = decode_e2m1_packed(case.b.cpu(), axis=-1).transpose(0, 1)            # [N, K]
    b_deq = dequantize(b_vals, _scales(case.sfb, case.k), 1, 32)
    return close(case.d[idx.to(case.d.device)], gemm_ref(a_deq, b_deq, torch.bfloat16))


def grouped_case(case, sizes, masked: bool, samples: int = 6) -> bool:
    """m-grouped contiguous (psum layout) or masked FP8 GEMM: the first 64 valid rows and the last 64 of a few groups."""
    g_all = [g for g, s in enumerate(sizes) if s > 0]
    picks = g_all[:: max(1, len(g_all) // samples)][:samples]
    ok, psum_start, starts = True, 0, []
    for s in sizes:
        starts.append(psum_start)
        psum_start = (psum_start + s + 255) // 256 * 256
    for g in picks:
        rows = sizes[g]
        b_deq = dequantize(decode_e4m3(case.b[g].cpu()), _scales(case.sfb[g], case.k), 1, 32)
        for lo in {0, max(0, rows - 64)}:
            hi = min(rows, lo + 64)
            if masked:
                a_blk, sf_blk, d_blk = case.a[g, lo:hi], case.sfa[g, lo:hi], case.d[g, lo:hi]
            else:
                r0 = starts[g]
                a_blk, sf_blk, d_blk = case.a[r0 + lo:r0 + hi], case.sfa[r0 + lo:r0 + hi], case.d[r0 + lo:r0 + hi]
            a_deq = dequantize(decode_e4m3(a_blk.cpu()), _scales(sf_blk, case.k), 1, 32)
            ok = ok and close(d_blk, gemm_ref(a_deq, b_deq, torch.bfloat16))
    return ok


def dense_row(case, rows: int = 8) -> bool:
    """Dense NT GEMM with K-major operands of kinds `case.kind_a` / `case.kind_b` ('fp8' or 'fp4')."""
    idx = torch.randperm(case.m, generator=torch.Generator().manual_seed(3))[:rows].sort().values
    a_deq = dequantize(_values(case.kind_a, case.a[idx.to(case.a.device)]), _scales(case.sfa, case.k)[idx], 1, 32)
    b_deq = dequantize(_values(case.kind_b, case.b), _scales(case.sfb, case.k), 1, 32)
    return close(case.d[idx.to(case.d.device)], gemm_ref(a_deq, b_deq, torch.bfloat16))


def grouped_row(case, rows: int = 16) -> bool:
    """m-grouped contiguous FP8 x packed-FP4 GEMM: the first and the last `rows` valid rows of the first and last group."""
    ok, start, starts = True, 0, []
    for s in case.sizes:
        starts.append(start)
        start = (start + s + 255) // 256 * 256
    for g in (0, len(case.sizes) - 1):
        b_deq = dequantize(_values('fp4', case.b[g]), _scales(case.sfb[g], case.k), 1, 32)
        for lo in {0, max(0, case.sizes[g] - rows)}:
            r = slice(starts[g] + lo, starts[g] + min(case.sizes[g], lo + rows))
            a_deq = dequantize(_values('fp8', case.a[r]), _scales(case.sfa[r], case.k), 1, 32)
            ok = ok and close(case.d[r], gemm_ref(a_deq, b_deq, torch.bfloat16))
    return ok


def moe_mlp_case(case, rows: int = 24) -> bool:
    """The expert MLP chain (GEMM, SwiGLU * weight -> FP8, GEMM) on the first rows of the first and of the last expert:
    the first GEMM against the oracle; the quantiser against the oracle applied to the GEMM's own BF16 output (codes
    within one E4M3 step where the device's exp differs in the last bit, scales equal); the second GEMM against the
    oracle applied to the quantiser's own output."""
    from .quant import swiglu_quant_ref
    ok, start, starts = True, 0, []
    for s_ in case.sizes:
        starts.append(start)
        start = (start + s_ + 255) // 256 * 256
    for g in (0, len(case.sizes) - 1):
        n_rows = min(rows, case.sizes[g])
        if n_rows == 0:
            continue
        r = slice(starts[g], starts[g] + n_rows)
        x_deq = dequantize(_values('fp8', case.x[r]), _scales(case.sfx[r], case.hidden), 1, 32)
        w1_deq = dequantize(_values('fp4', case.w1[g]), _scales(case.sfw1[g], case.hidden), 1, 32)
        ok = ok and close(case.y1[r], gemm_ref(x_deq, w1_deq, torch.bfloat16))
        codes, sf, _, deq = swiglu_quant_ref(case.y1[r].cpu(), case.topk_weights[r].cpu())
        a2_deq = dequantize(_values('fp8', case.a2[r]), _scales(case.sfa2[r], case.intermediate), 1, 32)
        ok = ok and close(a2_deq, deq)
        w2_deq = dequantize(_values('fp4', case.w2[g]), _scales(case.sfw2[g], case.intermediate), 1, 32)
        ok = ok and close(case.y2[r], gemm_ref(a2_deq, w2_deq, torch.bfloat16))
    return ok
