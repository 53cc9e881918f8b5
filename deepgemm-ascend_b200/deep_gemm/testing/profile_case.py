"""Run one GEMM shape a few times: the small, self-ending workload to put under `ncu`.

    python -m deep_gemm.testing.profile_case --m 4096 --n 7168 --k 16384 --iters 3 [--block-n 192 --cta-group 1 ...]

Operands are random E4M3 codes with random UE8M0 scales already in the required layout, so only the GEMM kernel
(and the split-K finalisation, when the tiling uses it) is launched.
"""

from __future__ import annotations

import argparse

import torch

import deep_gemm


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--m', type=int, default=4096)
    ap.add_argument('--n', type=int, default=7168)
    ap.add_argument('--k', type=int, default=16384)
    ap.add_argument('--groups', type=int, default=0, help='>0: m-grouped contiguous with this many groups of m rows')
    ap.add_argument('--iters', type=int, default=3)
    ap.add_argument('--block-n', type=int, default=0)
    ap.add_argument('--cta-group', type=int, default=0)
    ap.add_argument('--split-k', type=int, default=0)
    ap.add_argument('--stages', type=int, default=0)
    ap.add_argument('--raster-group', type=int, default=0, help='row blocks per group of the dense tile walk (0 = default)')
    ap.add_argument('--out', default='bf16', choices=['bf16', 'f32'])
    ap.add_argument('--fp4', action='store_true', help='both operands packed E2M1 (dense only)')
    ap.add_argument('--bf16', action='store_true', help='BF16 operands, no scale factors (dense only)')
    ap.add_argument('--quant', default='', choices=['', 'swiglu', 'cast'],
                    help='run the FP8 producer on [m, k] activations instead of a GEMM')
    ap.add_argument('--mixed', action='store_true', help='FP8 x packed FP4 "NN": B is [k, n / 2] packed E2M1 (dense only)')
    ap.add_argument('--masked', type=int, default=0, help='>0: m-grouped masked with this many groups of at most m rows')
    ap.add_argument('--layout', action='store_true',
                    help='run transform_sf_into_required_layout on FP32 scales [m, k / 32] instead of a GEMM')
    args = ap.parse_args()

    torch.manual_seed(0)
    dev = torch.device('cuda', 0)
    m, n, k, g = args.m, args.n, args.k, args.groups
    k64 = (k + 63) // 64
    rows = m * g if g else m

    if args.quant:
        x = torch.randn(m, k * (2 if args.quant == 'swiglu' else 1), device=dev).bfloat16()
        for _ in range(args.iters):
            if args.quant == 'swiglu':
                deep_gemm.swiglu_apply_weight_to_fp8(x)
            else:
                deep_gemm.cast_to_fp8(x)
        torch.cuda.synchronize()
        print('status', deep_gemm.device_status(), 'launches', args.iters)
        return

    if args.layout:
        sf = (torch.randint(100, 140, (m, k // 32), dtype=torch.int32, device=dev) << 23).view(torch.float32)
        for _ in range(args.iters):
            deep_gemm.transform_sf_into_required_layout(sf, m, k, (1, 1, 32), is_sfa=True)
        torch.cuda.synchronize()
        print('status', deep_gemm.device_status(), 'launches', args.iters)
        return

    def codes(*shape):
        return torch.randint(0, 120, shape, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)

    def scales(lead, mn):
        t = torch.randint(120, 130, (*lead, k64, mn), dtype=torch.int16, device=dev)
        return (t | (t << 8)).transpose(-2, -1)

    a, sfa = codes(rows, k), scales((), rows)
    b, sfb = (codes(g, n, k), scales((g,), n)) if g else (codes(n, k), scales((), n))
    if args.fp4:
        a = torch.randint(-128, 128, (rows, k // 2), dtype=torch.int8, device=dev)
        b = torch.randint(-128, 128, (n, k // 2), dtype=torch.int8, device=dev)
    d = torch.empty(rows, n, dtype=torch.bfloat16 if args.out == 'bf16' else torch.float32, device=dev)
    if args.bf16:
        a_bf16 = torch.randn(rows, k, device=dev).bfloat16()
        b_bf16 = torch.randn(n, k, device=dev).bfloat16()
    config = {key: val for key, val in (('block_n', args.block_n), ('cta_group', args.cta_group),
                                        ('split_k', args.split_k), ('num_stages', args.stages),
                                        ('raster_group', args.raster_group)) if val}
    layout = torch.arange(1, g + 1, dtype=torch.int32, device=dev) * m if g else None
    if args.mixed:
        b_packed = torch.randint(-128, 128, (k, n // 2), dtype=torch.int8, device=dev)
    if args.masked:
        gm = args.masked
        a3, sfa3 = codes(gm, m, k), scales((gm,), m)
        b3, sfb3 = codes(gm, n, k), scales((gm,), n)
        d3 = torch.empty(gm, m, n, dtype=torch.bfloat16, device=dev)
        mask = torch.randint(0, m + 1, (gm,), dtype=torch.int32, device=dev)
    for _ in range(args.iters):
        if args.masked:
            deep_gemm.m_grouped_fp8_gemm_nt_masked((a3, sfa3), (b3, sfb3), d3, mask, m // 2, config=config or None)
        elif args.mixed:
            deep_gemm.fp8_fp4_gemm_nn((a, sfa), (b_packed, sfb.transpose(0, 1)), d, config=config or None)
        elif args.bf16:
            deep_gemm.bf16_gemm_nt(a_bf16, b_bf16, d, config=config or None)
        elif g:
            deep_gemm.m_grouped_fp8_gemm_nt_contiguous((a, sfa), (b, sfb), d, layout, config=config or None)
        else:
            deep_gemm.fp8_gemm_nt((a, sfa), (b, sfb), d, config=config or None)
    torch.cuda.synchronize()
    print('status', deep_gemm.device_status(), 'launches', args.iters)


if __name__ == '__main__':
    main()
