"""Every row of the reference's own published tables (README.md:108-147), timed on this GPU.

The reference measured on an Ascend 950DT with cold L2 (README.md:102); the figures below are its published latency
and TFLOPS per row, kept here only to print them beside this build's numbers. The dense rows are timed like the
shapes of the dense sweep (a CUDA graph of back-to-back launches over rotating operand sets that together exceed L2
several times); the m-grouped rows run for a millisecond or more and are timed per launch after an untimed L2 flush.
Every dense row is also timed the reference's way: alone, after a buffer larger than L2 has been written, its duration
read from the profiler's activity trace (that leaves L2 full of dirty lines, whose write-back the kernel then pays for).
Operands are synthetic: uniform E4M3 / E2M1 codes with power-of-two UE8M0 scales per 32 elements of K, already in the
required layout, BF16 output. The caller may pass checkers that compare a sampled row block of every row with a reference
on the host (the benchmark passes the CPU oracle's).
"""

from __future__ import annotations

import ctypes
import json
import math
import random

import torch

from .. import _api
from .. import _lib as L
from .bench import bench_graph, bench_msprof
from .moe_bench import _codes, _flush_timed, _scales
from .sharding import shard_psum_layout

# (operand kinds, M, N, K, published latency in us, published TFLOPS, where)
DENSE_ROWS = [
    ('fp8xfp8', 4096, 7168, 16384, 1117.6, 861, 'README.md:112,130'),
    ('fp8xfp4', 4096, 7168, 16384, 1117.8, 861, 'README.md:111'),
    ('fp4xfp4', 4096, 7168, 16384, 565.6, 1701, 'README.md:110'),
    ('fp8xfp8', 128, 2112, 7168, 15.0, 258, 'README.md:119'),
    ('fp8xfp8', 128, 576, 7168, 10.1, 105, 'README.md:120'),
    ('fp8xfp8', 128, 24576, 1536, 20.6, 468, 'README.md:121'),
    ('fp8xfp8', 128, 32768, 512, 10.4, 415, 'README.md:122'),
    ('fp8xfp8', 128, 7168, 16384, 54.8, 549, 'README.md:123'),
    ('fp8xfp8', 128, 4096, 7168, 19.0, 397, 'README.md:124'),
    ('fp8xfp8', 128, 7168, 2048, 10.1, 373, 'README.md:125'),
    ('fp8xfp8', 4096, 2112, 7168, 156.9, 790, 'README.md:126'),
    ('fp8xfp8', 4096, 576, 7168, 54.6, 619, 'README.md:127'),
    ('fp8xfp8', 4096, 24576, 1536, 362.2, 854, 'README.md:128'),
    ('fp8xfp8', 4096, 32768, 512, 164.3, 837, 'README.md:129'),
    ('fp8xfp8', 4096, 4096, 7168, 282.9, 850, 'README.md:131'),
    ('fp8xfp8', 4096, 7168, 2048, 143.4, 838, 'README.md:132'),
]
# m-grouped contiguous, FP8 x packed FP4, BF16 out: (groups, rows per group, N, K, latency in us, TFLOPS, where)
GROUPED_ROWS = [
    (4, 8192, 6144, 7168, 3722.4, 818, 'README.md:140'),
    (4, 8192, 7168, 3072, 1778.0, 856, 'README.md:141'),
    (4, 8192, 4096, 4096, 1356.1, 855, 'README.md:142'),
    (4, 8192, 4096, 2048, 680.6, 852, 'README.md:143'),
    (8, 4096, 6144, 7168, 3689.4, 831, 'README.md:144'),
    (8, 4096, 7168, 3072, 1778.9, 862, 'README.md:145'),
    (8, 4096, 4096, 4096, 1356.5, 861, 'README.md:146'),
    (8, 4096, 4096, 2048, 681.0, 858, 'README.md:147'),
]


def _operand(kind: str, lead, mn: int, k: int, device, gen) -> torch.Tensor:
    """K-major operand [..., mn, k]: E4M3 bytes, or packed E2M1 (two codes per byte along K) as int8 [..., mn, k / 2]."""
    if kind == 'fp8':
        return _codes((*lead, mn, k), device, gen)
    return torch.randint(-128, 128, (*lead, mn, k // 2), dtype=torch.int8, device=device, generator=gen)


class DenseRow:
    def __init__(self, kinds: str, m: int, n: int, k: int, device, seed: int):
        gen = torch.Generator(device=device).manual_seed(seed)
        self.kind_a, self.kind_b = kinds.split('x')
        self.m, self.n, self.k = m, n, k
        self.a = _operand(self.kind_a, (), m, k, device, gen)
        self.b = _operand(self.kind_b, (), n, k, device, gen)
        self.sfa = _scales((), m, k, device, gen)
        self.sfb = _scales((), n, k, device, gen)
        self.d = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        self.desc = _api._run_gemm(L.GEMM_NORMAL, self.a, self.b, self.d, None, _api.Identity(), self.sfa, self.sfb,
                                   (1, 1, 32), None, None, None, 'nk', False)
        lib = L.lib()
        cfg = L.GemmConfig()
        L.check(lib.dg_select_config(ctypes.byref(self.desc), ctypes.byref(cfg)))
        self.config = cfg.as_dict()
        ws_bytes = lib.dg_gemm_workspace_bytes(ctypes.byref(self.desc), None)
        self.ws = _api._workspace(device, ws_bytes) if ws_bytes else None
        bits_a, bits_b = (8 if self.kind_a == 'fp8' else 4), (8 if self.kind_b == 'fp8' else 4)
        self.flops = 2.0 * m * n * k
        self.bytes = m * k * bits_a // 8 + n * k * bits_b // 8 + (m + n) * ((k + 63) // 64) * 2 + m * n * 2

    def launch(self, lib, sptr):
        L.check(lib.dg_gemm_launch(ctypes.byref(self.desc), None, self.ws.data_ptr() if self.ws is not None else None,
                                   self.ws.numel() if self.ws is not None else 0, sptr))


class GroupedRow:
    """m-grouped contiguous GEMM on the 256-row psum layout: A [rows, K] E4M3, B [G, N, K / 2] packed E2M1, K-major."""

    def __init__(self, sizes, n: int, k: int, device, seed: int):
        gen = torch.Generator(device=device).manual_seed(seed)
        self.sizes, self.n, self.k, g = list(sizes), n, k, len(sizes)
        local = shard_psum_layout(self.sizes, 1, 0)
        self.rows, self.valid_rows = local['rows'], sum(sizes)
        self.a = _codes((self.rows, k), device, gen)
        self.b = _operand('fp4', (g,), n, k, device, gen)
        self.sfa = _scales((), self.rows, k, device, gen)
        self.sfb = _scales((g,), n, k, device, gen)
        self.d = torch.empty(self.rows, n, dtype=torch.bfloat16, device=device)
        self.layout = torch.tensor(local['psum'], dtype=torch.int32, device=device)
        self.desc = _api._run_gemm(L.GEMM_M_GROUPED_PSUM, self.a, self.b, self.d, None, _api.Identity(), self.sfa, self.sfb,
                                   (1, 1, 32), None, None, self.layout, 'nk', False, expected_m=max(1, self.valid_rows // g))
        cfg = L.GemmConfig()
        L.check(L.lib().dg_select_config(ctypes.byref(self.desc), ctypes.byref(cfg)))
        self.config = cfg.as_dict()
        k64 = (k + 63) // 64
        self.flops = 2.0 * self.valid_rows * n * k
        self.bytes = self.valid_rows * (k + k64 * 2 + n * 2) + g * n * (k // 2 + k64 * 2)

    def launch(self, lib, sptr):
        L.check(lib.dg_gemm_launch(ctypes.byref(self.desc), None, None, 0, sptr))


def time_published(device, steps: int, alone_too: bool = False, check_dense=None, check_grouped=None) -> dict:
    """All rows on one GPU. Returns {'rows': [...], 'tflops', 'published_tflops', 'geomean_speedup', 'verified'}."""
    lib = L.lib()
    rows, ok = [], True
    for i, (kinds, m, n, k, pub_us, pub_tf, where) in enumerate(DENSE_ROWS):
        first = DenseRow(kinds, m, n, k, device, seed=500 + i)
        copies = max(3, min(32, -(-512_000_000 // first.bytes)))
        sets = [first] + [DenseRow(kinds, m, n, k, device, seed=9000 + 40 * i + j) for j in range(copies - 1)]
        us = bench_graph([(lambda sptr, s=s: s.launch(lib, sptr)) for s in sets], 3, steps).dur_us
        ok = (check_dense(first) if check_dense is not None else True) and ok
        # the reference's own method (deep_gemm/testing/bench.py:284-400): the kernel alone after a buffer larger than L2
        # has been written, its duration taken from the profiler's activity trace; None where no trace can be had
        alone = None
        try:
            sptr = torch.cuda.current_stream(device).cuda_stream
            if alone_too:
                alone = bench_msprof(lambda: first.launch(lib, sptr), kernel_names='mx_gemm_kernel', num_warmups=2, num_tests=10).dur_us
        except Exception:      # noqa: BLE001 - the trace is an extra; the CUDA-event figures above stand without it
            alone = None
        rows.append({'case': 'dense %s %dx%dx%d' % (kinds, m, n, k), 'us': round(us, 2),
                     'tflops': round(first.flops / us / 1e6, 1), 'gbs': round(first.bytes / us / 1e3, 1),
                     'published_us': pub_us, 'published_tflops': pub_tf, 'published_at': where,
                     'speedup': round(pub_us / us, 2), 'us_alone_after_written_flush': round(alone, 2) if alone else None,
                     'block_n': first.config['block_n'],
                     'cta_group': first.config['cta_group'], 'split_k': first.config['split_k'], 'flops': first.flops})
        del sets, first
    torch.cuda.empty_cache()
    for i, (g, per_group, n, k, pub_us, pub_tf, where) in enumerate(GROUPED_ROWS):
        random.seed(4000 + i)
        sizes = [int(random.uniform(0.7, 1.3) * per_group) for _ in range(g)]          # tests/generators.py:212-220
        case = GroupedRow(sizes, n, k, device, seed=700 + i)
        us = _flush_timed(lib, device, lambda sptr: case.launch(lib, sptr), steps)
        ok = (check_grouped(case) if check_grouped is not None else True) and ok
        # the published row is for groups x rows-per-group rows; scale its latency to the rows drawn here
        pub_scaled = pub_us * case.valid_rows / (g * per_group)
        rows.append({'case': 'm-grouped fp8xfp4 %d x %d rows (%d valid), N=%d K=%d' % (g, per_group, case.valid_rows, n, k),
                     'us': round(us, 1), 'tflops': round(case.flops / us / 1e6, 1), 'gbs': round(case.bytes / us / 1e3, 1),
                     'published_us': pub_us, 'published_tflops': pub_tf, 'published_at': where,
                     'speedup': round(pub_scaled / us, 2), 'block_n': case.config['block_n'],
                     'cta_group': case.config['cta_group'], 'split_k': 1, 'flops': case.flops})
        del case
        torch.cuda.empty_cache()
    flops = sum(r['flops'] for r in rows)
    ours_s = sum(r['us'] for r in rows) * 1e-6
    theirs_s = sum(r['flops'] / (r['published_tflops'] * 1e12) for r in rows)
    for r in rows:
        del r['flops']
    return {'rows': rows, 'tflops': flops / ours_s / 1e12, 'published_tflops': flops / theirs_s / 1e12,
            'geomean_speedup': math.exp(sum(math.log(r['speedup']) for r in rows) / len(rows)),
            'verified': ok if (check_dense is not None and check_grouped is not None) else None,
            'us_total': ours_s * 1e6}


def run_published(args, rank, world, device, emit=None, check_dense=None, check_grouped=None):
    r = time_published(device, max(3, min(args.steps, 10)), alone_too=True, check_dense=check_dense, check_grouped=check_grouped)
    if rank != 0:
        return
    line = {'metric': 'fp8_block_scaled_gemm_tflops', 'value': world * r['tflops'], 'unit': 'TFLOP/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': r['us_total'] / 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': r['tflops'] / r['published_tflops'],
            'vs_baseline_is': 'same rows, the reference\'s published TFLOPS on Ascend 950DT (other hardware): %.0f TFLOP/s '
                              'over the table' % r['published_tflops'],
            'dtype': 'fp8_e4m3 / fp4_e2m1 x ue8m0, fp32 accumulate', 'data': 'synthetic',
            'config': {'workload': 'every row of the reference\'s published tables: %d dense rows (FP8xFP8, FP8xFP4, FP4xFP4), '
                                   '%d m-grouped contiguous FP8xFP4 rows' % (len(DENSE_ROWS), len(GROUPED_ROWS)),
                       'l2': 'dense rows: rotating operand sets larger than L2; grouped rows: flushed before every launch, untimed'},
            'geomean_speedup_vs_published': round(r['geomean_speedup'], 2), 'verified': r['verified'], 'rows': r['rows'],
            'device_status': _api.device_status()}
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)
