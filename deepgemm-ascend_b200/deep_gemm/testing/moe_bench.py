"""MoE workloads of the benchmark: m-grouped contiguous (psum layout) and m-grouped masked FP8 GEMM.

Experts are sharded across ranks (`sharding.py`); each rank runs the single-GPU kernel on its own experts, no
data-path collective. `--gather` times an NCCL all-gather of the outputs separately.
"""

from __future__ import annotations

import ctypes
import json
import random

import torch

from .. import _api
from .. import _lib as L
from .bench import l2_flush_buffer
from .sharding import shard_psum_layout

NK_LIST = [(4096, 7168), (7168, 2048)]


def _codes(shape, device, gen):
    raw = torch.randint(0, 254, shape, dtype=torch.uint8, device=device, generator=gen)
    raw += (raw >= 0x7F).to(torch.uint8)
    return raw.view(torch.float8_e4m3fn)


def _scales(lead, mn, k, device, gen):
    k64 = (k + 63) // 64
    e = torch.randint(118, 121, (*lead, k64, mn), dtype=torch.int16, device=device, generator=gen)
    return (e | (e << 8)).transpose(-2, -1)


class GroupedCase:
    def __init__(self, sizes, n, k, device, seed, masked_max_m=0):
        gen = torch.Generator(device=device).manual_seed(seed)
        self.n, self.k, g = n, k, len(sizes)
        self.valid_rows = sum(sizes)
        if masked_max_m:
            rows_shape, self.rows = (g, masked_max_m), g * masked_max_m
            layout = sizes
            gemm_type = L.GEMM_M_GROUPED_MASKED
        else:
            local = shard_psum_layout(sizes, 1, 0)
            rows_shape, self.rows = (local['rows'],), local['rows']
            layout = local['psum']
            gemm_type = L.GEMM_M_GROUPED_PSUM
        self.a = _codes((*rows_shape, k), device, gen)
        self.b = _codes((g, n, k), device, gen)
        self.sfa = _scales(rows_shape[:-1], rows_shape[-1], k, device, gen)
        self.sfb = _scales((g,), n, k, device, gen)
        self.d = torch.empty((*rows_shape, n), dtype=torch.bfloat16, device=device)
        self.layout = torch.tensor(layout, dtype=torch.int32, device=device)
        self.desc = _api._run_gemm(gemm_type, self.a, self.b, self.d, None, _api.Identity(), self.sfa, self.sfb,
                                   (1, 1, 32), None, None, self.layout, 'nk', False,
                                   expected_m=max(1, self.valid_rows // g))
        self.flops = 2.0 * self.valid_rows * n * k
        k64 = (k + 63) // 64
        self.bytes = self.valid_rows * (k + k64 * 2 + n * 2) + g * n * (k + k64 * 2)
        cfg = L.GemmConfig()
        L.check(L.lib().dg_select_config(ctypes.byref(self.desc), ctypes.byref(cfg)))
        self.config = cfg.as_dict()

    def launch(self, lib, sptr):
        rc = lib.dg_gemm_launch(ctypes.byref(self.desc), None, None, 0, sptr)
        if rc:
            raise RuntimeError(L.last_error())


def run(args, rank, world, device, emit=None):
    if args.workload == 'mixed':
        return run_mixed(args, rank, world, device, emit)
    if args.workload == 'fp4':
        return run_fp4(args, rank, world, device, emit)
    if args.workload == 'bf16':
        return run_bf16(args, rank, world, device, emit)
    if args.workload == 'quant':
        return run_quant(args, rank, world, device, emit)
    lib = L.lib()
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    flush = l2_flush_buffer(device)
    masked = args.workload == 'masked'
    per_rank = getattr(args, 'experts_per_gpu', 0) or (32 if masked else 8)
    random.seed(1234)                       # the global problem is the same on every rank
    g_total = per_rank * world
    if masked:
        sizes = [random.randint(0, 256) for _ in range(g_total)]
    else:
        sizes = [int(random.uniform(0.7, 1.3) * 8192) for _ in range(g_total)]
    mine = sizes[rank * per_rank:(rank + 1) * per_rank]
    cases = [GroupedCase(mine, n, k, device, seed=100 * rank + i, masked_max_m=256 if masked else 0)
             for i, (n, k) in enumerate(NK_LIST)]
    torch.cuda.synchronize(device)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    def step(events):
        for ci, c in enumerate(cases):
            L.check(lib.dg_l2_flush_launch(flush.data_ptr(), flush.numel(), sptr))
            if events is not None:
                events[ci][0].record(stream)
            c.launch(lib, sptr)
            if events is not None:
                events[ci][1].record(stream)

    for _ in range(max(args.warmup, 3)):
        step(None)
    barrier()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in cases]
          for _ in range(args.steps)]
    launches0 = lib.dg_kernel_launch_count()
    for s in range(args.steps):
        step(ev[s])
    barrier()
    launches = lib.dg_kernel_launch_count() - launches0
    per_case_us = [sum(ev[s][ci][0].elapsed_time(ev[s][ci][1]) for s in range(args.steps)) / args.steps * 1e3
                   for ci in range(len(cases))]
    step_ms = torch.tensor([sum(per_case_us) / 1e3], dtype=torch.float64, device=device)
    flops = torch.tensor([sum(c.flops for c in cases)], dtype=torch.float64, device=device)
    gather_ms = None
    if world > 1:
        torch.distributed.all_reduce(step_ms, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(flops, op=torch.distributed.ReduceOp.SUM)
        if getattr(args, 'gather', False):
            # outputs have rank-dependent row counts: gather equal-sized padded chunks
            rows = torch.tensor([cases[0].rows], dtype=torch.int64, device=device)
            torch.distributed.all_reduce(rows, op=torch.distributed.ReduceOp.MAX)
            chunk = torch.zeros(int(rows.item()), cases[0].n, dtype=torch.bfloat16, device=device)
            chunk[:cases[0].rows].copy_(cases[0].d.reshape(-1, cases[0].n))
            out = torch.empty(world * chunk.size(0), chunk.size(1), dtype=torch.bfloat16, device=device)
            torch.distributed.all_gather_into_tensor(out, chunk)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            torch.distributed.all_gather_into_tensor(out, chunk)
            e1.record(stream)
            barrier()
            g_ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
            torch.distributed.all_reduce(g_ms, op=torch.distributed.ReduceOp.MAX)
            gather_ms = float(g_ms.item())
    status = _api.device_status()
    if rank != 0:
        return
    value = float(flops.item()) / (float(step_ms.item()) * 1e-3) / 1e12
    line = {
        'metric': 'fp8_block_scaled_gemm_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': float(step_ms.item()),
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'fp8_e4m3 x ue8m0, fp32 accumulate', 'data': 'synthetic',
        'config': {'workload': ('m-grouped masked FP8 GEMM, %d experts x max_m 256 per GPU' if masked else
                                'm-grouped contiguous FP8 GEMM (psum layout), %d experts per GPU, m ~ U(0.7,1.3) x 8192')
                               % per_rank + ', (N,K) in ' + str(NK_LIST) + ', BF16 out',
                   'sharding': 'experts, contiguous blocks per rank, no data-path collective',
                   'l2': 'flushed before every GEMM, untimed', 'flops': 'valid rows only'},
        'gpu_launches': int(launches), 'device_status': status,
        'shapes': [{'rows': c.rows, 'valid_rows': c.valid_rows, 'n': c.n, 'k': c.k, 'us': round(per_case_us[i], 1),
                    'tflops': round(c.flops / per_case_us[i] / 1e6, 1), 'gbs': round(c.bytes / per_case_us[i] / 1e3, 1),
                    'block_n': c.config['block_n'], 'cta_group': c.config['cta_group']} for i, c in enumerate(cases)],
    }
    if gather_ms is not None:
        line['gather_ms'] = gather_ms
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)


def run_mixed(args, rank, world, device, emit=None):
    """FP8 x packed-FP4 GEMM "NN": A [M,K] E4M3 with per-128 scales, B [K, N/2] packed E2M1 (uniform codes) with
    per-32 scales, BF16 out; M=4096, N=7168, K=2048. Normalised by the FP8 peak (the MMA runs on E4M3 operands)."""
    lib = L.lib()
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    flush = l2_flush_buffer(device)
    gen = torch.Generator(device=device).manual_seed(7 + rank)
    m, n, k = 4096, 7168, 2048
    a = _codes((m, k), device, gen)
    b = torch.randint(-128, 128, (k, n // 2), dtype=torch.int8, device=device, generator=gen)
    sfa = _scales((), m, k, device, gen)
    sfb = _scales((), n, k, device, gen)
    d = torch.empty(m, n, dtype=torch.bfloat16, device=device)
    desc = _api._run_gemm(L.GEMM_NORMAL, a, b.transpose(0, 1), d, None, _api.Identity(), sfa, sfb,
                          (1, 1, 32), None, None, None, 'nk', False)
    cfg = L.GemmConfig()
    L.check(lib.dg_select_config(ctypes.byref(desc), ctypes.byref(cfg)))

    def once(events=None):
        L.check(lib.dg_l2_flush_launch(flush.data_ptr(), flush.numel(), sptr))
        if events:
            events[0].record(stream)
        L.check(lib.dg_gemm_launch(ctypes.byref(desc), None, None, 0, sptr))
        if events:
            events[1].record(stream)

    for _ in range(max(args.warmup, 3)):
        once()
    torch.cuda.synchronize(device)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for e in ev:
        once(e)
    torch.cuda.synchronize(device)
    us = sum(a_.elapsed_time(b_) for a_, b_ in ev) / args.steps * 1e3
    if rank != 0:
        return
    flops = 2.0 * m * n * k
    nbytes = m * k + n * k // 2 + (m + n) * ((k + 63) // 64) * 2 + m * n * 2
    line = {'metric': 'fp8_block_scaled_gemm_tflops', 'value': world * flops / us / 1e6, 'unit': 'TFLOP/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': us / 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp8_e4m3 x fp4_e2m1 (decoded to e4m3), ue8m0 scales',
            'data': 'synthetic',
            'config': {'workload': 'mixed FP8xFP4 GEMM NN, M=4096 N=7168 K=2048, BF16 out', 'l2': 'flushed, untimed'},
            'gbs': nbytes / us / 1e3, 'tiling': cfg.as_dict(), 'device_status': _api.device_status()}
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)


def run_fp4(args, rank, world, device, emit=None):
    """FP4 x FP4 GEMM "NT" (both operands packed E2M1, K-major, per-32 UE8M0 scales, BF16 out) on the shapes the
    reference publishes for this kind (README.md:108-113: 4096 x 7168 x 16384) plus two more of the dense sweep.
    Normalised by the dense FP4 peak (twice the FP8 figure)."""
    lib = L.lib()
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    flush = l2_flush_buffer(device)
    gen = torch.Generator(device=device).manual_seed(11 + rank)
    shapes = [(4096, 7168, 16384), (4096, 4096, 7168), (4096, 7168, 2048), (128, 7168, 16384)]
    rows = []
    for (m, n, k) in shapes:
        a = torch.randint(-128, 128, (m, k // 2), dtype=torch.int8, device=device, generator=gen)
        b = torch.randint(-128, 128, (n, k // 2), dtype=torch.int8, device=device, generator=gen)
        sfa = _scales((), m, k, device, gen)
        sfb = _scales((), n, k, device, gen)
        d = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        desc = _api._run_gemm(L.GEMM_NORMAL, a, b, d, None, _api.Identity(), sfa, sfb, (1, 1, 32), None, None, None, 'nk', False)
        cfg = L.GemmConfig()
        L.check(lib.dg_select_config(ctypes.byref(desc), ctypes.byref(cfg)))
        ws_bytes = lib.dg_gemm_workspace_bytes(ctypes.byref(desc), None)
        ws = _api._workspace(device, ws_bytes) if ws_bytes else None

        def once(events=None):
            L.check(lib.dg_l2_flush_launch(flush.data_ptr(), flush.numel(), sptr))
            if events:
                events[0].record(stream)
            L.check(lib.dg_gemm_launch(ctypes.byref(desc), None, ws.data_ptr() if ws is not None else None,
                                       ws.numel() if ws is not None else 0, sptr))
            if events:
                events[1].record(stream)

        for _ in range(max(args.warmup, 3)):
            once()
        torch.cuda.synchronize(device)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for e in ev:
            once(e)
        torch.cuda.synchronize(device)
        us = sum(a_.elapsed_time(b_) for a_, b_ in ev) / args.steps * 1e3
        nbytes = (m + n) * k // 2 + (m + n) * ((k + 63) // 64) * 2 + m * n * 2
        rows.append({'m': m, 'n': n, 'k': k, 'us': round(us, 2), 'tflops': round(2.0 * m * n * k / us / 1e6, 1),
                     'gbs': round(nbytes / us / 1e3, 1), 'tiling': cfg.as_dict()})
    if rank != 0:
        return
    flops = sum(2.0 * m * n * k for m, n, k in shapes)
    total_us = sum(r['us'] for r in rows)
    line = {'metric': 'fp4_block_scaled_gemm_tflops', 'value': world * flops / total_us / 1e6, 'unit': 'TFLOP/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': total_us / 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp4_e2m1 x fp4_e2m1, ue8m0 scales per 32 (kind::mxf4)',
            'data': 'synthetic',
            'config': {'workload': 'FP4xFP4 GEMM NT, BF16 out: ' + str(shapes), 'l2': 'flushed before every GEMM, untimed'},
            'shapes': rows, 'device_status': _api.device_status()}
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)


def run_quant(args, rank, world, device, emit=None):
    """The SwiGLU -> FP8 producer between the two expert GEMMs of the grouped workload: x [rows, 4096] BF16 (the
    output of the N = 4096 GEMM over 8 experts of about 8192 rows, psum layout) -> E4M3 [rows, 2048] + packed scales,
    and the plain cast of [rows, 7168] activations. HBM-bound; reported in GB/s of algorithmic bytes."""
    import deep_gemm
    from deep_gemm.testing import bench_events
    import json as _json
    peak = 6453.4
    try:
        import os
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', '..', '..', 'MEASURED_PEAKS.json')) as f:
            peak = float(_json.load(f)['hbm_gbs'])
    except (OSError, KeyError, ValueError):
        pass
    gen = torch.Generator(device=device).manual_seed(5 + rank)
    random.seed(1234 + rank)
    sizes = [int(random.uniform(0.7, 1.3) * 8192) for _ in range(8)]
    psum_list, rows = [], 0
    for s in sizes:
        psum_list.append(rows + s)
        rows = (rows + s + 255) // 256 * 256
    layout = torch.tensor(psum_list, dtype=torch.int32, device=device)
    valid = sum(sizes)
    out_rows = []
    x = torch.randn(rows, 4096, device=device, generator=gen).bfloat16()
    w = torch.rand(rows, device=device, generator=gen)
    p = bench_events(lambda: deep_gemm.swiglu_apply_weight_to_fp8(x, w, layout, None, 256), max(args.warmup, 3), args.steps)
    nbytes = valid * (4096 * 2 + 2048 + 2048 // 32 + 4)
    out_rows.append({'op': 'swiglu_apply_weight_to_fp8', 'rows': valid, 'hidden': 2048, 'us': round(p.dur_us, 2),
                     'gbs': round(nbytes / p.dur_us / 1e3, 1)})
    total_bytes, total_us = nbytes, p.dur_us
    del x
    x = torch.randn(rows, 7168, device=device, generator=gen).bfloat16()
    p = bench_events(lambda: deep_gemm.cast_to_fp8(x, layout, 256), max(args.warmup, 3), args.steps)
    nbytes = valid * (7168 * 2 + 7168 + 7168 // 32)
    out_rows.append({'op': 'cast_to_fp8', 'rows': valid, 'hidden': 7168, 'us': round(p.dur_us, 2),
                     'gbs': round(nbytes / p.dur_us / 1e3, 1)})
    total_bytes += nbytes
    total_us += p.dur_us
    if rank != 0:
        return
    achieved = total_bytes / total_us / 1e3
    line = {'metric': 'fp8_quantiser_gbs', 'value': world * achieved, 'unit': 'GB/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': total_us / 1e3, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'bf16 -> fp8_e4m3 + ue8m0 per 1x32', 'data': 'synthetic',
            'config': {'workload': 'SwiGLU->FP8 of [%d, 4096] and cast of [%d, 7168], 8 experts in psum layout' % (valid, valid),
                       'l2': 'flushed before every launch, untimed'},
            'roofline': {'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak,
                         'traffic': None, 'kernel': 'quant_fp8_kernel'},
            'ops': out_rows, 'device_status': _api.device_status()}
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)


def run_bf16(args, rank, world, device, emit=None):
    """BF16 GEMM "NT" (kind::f16, no scale factors), BF16 out, on three M = 4096 shapes of the dense sweep and one
    decode shape. Normalised by the measured BF16 burst figure."""
    lib = L.lib()
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    flush = l2_flush_buffer(device)
    gen = torch.Generator(device=device).manual_seed(13 + rank)
    shapes = [(4096, 7168, 16384), (4096, 4096, 7168), (4096, 7168, 2048), (128, 7168, 16384)]
    rows = []
    for (m, n, k) in shapes:
        a = torch.randn(m, k, device=device, generator=gen).bfloat16()
        b = torch.randn(n, k, device=device, generator=gen).bfloat16()
        d = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        desc = _api._run_gemm(L.GEMM_NORMAL, a, b, d, None, _api.Identity(), None, None, None, None, None, None, 'nk', False)
        cfg = L.GemmConfig()
        L.check(lib.dg_select_config(ctypes.byref(desc), ctypes.byref(cfg)))
        ws_bytes = lib.dg_gemm_workspace_bytes(ctypes.byref(desc), None)
        ws = _api._workspace(device, ws_bytes) if ws_bytes else None

        def once(events=None):
            L.check(lib.dg_l2_flush_launch(flush.data_ptr(), flush.numel(), sptr))
            if events:
                events[0].record(stream)
            L.check(lib.dg_gemm_launch(ctypes.byref(desc), None, ws.data_ptr() if ws is not None else None,
                                       ws.numel() if ws is not None else 0, sptr))
            if events:
                events[1].record(stream)

        for _ in range(max(args.warmup, 3)):
            once()
        torch.cuda.synchronize(device)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for e in ev:
            once(e)
        torch.cuda.synchronize(device)
        us = sum(a_.elapsed_time(b_) for a_, b_ in ev) / args.steps * 1e3
        nbytes = (m + n) * k * 2 + m * n * 2
        c = cfg.as_dict()
        rows.append({'m': m, 'n': n, 'k': k, 'us': round(us, 2), 'tflops': round(2.0 * m * n * k / us / 1e6, 1),
                     'gbs': round(nbytes / us / 1e3, 1), 'block_n': c['block_n'], 'cta_group': c['cta_group'],
                     'split_k': c['split_k'], 'stages': c['num_stages']})
    if rank != 0:
        return
    flops = sum(2.0 * m * n * k for m, n, k in shapes)
    total_us = sum(r['us'] for r in rows)
    line = {'metric': 'bf16_gemm_tflops', 'value': world * flops / total_us / 1e6, 'unit': 'TFLOP/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': total_us / 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16 x bf16, fp32 accumulate (kind::f16)', 'data': 'synthetic',
            'config': {'workload': 'BF16 GEMM NT, BF16 out: ' + str(shapes), 'l2': 'flushed before every GEMM, untimed'},
            'shapes': rows, 'device_status': _api.device_status()}
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)
