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


def grouped_config(world: int, g_total: int, masked: bool) -> dict:
    """The `config` object of the grouped workloads; the reference arm of the benchmark prints the same one."""
    return {'workload': ('m-grouped masked FP8 GEMM, %d experts x max_m 256, valid rows ~ U[0,256]' if masked else
                         'm-grouped contiguous FP8 GEMM (psum layout), %d experts in total, rows per expert ~ U(0.7,1.3) x 8192')
                        % g_total + ', (N,K) in ' + str(NK_LIST) + ', BF16 out',
            'sharding': 'experts in contiguous blocks over %d rank(s)%s, no data-path collective'
                        % (world, '' if masked else ', block boundaries balanced by rows'),
            'l2': 'flushed before every GEMM, untimed', 'flops': 'valid rows only'}


def grouped_sizes(g_total: int, masked: bool) -> list:
    """Rows per expert of the global problem: the same on every rank and in the reference arm."""
    random.seed(1234)
    if masked:
        return [random.randint(0, 256) for _ in range(g_total)]
    return [int(random.uniform(0.7, 1.3) * 8192) for _ in range(g_total)]


def _flush_timed(lib, device, launch, steps, warmup=3):
    """Mean microseconds of `launch(sptr)` over `steps` launches, each after an untimed write of a buffer larger
    than L2, one CUDA-event pair per launch."""
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    flush = l2_flush_buffer(device)
    for _ in range(warmup):
        L.check(lib.dg_l2_flush_launch(flush.data_ptr(), flush.numel(), sptr))
        launch(sptr)
    torch.cuda.synchronize(device)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in ev:
        L.check(lib.dg_l2_flush_launch(flush.data_ptr(), flush.numel(), sptr))
        e0.record(stream)
        launch(sptr)
        e1.record(stream)
    torch.cuda.synchronize(device)
    return sum(e0.elapsed_time(e1) for e0, e1 in ev) / steps * 1e3


class MixedCase:
    """FP8 x packed-FP4 GEMM "NN" (configuration 3): A [M, K] E4M3, B [K, N/2] packed E2M1 (uniform codes), per-32
    UE8M0 scales already in the required layout, BF16 out."""

    def __init__(self, device, seed=7, m=4096, n=7168, k=2048):
        gen = torch.Generator(device=device).manual_seed(seed)
        self.m, self.n, self.k = m, n, k
        self.a = _codes((m, k), device, gen)
        self.b = torch.randint(-128, 128, (k, n // 2), dtype=torch.int8, device=device, generator=gen)
        self.sfa = _scales((), m, k, device, gen)
        self.sfb = _scales((), n, k, device, gen)
        self.d = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        self.desc = _api._run_gemm(L.GEMM_NORMAL, self.a, self.b.transpose(0, 1), self.d, None, _api.Identity(), self.sfa,
                                   self.sfb, (1, 1, 32), None, None, None, 'nk', False)
        cfg = L.GemmConfig()
        L.check(L.lib().dg_select_config(ctypes.byref(self.desc), ctypes.byref(cfg)))
        self.config = cfg.as_dict()
        self.flops = 2.0 * m * n * k
        self.bytes = m * k + n * k // 2 + (m + n) * ((k + 63) // 64) * 2 + m * n * 2

    def launch(self, lib, sptr):
        L.check(lib.dg_gemm_launch(ctypes.byref(self.desc), None, None, 0, sptr))


def _graph_timed(lib, cases, steps) -> float:
    """Mean microseconds per launch of `cases` (same problem, operands of their own, together several times the L2
    capacity) launched back to back as one CUDA graph: the method the dense sweep's per-shape figures use."""
    from .bench import bench_graph
    return bench_graph([(lambda sptr, c=c: c.launch(lib, sptr)) for c in cases], 3, steps).dur_us


def time_mixed(device, steps: int, check=None) -> dict:
    lib = L.lib()
    cases = [MixedCase(device, seed=7 + i) for i in range(7)]           # 7 x 75 MB of operands and outputs
    us = _graph_timed(lib, cases, steps)
    case = cases[0]
    return {'us': us, 'tflops': case.flops / us / 1e6, 'gbs': case.bytes / us / 1e3, 'tiling': case.config,
            'verified': check(case) if check is not None else None}


def time_grouped(device, sizes, steps: int, masked: bool, check=None) -> dict:
    """Both (N, K) of the MoE configurations on one GPU for the given per-expert row counts."""
    lib = L.lib()
    shapes, flops, us_total, nbytes, ok = [], 0.0, 0.0, 0.0, True
    for i, (n, k) in enumerate(NK_LIST):
        case = GroupedCase(sizes, n, k, device, seed=100 + i, masked_max_m=256 if masked else 0)
        if masked:      # 100-200 us per launch: graph of three operand sets (0.5-1 GB each); the contiguous layout runs for milliseconds
            extra = [GroupedCase(sizes, n, k, device, seed=200 + 10 * i + j, masked_max_m=256) for j in range(2)]
            us = _graph_timed(lib, [case] + extra, steps)
            del extra
        else:
            us = _flush_timed(lib, device, lambda sptr: case.launch(lib, sptr), steps)
        ok = ok and (check(case, sizes, masked) if check is not None else True)
        shapes.append({'rows': case.rows, 'valid_rows': case.valid_rows, 'n': n, 'k': k, 'us': round(us, 1),
                       'tflops': round(case.flops / us / 1e6, 1), 'gbs': round(case.bytes / us / 1e3, 1),
                       'block_n': case.config['block_n'], 'cta_group': case.config['cta_group']})
        flops += case.flops
        nbytes += case.bytes
        us_total += us
        del case
        torch.cuda.empty_cache()
    return {'shapes': shapes, 'tflops': flops / us_total / 1e6, 'gbs': nbytes / us_total / 1e3,
            'verified': ok if check is not None else None}


def run(args, rank, world, device, emit=None, pk=None, checks=None):
    """`checks`: optional callables that compare a timed case with a reference on the host (the benchmark passes the
    CPU oracle's: 'mixed', 'grouped', 'dense_row', 'grouped_row'); without them the lines carry `verified: null`."""
    checks = checks or {}
    if args.workload == 'mixed':
        return run_mixed(args, rank, world, device, emit, checks.get('mixed'))
    if args.workload == 'fp4':
        return run_fp4(args, rank, world, device, emit)
    if args.workload == 'bf16':
        return run_bf16(args, rank, world, device, emit)
    if args.workload == 'quant':
        return run_quant(args, rank, world, device, emit)
    if args.workload == 'layout':
        return run_layout(args, rank, world, device, emit, pk)
    if args.workload == 'moe_mlp':
        return run_moe_mlp(args, rank, world, device, emit, checks.get('moe_mlp'))
    if args.workload == 'published':
        from .published_bench import run_published
        return run_published(args, rank, world, device, emit, checks.get('dense_row'), checks.get('grouped_row'))
    return run_grouped(args, rank, world, device, emit, pk or {'bf16_tflops': 1590.0, 'hbm_gbs': 6650.0, 'source': 'fallback'},
                       checks.get('grouped'))


def run_grouped(args, rank, world, device, emit, pk, check=None):
    """m-grouped contiguous (or masked) FP8 GEMM with a FIXED global expert count sharded over the ranks: every rank
    owns a contiguous block of experts (`sharding.expert_range`) and runs the single-GPU kernel on its local psum
    layout; nothing is exchanged on the data path. The NCCL all-gather of the outputs (equal, padded chunks) is timed
    on its own. The end-to-end leg copies the rank's A, B and scales from pinned host memory, calls the public API and
    copies D back, inside the timed region."""
    import deep_gemm
    from .sharding import balanced_expert_ranges, expert_range
    lib = L.lib()
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    flush = l2_flush_buffer(device)
    masked = args.workload == 'masked'
    g_total = getattr(args, 'experts', 0) or 32
    sizes = grouped_sizes(g_total, masked)  # the global problem is the same on every rank
    # contiguous blocks of experts: balanced by rows for the contiguous layout, by count for the masked one (whose cost
    # is the experts' B, the same for every expert)
    g0, g1 = expert_range(g_total, world, rank) if masked else balanced_expert_ranges(sizes, world)[rank]
    mine = sizes[g0:g1]
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

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
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
    verified = all(check(c, mine, masked, samples=2) for c in cases) if check is not None else None

    def reduce_max(x):
        t = torch.tensor([x], dtype=torch.float64, device=device)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(x):
        t = torch.tensor([x], dtype=torch.float64, device=device)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.SUM)
        return float(t.item())

    gemm_ms = reduce_max(sum(per_case_us) / 1e3)
    flops = reduce_sum(sum(c.flops for c in cases))
    nbytes = reduce_sum(sum(c.bytes for c in cases))
    verified = reduce_sum(0.0 if verified else 1.0) == 0.0

    # ---- the optional gather of the outputs, timed separately (both (N, K), one after the other)
    gather_ms = None
    if world > 1 and not getattr(args, 'no_gather', False):
        chunks, outs = [], []
        for c in cases:
            rows = int(reduce_max(float(c.rows)))
            chunk = torch.zeros(rows, c.n, dtype=torch.bfloat16, device=device)
            chunk[:c.rows].copy_(c.d.reshape(-1, c.n))
            chunks.append(chunk)
            outs.append(torch.empty(world * rows, c.n, dtype=torch.bfloat16, device=device))
        for out, chunk in zip(outs, chunks):
            torch.distributed.all_gather_into_tensor(out, chunk)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record(stream)
        for _ in range(reps):
            for out, chunk in zip(outs, chunks):
                torch.distributed.all_gather_into_tensor(out, chunk)
        e1.record(stream)
        barrier()
        gather_ms = reduce_max(e0.elapsed_time(e1) / reps)
        gathered_bytes = sum(o.numel() * 2 for o in outs)
        del chunks, outs

    # ---- end to end: host buffers -> device, the public API call, D back to the host
    hosts = []
    for c in cases:
        hosts.append({'a': c.a.view(torch.uint8).cpu().pin_memory(), 'b': c.b.view(torch.uint8).cpu().pin_memory(),
                      # (scales stay in the required layout: MN contiguous, so the host copy is of the transposed view)
                      'sfa': c.sfa.transpose(-2, -1).contiguous().cpu().pin_memory(),
                      'sfb': c.sfb.transpose(-2, -1).contiguous().cpu().pin_memory(),
                      'd': torch.empty(c.d.shape, dtype=torch.bfloat16).pin_memory()})
    sfa_dev = [torch.empty_like(c.sfa.transpose(-2, -1).contiguous()) for c in cases]
    sfb_dev = [torch.empty_like(c.sfb.transpose(-2, -1).contiguous()) for c in cases]
    h2d = sum(h['a'].numel() + h['b'].numel() + 2 * (h['sfa'].numel() + h['sfb'].numel()) for h in hosts)
    d2h = sum(h['d'].numel() * 2 for h in hosts)

    def e2e_step():
        for c, h, sa, sb in zip(cases, hosts, sfa_dev, sfb_dev):
            c.a.view(torch.uint8).copy_(h['a'], non_blocking=True)
            c.b.view(torch.uint8).copy_(h['b'], non_blocking=True)
            sa.copy_(h['sfa'], non_blocking=True)
            sb.copy_(h['sfb'], non_blocking=True)
            sa_t, sb_t = sa.transpose(-2, -1), sb.transpose(-2, -1)
            if masked:
                deep_gemm.m_grouped_fp8_gemm_nt_masked((c.a, sa_t), (c.b, sb_t), c.d, c.layout, max(1, c.valid_rows // len(mine)))
            else:
                deep_gemm.m_grouped_fp8_gemm_nt_contiguous((c.a, sa_t), (c.b, sb_t), c.d, c.layout)
            h['d'].copy_(c.d, non_blocking=True)

    e2e_step()
    barrier()
    import time
    e2e_steps = max(1, min(args.steps, 3))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = reduce_max((time.perf_counter() - t0) / e2e_steps)
    status = _api.device_status()
    if rank != 0:
        return
    value = flops / (gemm_ms * 1e-3) / 1e12
    fp8_peak = 2.0 * pk['bf16_tflops'] * world
    line = {
        'metric': 'fp8_block_scaled_gemm_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': warmup, 'ms_per_step': gemm_ms,
        'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None,
        'dtype': 'fp8_e4m3 x ue8m0, fp32 accumulate', 'data': 'synthetic',
        'config': grouped_config(world, g_total, masked),
        'verified': verified,
        'gemm_ms': gemm_ms, 'gather_ms': gather_ms,
        'gemm_plus_gather_ms': (gemm_ms + gather_ms) if gather_ms is not None else None,
        'roofline': ({'bound': 'hbm', 'achieved': nbytes / (gemm_ms * 1e-3) / 1e9, 'peak': pk['hbm_gbs'] * world, 'unit': 'GB/s',
                      'frac': nbytes / (gemm_ms * 1e-3) / 1e9 / (pk['hbm_gbs'] * world), 'traffic': None,
                      'peak_source': 'copy bandwidth of MEASURED_PEAKS.json x ranks (%s)' % pk['source']} if masked else
                     {'bound': 'tensor', 'achieved': value, 'peak': fp8_peak, 'unit': 'TFLOP/s', 'frac': value / fp8_peak,
                      'frac_of_nominal': value / (4500.0 * world), 'traffic': None,
                      'peak_source': '2 x the BF16 burst figure of MEASURED_PEAKS.json x ranks (%s): derived' % pk['source']}),
        'e2e': {'value': flops / e2e_s / 1e12, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
                'steps': e2e_steps, 'bytes_are': 'per rank (rank 0)'},
        'gpu_launches': int(launches), 'device_status': status,
        'shapes': [{'rows': c.rows, 'valid_rows': c.valid_rows, 'n': c.n, 'k': c.k, 'us': round(per_case_us[i], 1),
                    'tflops': round(c.flops / per_case_us[i] / 1e6, 1), 'gbs': round(c.bytes / per_case_us[i] / 1e3, 1),
                    'block_n': c.config['block_n'], 'cta_group': c.config['cta_group']} for i, c in enumerate(cases)],
        'shapes_are': 'rank 0',
    }
    if gather_ms is not None:
        line['gather_gbs_per_rank'] = gathered_bytes * (world - 1) / world / (gather_ms * 1e-3) / 1e9
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)


def run_mixed(args, rank, world, device, emit=None, check=None):
    """FP8 x packed-FP4 GEMM "NN": A [M,K] E4M3 with per-128 scales, B [K, N/2] packed E2M1 (uniform codes) with
    per-32 scales, BF16 out; M=4096, N=7168, K=2048. Normalised by the FP8 peak (the MMA runs on E4M3 operands)."""
    lib = L.lib()
    case = MixedCase(device, seed=7 + rank)
    us = _flush_timed(lib, device, lambda sptr: case.launch(lib, sptr), args.steps, max(args.warmup, 3))
    if rank != 0:
        return
    m, n, k = case.m, case.n, case.k
    line = {'metric': 'fp8_block_scaled_gemm_tflops', 'value': world * case.flops / us / 1e6, 'unit': 'TFLOP/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': us / 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp8_e4m3 x fp4_e2m1 (kind::mxf8f6f4), ue8m0 scales',
            'data': 'synthetic',
            'config': {'workload': 'mixed FP8xFP4 GEMM NN, M=%d N=%d K=%d, BF16 out' % (m, n, k), 'l2': 'flushed, untimed'},
            'gbs': case.bytes / us / 1e3, 'tiling': case.config, 'verified': check(case) if check is not None else None,
            'device_status': _api.device_status()}
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


class ExpertMlpCase:
    """The expert MLP of an MoE layer as the reference's unfused baseline runs it (tests/test_mega_moe.py:139-145): an
    m-grouped FP8 x FP4 GEMM to 2 * intermediate columns, SwiGLU with the routing weight applied and quantised to E4M3
    with per-32 scales, a second m-grouped FP8 x FP4 GEMM back to `hidden` columns. Tokens sit on the 256-row psum
    layout; every call goes through the public API."""

    def __init__(self, sizes, hidden: int, intermediate: int, device, seed: int):
        gen = torch.Generator(device=device).manual_seed(seed)
        self.sizes, self.hidden, self.intermediate, g = list(sizes), hidden, intermediate, len(sizes)
        local = shard_psum_layout(self.sizes, 1, 0)
        self.rows, self.valid_rows = local['rows'], sum(sizes)
        self.x = _codes((self.rows, hidden), device, gen)
        self.sfx = _scales((), self.rows, hidden, device, gen)
        self.w1 = torch.randint(-128, 128, (g, 2 * intermediate, hidden // 2), dtype=torch.int8, device=device, generator=gen)
        self.sfw1 = _scales((g,), 2 * intermediate, hidden, device, gen)
        self.w2 = torch.randint(-128, 128, (g, hidden, intermediate // 2), dtype=torch.int8, device=device, generator=gen)
        self.sfw2 = _scales((g,), hidden, intermediate, device, gen)
        self.topk_weights = torch.rand(self.rows, device=device, generator=gen) + 0.25
        self.layout = torch.tensor(local['psum'], dtype=torch.int32, device=device)
        self.y1 = torch.empty(self.rows, 2 * intermediate, dtype=torch.bfloat16, device=device)
        self.y2 = torch.empty(self.rows, hidden, dtype=torch.bfloat16, device=device)
        self.a2 = self.sfa2 = None
        self.flops = 2.0 * self.valid_rows * (2 * intermediate * hidden + hidden * intermediate)
        k64 = lambda k: (k + 63) // 64                                                  # noqa: E731
        self.bytes = (self.valid_rows * (hidden + k64(hidden) * 2 + 2 * intermediate * 2)               # GEMM 1: A, SFA, D
                      + g * 2 * intermediate * (hidden // 2 + k64(hidden) * 2)                         #         B, SFB
                      + self.valid_rows * (2 * intermediate * 2 + 4 + intermediate + k64(intermediate) * 2)   # SwiGLU: in, weight, out, scales
                      + self.valid_rows * (intermediate + k64(intermediate) * 2 + hidden * 2)         # GEMM 2: A, SFA, D
                      + g * hidden * (intermediate // 2 + k64(intermediate) * 2))                      #         B, SFB

    def run(self):
        import deep_gemm
        deep_gemm.m_grouped_fp8_fp4_gemm_nt_contiguous((self.x, self.sfx), (self.w1, self.sfw1), self.y1, self.layout)
        self.a2, self.sfa2 = deep_gemm.swiglu_apply_weight_to_fp8(self.y1, self.topk_weights, self.layout, expert_alignment=256)
        deep_gemm.m_grouped_fp8_fp4_gemm_nt_contiguous((self.a2, self.sfa2), (self.w2, self.sfw2), self.y2, self.layout)


def run_moe_mlp(args, rank, world, device, emit=None, check=None):
    """`--workload moe_mlp`: 8 experts of about 8192 tokens, hidden 7168, intermediate 2048 (the two (N, K) of the grouped
    configuration are exactly this layer's two GEMMs). One step = the three launches; an untimed L2 flush before each
    step, one CUDA-event pair around it."""
    lib = L.lib()
    stream = torch.cuda.current_stream(device)
    flush = l2_flush_buffer(device)
    sizes = grouped_sizes(8, False)
    case = ExpertMlpCase(sizes, 7168, 2048, device, seed=31 + rank)
    for _ in range(max(args.warmup, 3)):
        case.run()
    torch.cuda.synchronize(device)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    launches0 = lib.dg_kernel_launch_count()
    for e0, e1 in ev:
        L.check(lib.dg_l2_flush_launch(flush.data_ptr(), flush.numel(), stream.cuda_stream))
        e0.record(stream)
        case.run()
        e1.record(stream)
    torch.cuda.synchronize(device)
    launches = lib.dg_kernel_launch_count() - launches0               # (the flush kernel is not counted)
    ms = sum(e0.elapsed_time(e1) for e0, e1 in ev) / args.steps
    if rank != 0:
        return
    line = {'metric': 'fp8_block_scaled_gemm_tflops', 'value': world * case.flops / ms / 1e9, 'unit': 'TFLOP/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': ms, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'fp8_e4m3 x fp4_e2m1, ue8m0 scales, bf16 between the GEMMs', 'data': 'synthetic',
            'config': {'workload': 'MoE expert MLP, 8 experts, %d tokens on the 256-row psum layout, hidden 7168, intermediate 2048: '
                                   'm-grouped FP8xFP4 GEMM -> SwiGLU * routing weight -> FP8 (per-32 scales) -> m-grouped FP8xFP4 GEMM'
                                   % case.valid_rows, 'l2': 'flushed before every step, untimed'},
            'gbs': case.bytes / ms / 1e6, 'gpu_launches': int(launches),
            'verified': check(case) if check is not None else None, 'device_status': _api.device_status()}
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)


def run_layout(args, rank, world, device, emit=None, pk=None):
    """Scale-factor relayout (`transform_sf_into_required_layout`) on large cases of the reference's layout
    performance list (tests/generators.py:725-747): batched FP32 scales [8, 32768, K/32], an m-grouped psum layout of
    262144 rows in 128 groups, per-row, per-32-row and per-128-row granularity, FP32 and packed int16 sources, K- and
    MN-major. HBM-bound: bytes = source read + int16 result written."""
    import deep_gemm
    from .bench import bench_events
    peak = (pk or {}).get('hbm_gbs', 6453.4)
    gen = torch.Generator(device=device).manual_seed(3 + rank)
    rows_out, total_bytes, total_us = [], 0.0, 0.0
    batches, batch_mn, k = 8, 32768, 7168
    total_mn = batches * batch_mn
    group_sizes = [total_mn // 128 - 1] * 128
    psum, acc = [], 0
    for sz in group_sizes:
        psum.append(acc + sz)
        acc = (acc + sz + 255) // 256 * 256
    layout = torch.tensor(psum, dtype=torch.int32, device=device)
    cases = []
    for gran in (1, 32, 128):
        cases.append(('batched fp32 K-major gran_mn=%d' % gran, torch.float32, False, gran, None))
    cases.append(('m-grouped (128 groups) fp32 K-major gran_mn=1', torch.float32, False, 1, layout))
    cases.append(('m-grouped (128 groups) fp32 MN-major gran_mn=1', torch.float32, True, 1, layout))
    cases.append(('m-grouped (128 groups) int16 K-major gran_mn=1', torch.int16, False, 1, layout))
    for name, dtype, mn_major, gran, lay in cases:
        cols = k // 32 if dtype == torch.float32 else k // 64
        lead = (batches, batch_mn // gran) if lay is None else (total_mn // gran,)
        if dtype == torch.float32:
            src = (torch.randint(100, 140, (*lead, cols), dtype=torch.int32, device=device, generator=gen) << 23).view(torch.float32)
        else:
            src = torch.randint(0, 32000, (*lead, cols), dtype=torch.int16, device=device, generator=gen)
        if mn_major:
            src = src.transpose(-2, -1).contiguous().transpose(-2, -1)
        mn = batch_mn if lay is None else total_mn

        def fn():
            return deep_gemm.transform_sf_into_required_layout(src, mn, k, (gran, gran, 32), batches if lay is None else None,
                                                               True, False, lay)
        out = fn()
        p = bench_events(fn, max(args.warmup, 3), args.steps)
        nbytes = src.numel() * src.element_size() + out.numel() * 2
        rows_out.append({'case': name, 'us': round(p.dur_us, 1), 'gbs': round(nbytes / p.dur_us / 1e3, 1),
                         'mb': round(nbytes / 1e6, 1)})
        total_bytes += nbytes
        total_us += p.dur_us
        del src, out
    if rank != 0:
        return
    achieved = total_bytes / total_us / 1e3
    line = {'metric': 'sf_transform_gbs', 'value': world * achieved, 'unit': 'GB/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': max(args.warmup, 3), 'ms_per_step': total_us / 1e3, 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': 'u8 (UE8M0 exponent bytes)', 'data': 'synthetic',
            'config': {'workload': 'transform_sf_into_required_layout, 262144 rows x K=7168, six large cases of the '
                                   "reference's layout performance list", 'l2': 'flushed before every launch, untimed'},
            'roofline': {'bound': 'hbm', 'achieved': achieved, 'peak': peak, 'unit': 'GB/s', 'frac': achieved / peak,
                         'traffic': None, 'kernel': 'transform_sf_kernel'},
            'cases': rows_out, 'device_status': _api.device_status()}
    (emit or (lambda l: print(json.dumps(l), flush=True)))(line)
