"""Benchmark of the block-scaled FP8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload auto|dense|grouped|masked|mixed|fp4|bf16|quant|layout|published|moe_mlp]

One GPU (`--workload auto` = `dense`): one "step" is one pass over the dense FP8 NT sweep the baseline names: M in
{64, 128, 4096} times six (N, K) pairs, BF16 output, A quantised per 1x128 and B per 128x128 from N(0,1) data
(synthetic, seeded). Every GEMM has its own operands, so a step touches about 1.5 GB and no launch finds its inputs
in L2. The K steps are K replays of a CUDA graph of the 18 launches between one CUDA-event pair (`value`). Per-shape
times, and the two roofline figures built from them, come from a second measurement in which every shape is launched
back to back on rotating operand sets (again larger than L2) as a graph of its own. The same line carries short legs
for the other three configurations (mixed FP8xFP4, m-grouped contiguous with 32 experts, m-grouped masked), each with
its own roofline, a leg over every row of the reference's own published tables (`--workload published` alone), `e2e` (the sweep through the public Python API from pinned host buffers, copies inside the timed
region), `cpu_baseline` (the CPU oracle on the host cores over the same 18 shapes) and `verified`: after the timed
region a row sample of every output is compared with the CPU oracle.

Several GPUs (torchrun, one rank per GPU; `--workload auto` = `grouped`): the m-grouped contiguous GEMM with a fixed
global expert count sharded over the ranks (strong scaling), no collective on the data path; the NCCL all-gather of
the outputs is timed separately (`gather_ms`). `--workload dense` at N > 1 runs N independent N-slabs instead.

`--impl reference` times the reference's CPU implementation of the path (its dequantise-then-matmul test oracle) on
the host cores on the workload this build's arm runs with the same arguments: the same 18 shapes on one GPU, a bounded
sample of the same sharded grouped problem (and the same `config` object) with `--gpus N`, N > 1.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, 'deepgemm-ascend_b200'))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

NK_LIST = [(2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]
M_LIST = [64, 128, 4096]
SWEEP = [(m, n, k) for m in M_LIST for (n, k) in NK_LIST]
FP8_MAX = 448.0
NOMINAL_FP8_TFLOPS, NOMINAL_HBM_GBS = 4500.0, 8000.0
GLOBAL_EXPERTS = 32

DENSE_WORKLOAD = ('dense FP8 NT sweep: M in {64,128,4096} x (N,K) in ' + str(NK_LIST) +
                  ', BF16 out, A scaled per 1x128, B per 128x128 (UE8M0)')

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of single launches taken from ncu captures of this
# library, keyed by (m, n, k, block_n): reported as `roofline.traffic` only when the launch timed here uses the same
# tiling as the captured one, otherwise null.
NCU_DRAM_TRAFFIC = {(4096, 7168, 16384, 448): 489.5e6, (4096, 7168, 16384, 320): 513.0e6, (4096, 7168, 16384, 224): 558.0e6}


def peaks() -> dict:
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return {'hbm_gbs': p['hbm_gbs'], 'bf16_tflops': p['bf16_tflops'],
                'bf16_tflops_sustained': p.get('bf16_tflops_sustained', p['bf16_tflops']), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0, 'source': 'fallback'}


def measure_write_bandwidth(device) -> float:
    """GB/s of a pure write stream on this GPU (a 1 GiB fill, best of 5, CUDA events): HBM takes writes at roughly
    half the rate of the read+write copy that MEASURED_PEAKS.json records, which is what bounds a GEMM whose output
    is most of its traffic (4096 x 32768 x 512: 268 MB of D against 19 MB of operands)."""
    buf = torch.empty(1 << 30, dtype=torch.uint8, device=device)
    best = float('inf')
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        buf.fill_(1)
        e1.record()
        torch.cuda.synchronize(device)
        best = min(best, e0.elapsed_time(e1))
    del buf
    return (1 << 30) / best / 1e6


def dense_config(world: int) -> dict:
    """The `config` object of the dense workload; the reference arm prints the same one."""
    return {'workload': DENSE_WORKLOAD,
            'l2': 'inputs larger than L2: every GEMM has its own operands (1.5 GB per step against 126 MB of L2)',
            'sharding': 'none' if world == 1 else 'N-slabs, one per rank, no collective'}


# ----------------------------------------------------------------------------------------------------------------
# Synthetic inputs (generated with torch on the device: plumbing, not the measured path)
# ----------------------------------------------------------------------------------------------------------------
def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    bits = x.abs().float().view(torch.int32)
    exp = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).int()
    return (exp.clamp(1, 254) << 23).view(torch.float32)


def quantize_fp8(x: torch.Tensor, gran: tuple[int, int]):
    """x [MN, K] fp32 -> (e4m3 [MN, K], fp32 scales [ceil(MN/gm), ceil(K/gk)]); same rule as the reference's
    quantize_with_major (tests/generators.py:61-95)."""
    mn, k = x.shape
    gm, gk = gran
    pm, pk = -(-mn // gm) * gm, -(-k // gk) * gk
    padded = torch.zeros(pm, pk, dtype=torch.float32, device=x.device)
    padded[:mn, :k] = x
    amax = padded.view(pm // gm, gm, pk // gk, gk).abs().amax(dim=(1, 3))
    sf = ceil_to_ue8m0(amax.clamp(1e-4) / FP8_MAX)
    full = sf.repeat_interleave(gm, 0).repeat_interleave(gk, 1)[:mn, :k]
    return (x / full).to(torch.float8_e4m3fn), sf.contiguous()


def dense_bytes(m, n, k) -> int:
    k64 = -(-k // 64)
    return m * k + n * k + (m + n) * k64 * 2 + m * n * 2


class DenseCase:
    """One (M, N, K) problem with operands on the device, canonical scale factors, and a prepared C-ABI call."""

    def __init__(self, m, n, k, device, seed, data=None):
        import deep_gemm
        from deep_gemm import _api
        g = torch.Generator(device=device).manual_seed(seed)
        self.m, self.n, self.k = m, n, k
        if data is None:
            self.a, self.sfa32 = quantize_fp8(torch.randn(m, k, device=device, generator=g), (1, 128))
            self.b, self.sfb32 = quantize_fp8(torch.randn(n, k, device=device, generator=g), (128, 128))
        else:       # another operand set of the same shape: codes and scales drawn directly (timing only)
            self.a = torch.randint(0, 120, (m, k), dtype=torch.uint8, device=device, generator=g).view(torch.float8_e4m3fn)
            self.b = torch.randint(0, 120, (n, k), dtype=torch.uint8, device=device, generator=g).view(torch.float8_e4m3fn)
            self.sfa32 = torch.ones(m, k // 128, device=device)
            self.sfb32 = torch.ones(-(-n // 128), k // 128, device=device)
        self.d = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        # scale factors already in the required layout: the kernel-only number excludes the relayout
        self.sfa = deep_gemm.transform_sf_into_required_layout(self.sfa32, m, k, (1, 128, 128), is_sfa=True)
        self.sfb = deep_gemm.transform_sf_into_required_layout(self.sfb32, n, k, (1, 128, 128), is_sfa=False)
        self.desc = _api._run_gemm(_api.L.GEMM_NORMAL, self.a, self.b, self.d, None, _api.Identity(), self.sfa, self.sfb,
                                   (1, 1, 32), None, None, None, 'nk', False)
        self.flops = 2.0 * m * n * k
        self.bytes = dense_bytes(m, n, k)
        self.ws = None
        lib = _api.L.lib()
        ws_bytes = lib.dg_gemm_workspace_bytes(ctypes.byref(self.desc), None)
        if ws_bytes:
            self.ws = _api._workspace(self.d.device, ws_bytes)
        cfg = _api.L.GemmConfig()
        _api.L.check(lib.dg_select_config(ctypes.byref(self.desc), ctypes.byref(cfg)))
        self.config = cfg.as_dict()

    def launch(self, lib, stream_ptr):
        rc = lib.dg_gemm_launch(ctypes.byref(self.desc), None, self.ws.data_ptr() if self.ws is not None else None,
                                self.ws.numel() if self.ws is not None else 0, stream_ptr)
        if rc != 0:
            raise RuntimeError(lib.dg_last_error().decode())

    def pin_host_copies(self):
        self.h_a = self.a.view(torch.uint8).cpu().pin_memory()
        self.h_b = self.b.view(torch.uint8).cpu().pin_memory()
        self.h_sfa = self.sfa32.cpu().pin_memory()
        self.h_sfb = self.sfb32.cpu().pin_memory()
        self.h_d = torch.empty(self.m, self.n, dtype=torch.bfloat16).pin_memory()
        self.h2d = self.h_a.numel() + self.h_b.numel() + 4 * (self.h_sfa.numel() + self.h_sfb.numel())
        self.d2h = self.h_d.numel() * 2

    def verify(self, rows: int = 16) -> bool:
        """A row sample of D against the CPU oracle (dequantise, FP32 matmul, one cast), within the parity tolerance."""
        import oracle
        idx = torch.randperm(self.m, generator=torch.Generator().manual_seed(self.m + self.n))[:rows].sort().values
        a_deq = oracle.dequantize(oracle.decode_e4m3(self.a[idx.to(self.a.device)].cpu()), self.sfa32.cpu()[idx], 1, 128)
        b_deq = oracle.dequantize(oracle.decode_e4m3(self.b.cpu()), self.sfb32.cpu(), 128, 128)
        ref = oracle.gemm_ref(a_deq, b_deq, torch.bfloat16)
        out = self.d[idx.to(self.d.device)].cpu()
        return bool(torch.isfinite(out.float()).all()) and oracle.calc_diff(out, ref) <= 1e-3 and \
            oracle.max_rel_err(out, ref) <= 2e-2


# ----------------------------------------------------------------------------------------------------------------
# Clock sampling during the timed region
# ----------------------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index: int):
        self.samples, self.proc = [], None
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={gpu_index}', f'--query-gpu={self.FIELDS}',
                                          '--format=csv,noheader,nounits', '-lms', '20'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        reasons = set()
        for s in self.samples:
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), s[2:]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': sm[len(sm) // 2] if sm else None,
                'sm_max_mhz': int(self.samples[0][1]) if self.samples and self.samples[0][1].isdigit() else None,
                'samples': len(sm), 'reasons': sorted(reasons)}


# ----------------------------------------------------------------------------------------------------------------
# CPU baseline: the reference's dequantise-then-matmul oracle on the host cores
# ----------------------------------------------------------------------------------------------------------------
CPU_SAMPLE_TEXT = 'dequantise + FP32 matmul + BF16 cast (torch CPU) of all 18 shapes of the sweep, inputs quantised before the clock starts'


def cpu_inputs(shapes):
    """Quantised operands of `shapes` on the host (seeded), B shared by the shapes with the same (N, K)."""
    import oracle
    torch.manual_seed(0)
    weights, out = {}, []
    for (m, n, k) in shapes:
        if (n, k) not in weights:
            b, sfb, _ = oracle.quantize_e4m3(torch.randn(n, k), (128, 128))
            weights[(n, k)] = (b, sfb)
        a, sfa, _ = oracle.quantize_e4m3(torch.randn(m, k), (1, 128))
        out.append((a, sfa) + weights[(n, k)])
    return out


def cpu_oracle_pass(inputs) -> tuple[float, float]:
    """One pass of the oracle over prepared inputs: (flops, seconds). Only dequantise + matmul + cast is timed."""
    import oracle
    flops = 0.0
    t0 = time.perf_counter()
    for (a, sfa, b, sfb) in inputs:
        a_deq = oracle.dequantize(oracle.decode_e4m3(a), sfa, 1, 128)
        b_deq = oracle.dequantize(oracle.decode_e4m3(b), sfb, 128, 128)
        oracle.gemm_ref(a_deq, b_deq, torch.bfloat16)
        flops += 2.0 * a.shape[0] * b.shape[0] * a.shape[1]
    return flops, time.perf_counter() - t0


def run_reference_grouped(args, world, masked: bool):
    """The grouped workload of the multi-GPU arm on the host cores: the oracle (dequantise per 1x32 + FP32 matmul + BF16
    cast) over a bounded sample of the same global problem: every eighth expert, its first 1024 valid rows (all valid
    rows of a masked expert), both (N, K). Operands are drawn before the clock starts."""
    import oracle
    from deep_gemm.testing import moe_bench
    g_total = args.experts or GLOBAL_EXPERTS
    sizes = moe_bench.grouped_sizes(g_total, masked)
    torch.manual_seed(0)
    table = torch.tensor([2.0 ** -9, 2.0 ** -8, 2.0 ** -7])
    inputs = []
    for (n, k) in moe_bench.NK_LIST:
        for g in range(0, g_total, 8):
            rows = min(sizes[g], 1024)
            if rows == 0:
                continue
            def operand(mn):
                raw = torch.randint(0, 254, (mn, k), dtype=torch.uint8)
                raw += (raw >= 0x7F).to(torch.uint8)
                return raw.view(torch.float8_e4m3fn), table[torch.randint(0, 3, (mn, k // 32))].contiguous()
            inputs.append(operand(rows) + operand(n))

    def one_pass():
        flops, t0 = 0.0, time.perf_counter()
        for (a, sfa, b, sfb) in inputs:
            oracle.gemm_ref(oracle.dequantize(oracle.decode_e4m3(a), sfa, 1, 32), oracle.dequantize(oracle.decode_e4m3(b), sfb, 1, 32),
                            torch.bfloat16)
            flops += 2.0 * a.shape[0] * b.shape[0] * a.shape[1]
        return flops, time.perf_counter() - t0

    for _ in range(min(args.warmup, 1)):
        one_pass()
    flops = seconds = 0.0
    for _ in range(args.steps):
        f, s = one_pass()
        flops += f
        seconds += s
    value = flops / seconds / 1e12
    sample = ('dequantise + FP32 matmul + BF16 cast (torch CPU) of every eighth expert, first 1024 valid rows, both (N, K): '
              '%.2f TFLOP per step of the %.1f TFLOP problem, operands drawn before the clock starts'
              % (flops / args.steps / 1e12, sum(2.0 * sum(sizes) * n * k for n, k in moe_bench.NK_LIST) / 1e12))
    emit({
        'impl': 'reference', 'metric': 'fp8_block_scaled_gemm_tflops', 'value': value, 'unit': 'TFLOP/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': seconds / args.steps * 1e3,
        'higher_is_better': True, 'scaling': 'strong', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': moe_bench.grouped_config(world, g_total, masked),
        'cpu_baseline': {'value': value, 'unit': 'TFLOP/s', 'cores': torch.get_num_threads(), 'kind': 'port', 'sample': sample},
        'e2e': {'value': value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    })


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path (its test oracle) on this box's host cores, on the workload this
    build's arm runs with the same arguments: the dense sweep on one GPU, the sharded grouped GEMM on several."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    ranks = max(world, args.gpus)
    workload = args.workload if args.workload != 'auto' else ('dense' if ranks == 1 else 'grouped')
    if workload in ('grouped', 'masked'):
        return run_reference_grouped(args, ranks, workload == 'masked')
    inputs = cpu_inputs(SWEEP)
    for _ in range(min(args.warmup, 1)):
        cpu_oracle_pass(inputs[:6])
    flops, seconds = 0.0, 0.0
    for _ in range(args.steps):
        f, s = cpu_oracle_pass(inputs)
        flops += f
        seconds += s
    value = flops / seconds / 1e12
    emit({
        'impl': 'reference', 'metric': 'fp8_block_scaled_gemm_tflops', 'value': value, 'unit': 'TFLOP/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': seconds / args.steps * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': dense_config(1),
        'cpu_baseline': {'value': value, 'unit': 'TFLOP/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                         'sample': CPU_SAMPLE_TEXT},
        'e2e': {'value': value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    })


# ----------------------------------------------------------------------------------------------------------------
# Dense sweep
# ----------------------------------------------------------------------------------------------------------------
def per_shape_times(lib, device, base_cases, use_graph=True) -> list[float]:
    """Mean microseconds per launch of every shape of the sweep: each shape runs as a CUDA graph of back-to-back
    launches over rotating operand sets that together exceed L2 several times, between one CUDA-event pair.
    Without graphs (`--no-graph`, for profilers): the same launches on the stream, one event pair around them."""
    from deep_gemm.testing import bench_graph
    out = []
    for ci, c in enumerate(base_cases):
        copies = max(3, min(32, -(-512_000_000 // c.bytes)))
        sets = [c] + [DenseCase(c.m, c.n, c.k, device, seed=7000 + 37 * ci + j, data='codes') for j in range(copies - 1)]
        if use_graph:
            out.append(bench_graph([(lambda sptr, s=s: s.launch(lib, sptr)) for s in sets], 3, 10).dur_us)
        else:
            stream = torch.cuda.current_stream(device)
            for s in sets:
                s.launch(lib, stream.cuda_stream)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(3):
                for s in sets:
                    s.launch(lib, stream.cuda_stream)
            e1.record(stream)
            torch.cuda.synchronize(device)
            out.append(e0.elapsed_time(e1) * 1e3 / (3 * len(sets)))
        del sets
    return out


def copies_of_same_bytes(device, base_cases) -> dict:
    """For every few-rows shape: microseconds per copy when device-to-device copies that move the same number of bytes
    (half read, half written) run back to back in a graph over rotating buffers, exactly like the GEMM launches of
    `per_shape_times`. A launch that moves 16-45 MB cannot reach the bandwidth of a long copy: this is what a plain copy
    of that size achieves on this box, start-up and tail included."""
    from deep_gemm.testing import bench_graph
    out = {}
    for c in base_cases:
        if c.m > 128:
            continue
        half = c.bytes // 2
        copies = max(3, min(32, -(-512_000_000 // c.bytes)))
        bufs = [(torch.empty(half, dtype=torch.uint8, device=device), torch.empty(half, dtype=torch.uint8, device=device))
                for _ in range(copies)]
        for src, _ in bufs:
            src.zero_()
        out[(c.m, c.n, c.k)] = bench_graph([(lambda sptr, sd=sd: sd[1].copy_(sd[0])) for sd in bufs], 3, 10).dur_us
        del bufs
    return out


def run_dense(args, rank, world, device):
    import deep_gemm
    from deep_gemm import _lib as L
    lib = L.lib()
    pk = peaks()
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    cases = [DenseCase(m, n, k, device, seed=1000 * rank + i) for i, (m, n, k) in enumerate(SWEEP)]
    torch.cuda.synchronize(device)

    # One step = the 18 GEMMs back to back. Every GEMM has its own operands and the sweep touches far more than the
    # L2 holds between two uses of the same buffer, so every launch finds its inputs in HBM without a flush kernel.
    footprint = sum(c.bytes for c in cases)
    l2_bytes = torch.cuda.get_device_properties(device).L2_cache_size
    assert footprint > 4 * l2_bytes, 'the sweep must not fit in L2'

    def sweep(stream_ptr):
        for c in cases:
            c.launch(lib, stream_ptr)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        sweep(sptr)
    barrier()
    # The step as a CUDA graph (launch-bound for the small shapes otherwise); plain stream launches if capture fails.
    graph, launches_per_step = None, 0
    try:
        if args.no_graph:
            raise RuntimeError('--no-graph')
        side = torch.cuda.Stream(device)
        graph = torch.cuda.CUDAGraph()
        launches0 = lib.dg_kernel_launch_count()
        with torch.cuda.graph(graph, stream=side):
            sweep(torch.cuda.current_stream(device).cuda_stream)
        launches_per_step = lib.dg_kernel_launch_count() - launches0
    except Exception as exc:      # noqa: BLE001 - any capture problem falls back to plain launches
        print(f'bench: graph capture failed ({exc}); timing plain stream launches', file=sys.stderr)
        graph = None
        torch.cuda.synchronize(device)

    def step():
        if graph is not None:
            graph.replay()
        else:
            sweep(sptr)

    # (the clock sampler also sees the warm-up replays: the timed region alone lasts only some tens of milliseconds)
    sampler = ClockSampler(device.index) if rank == 0 else None
    for _ in range(warmup):
        step()
    barrier()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.dg_kernel_launch_count()
    t_begin.record(stream)
    for _ in range(args.steps):
        step()
    t_end.record(stream)
    barrier()
    launches = launches_per_step * args.steps if graph is not None else lib.dg_kernel_launch_count() - launches0
    step_ms = t_begin.elapsed_time(t_end) / args.steps
    verified = all(c.verify() for c in cases) if rank == 0 else None

    # Per-shape times and the roofline figures
    per_case_us = per_shape_times(lib, device, cases, use_graph=graph is not None)
    copy_us = copies_of_same_bytes(device, cases) if rank == 0 and graph is not None else {}
    barrier()
    clocks = sampler.stop() if sampler else None
    status = deep_gemm.device_status()

    step_ms_t = torch.tensor([step_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(step_ms_t, op=torch.distributed.ReduceOp.MAX)
    step_ms_max = float(step_ms_t.item())
    flops_step = sum(c.flops for c in cases)
    value = world * flops_step / (step_ms_max * 1e-3) / 1e12

    # ---- end to end through the public API, host buffers, copies inside the timed region
    for c in cases:
        c.pin_host_copies()
    e2e_steps = max(1, min(args.steps, 5))

    # Three streams so that the PCIe link runs in both directions while the GPU computes: inputs of shape i+1 go up
    # while shape i is multiplied and the result of shape i-1 comes down. Every byte still crosses inside the timed
    # region, and each GEMM is the public API call on host-provided data.
    s_in, s_mm, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device)
    done_mm = [None] * len(cases)      # last GEMM that read case i's device inputs / wrote its D
    done_out = [None] * len(cases)     # last D2H copy of case i's D
    host_us = []

    def e2e_step():
        for i, c in enumerate(cases):
            with torch.cuda.stream(s_in):
                if done_mm[i] is not None:
                    s_in.wait_event(done_mm[i])          # do not overwrite inputs a previous GEMM still reads
                c.a.view(torch.uint8).copy_(c.h_a, non_blocking=True)
                c.b.view(torch.uint8).copy_(c.h_b, non_blocking=True)
                c.sfa32.copy_(c.h_sfa, non_blocking=True)
                c.sfb32.copy_(c.h_sfb, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            with torch.cuda.stream(s_mm):
                s_mm.wait_event(ready)
                if done_out[i] is not None:
                    s_mm.wait_event(done_out[i])         # D is still being copied out from the previous step
                h0 = time.perf_counter()
                deep_gemm.fp8_gemm_nt((c.a, c.sfa32), (c.b, c.sfb32), c.d, recipe=(1, 128, 128))
                host_us.append((time.perf_counter() - h0) * 1e6)
                done_mm[i] = torch.cuda.Event()
                done_mm[i].record(s_mm)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done_mm[i])
                c.h_d.copy_(c.d, non_blocking=True)
                done_out[i] = torch.cuda.Event()
                done_out[i].record(s_out)

    e2e_step()
    barrier()
    host_us.clear()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = torch.tensor([(time.perf_counter() - t0) / e2e_steps], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(e2e_s, op=torch.distributed.ReduceOp.MAX)
    e2e_value = world * flops_step / float(e2e_s.item()) / 1e12
    # host cost of one GEMM call with scale factors already in the required layout (no transform launched)
    c0 = cases[6]
    for _ in range(20):
        deep_gemm.fp8_gemm_nt((c0.a, c0.sfa), (c0.b, c0.sfb), c0.d)
    h0 = time.perf_counter()
    for _ in range(200):
        deep_gemm.fp8_gemm_nt((c0.a, c0.sfa), (c0.b, c0.sfb), c0.d)
    host_call_us = (time.perf_counter() - h0) / 200 * 1e6
    torch.cuda.synchronize(device)

    if rank != 0:
        return
    legs = other_config_legs(args, device, pk) if world == 1 and not args.no_legs and not args.no_graph else None

    big = [i for i, c in enumerate(cases) if c.m == 4096]
    small = [i for i, c in enumerate(cases) if c.m <= 128]
    tf_big = sum(cases[i].flops for i in big) / sum(per_case_us[i] for i in big) / 1e6
    gbs_small = sum(cases[i].bytes for i in small) / sum(per_case_us[i] for i in small) / 1e3
    # the same twelve byte counts as plain device-to-device copies, launched and timed the same way
    gbs_copies = (sum(cases[i].bytes for i in small) / sum(copy_us[(cases[i].m, cases[i].n, cases[i].k)] for i in small) / 1e3
                  if copy_us else None)
    fp8_peak = 2.0 * pk['bf16_tflops']
    top = max(big, key=lambda i: cases[i].flops)
    write_gbs = measure_write_bandwidth(device)

    def roofs(c, us):
        # the three lower bounds of one launch, in microseconds, and the fraction of the tightest one that was reached
        floors = {'tensor': c.flops / fp8_peak / 1e6, 'hbm': c.bytes / pk['hbm_gbs'] / 1e3,
                  'hbm_write': c.m * c.n * 2 / write_gbs / 1e3}
        bound = max(floors, key=floors.get)
        out = {'bound': bound, 'floor_us': round(floors[bound], 2), 'frac': round(floors[bound] / us, 3)}
        if (c.m, c.n, c.k) in copy_us:      # a device-to-device copy of the same bytes, timed the same way
            out['copy_of_same_bytes_us'] = round(copy_us[(c.m, c.n, c.k)], 2)
            out['frac_of_that_copy'] = round(copy_us[(c.m, c.n, c.k)] / us, 3)
        return out
    shapes = [{'m': c.m, 'n': c.n, 'k': c.k, 'us': round(per_case_us[i], 2),
               'tflops': round(c.flops / per_case_us[i] / 1e6, 1), 'gbs': round(c.bytes / per_case_us[i] / 1e3, 1),
               'block_n': c.config['block_n'], 'cta_group': c.config['cta_group'], 'split_k': c.config['split_k'],
               'split_in_cluster': bool(c.config['cluster_split']),
               'stages': c.config['num_stages'], 'roof': roofs(c, per_case_us[i])} for i, c in enumerate(cases)]
    line = {
        'metric': 'fp8_block_scaled_gemm_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': step_ms_max, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp8_e4m3 x ue8m0, fp32 accumulate', 'data': 'synthetic',
        'config': dense_config(world),
        'timing': ('one CUDA-event pair around the %d steps, each step one replay of a CUDA graph of the 18 launches'
                   % args.steps if graph is not None else 'one CUDA-event pair around the steps, plain stream launches')
                  + '; per-shape and roofline figures: every shape as a graph of back-to-back launches over rotating '
                    'operand sets (more than 4x L2 in total), one event pair around 10 replays',
        'verified': verified,
        'roofline': {'bound': 'tensor', 'achieved': tf_big, 'peak': fp8_peak, 'unit': 'TFLOP/s', 'frac': tf_big / fp8_peak,
                     'traffic': NCU_DRAM_TRAFFIC.get((cases[top].m, cases[top].n, cases[top].k, cases[top].config['block_n'])),
                     'traffic_of': 'one launch of %dx%dx%d (algorithmic %.1f MB), ncu capture of the same tiling'
                                   % (cases[top].m, cases[top].n, cases[top].k, cases[top].bytes / 1e6),
                     'kernel': 'mx_gemm_kernel on the six M=4096 launches',
                     'peak_source': '2 x the BF16 burst figure of MEASURED_PEAKS.json (%s): derived, no FP8 figure is measured'
                                    % pk['source'],
                     'frac_of_nominal': tf_big / NOMINAL_FP8_TFLOPS, 'nominal_peak': NOMINAL_FP8_TFLOPS,
                     'hbm': {'bound': 'hbm', 'achieved': gbs_small, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                             'frac': gbs_small / pk['hbm_gbs'], 'frac_of_nominal': gbs_small / NOMINAL_HBM_GBS,
                             'kernel': 'mx_gemm_kernel (+ split-K finalisation where used) on the twelve M<=128 launches',
                             'peak_source': 'copy bandwidth of MEASURED_PEAKS.json (%s)' % pk['source'],
                             'copies_of_same_bytes_gbs': round(gbs_copies, 1) if gbs_copies else None,
                             'frac_of_copies_of_same_bytes': round(gbs_small / gbs_copies, 3) if gbs_copies else None}},
        'e2e': {'value': e2e_value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': sum(c.h2d for c in cases),
                'd2h_bytes_per_step': sum(c.d2h for c in cases), 'steps': e2e_steps},
        'host_us_per_call': {'fp8_gemm_nt, scales in the required layout (plan reused)': round(host_call_us, 1),
                             'fp8_gemm_nt with FP32 scales (two transforms launched), median':
                                 round(sorted(host_us)[len(host_us) // 2], 1) if host_us else None},
        'hbm_write_gbs': round(write_gbs, 1),
        'gpu_launches': int(launches),
        'clocks': clocks,
        'device_status': status,
        'shapes': shapes,
    }
    if world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        flops, seconds = cpu_oracle_pass(cpu_inputs(SWEEP))
        line['cpu_baseline'] = {'value': flops / seconds / 1e12, 'unit': 'TFLOP/s', 'cores': torch.get_num_threads(),
                                'kind': 'port', 'sample': CPU_SAMPLE_TEXT + ' (%.1f s)' % seconds}
    if legs is not None:
        line['configs'] = legs
        line['verified'] = bool(verified and all(v.get('verified', True) for v in legs.values()))
    emit(line)


def oracle_checks() -> dict:
    """The CPU oracle's checkers for the workloads of `deep_gemm.testing` (which know nothing of the oracle themselves)."""
    from oracle import checks
    return {'mixed': checks.mixed_case, 'grouped': checks.grouped_case, 'dense_row': checks.dense_row,
            'grouped_row': checks.grouped_row, 'moe_mlp': checks.moe_mlp_case}


def other_config_legs(args, device, pk) -> dict:
    """Short legs for the configurations the sweep does not contain: mixed FP8xFP4 (config 3), m-grouped contiguous
    with 32 experts (config 4) and m-grouped masked 32 x 256 (config 5), verified on a row sample, with the roofline
    that bounds each. The mixed and the masked GEMM (tens to hundreds of microseconds) are timed like the sweep's
    shapes, as graphs of back-to-back launches over rotating operand sets larger than L2; the contiguous one
    (milliseconds) per launch after an untimed L2 flush."""
    from deep_gemm.testing import moe_bench
    fp8_peak = 2.0 * pk['bf16_tflops']
    steps = max(3, min(args.steps, 10))
    out = {}
    checks = oracle_checks()
    r = moe_bench.time_mixed(device, steps, checks['mixed'])
    out['mixed_fp8_fp4_nn_4096x7168x2048'] = {
        'us': round(r['us'], 2), 'tflops': round(r['tflops'], 1), 'verified': r['verified'], 'tiling': r['tiling'],
        'roofline': {'bound': 'tensor', 'achieved': r['tflops'], 'peak': fp8_peak, 'unit': 'TFLOP/s',
                     'frac': r['tflops'] / fp8_peak, 'frac_of_nominal': r['tflops'] / NOMINAL_FP8_TFLOPS, 'traffic': None}}
    random.seed(1234)
    sizes = [int(random.uniform(0.7, 1.3) * 8192) for _ in range(GLOBAL_EXPERTS)]
    r = moe_bench.time_grouped(device, sizes, steps, masked=False, check=checks['grouped'])
    out['m_grouped_contiguous_32_experts'] = {
        'shapes': r['shapes'], 'tflops': round(r['tflops'], 1), 'verified': r['verified'],
        'roofline': {'bound': 'tensor', 'achieved': r['tflops'], 'peak': fp8_peak, 'unit': 'TFLOP/s',
                     'frac': r['tflops'] / fp8_peak, 'frac_of_nominal': r['tflops'] / NOMINAL_FP8_TFLOPS, 'traffic': None}}
    masked = [random.randint(0, 256) for _ in range(GLOBAL_EXPERTS)]
    r = moe_bench.time_grouped(device, masked, steps, masked=True, check=checks['grouped'])
    out['m_grouped_masked_32x256'] = {
        'shapes': r['shapes'], 'tflops': round(r['tflops'], 1), 'gbs': round(r['gbs'], 1), 'verified': r['verified'],
        'roofline': {'bound': 'hbm', 'achieved': r['gbs'], 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                     'frac': r['gbs'] / pk['hbm_gbs'], 'frac_of_nominal': r['gbs'] / NOMINAL_HBM_GBS, 'traffic': None}}
    # every row of the reference's own published tables (other hardware), for the ratio a reader will want to see
    from deep_gemm.testing import published_bench
    r = published_bench.time_published(device, steps, check_dense=checks['dense_row'], check_grouped=checks['grouped_row'])
    out['reference_published_tables'] = {
        'tflops': round(r['tflops'], 1), 'published_tflops_other_hardware': round(r['published_tflops'], 1),
        'geomean_speedup_vs_published': round(r['geomean_speedup'], 2), 'verified': r['verified'], 'rows': r['rows']}
    return out


def emit(line: dict) -> None:
    """Write the result line to the process's original stdout (everything else is routed to stderr)."""
    os.write(_RESULT_FD, (json.dumps(line) + '\n').encode())


_RESULT_FD = 1


def main():
    global _RESULT_FD
    # Libraries (NCCL's version banner, for one) print to stdout; keep stdout for the one JSON line.
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='auto',
                    choices=['auto', 'dense', 'grouped', 'masked', 'mixed', 'fp4', 'bf16', 'quant', 'layout', 'published', 'moe_mlp'])
    ap.add_argument('--experts', type=int, default=0, help='grouped / masked workloads: global expert count (default 32)')
    ap.add_argument('--no-graph', action='store_true',
                    help='dense workload: plain stream launches instead of a CUDA graph (for profilers that cannot follow a capture)')
    ap.add_argument('--no-legs', action='store_true', help='dense workload: skip the legs for the other configurations')
    ap.add_argument('--no-gather', action='store_true', help='grouped workload, N > 1: skip the NCCL all-gather of D')
    args = ap.parse_args()

    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if args.impl == 'reference':
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: there is no CPU fallback for the measured path')
    device = torch.device('cuda', local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        torch.distributed.init_process_group('nccl', device_id=device)
    workload = args.workload if args.workload != 'auto' else ('dense' if world == 1 else 'grouped')
    args.workload = workload
    try:
        if workload == 'dense':
            run_dense(args, rank, world, device)
        else:
            from deep_gemm.testing import moe_bench
            moe_bench.run(args, rank, world, device, emit, peaks(), oracle_checks())
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == '__main__':
    main()
