"""Benchmark of the block-scaled FP8 GEMM hot path on B200.

One "step" is one pass over the dense FP8 NT sweep named by the baseline: M in {64, 128, 4096} times six (N, K)
pairs, BF16 output, A quantised per 1x128 and B per 128x128 from N(0,1) data (synthetic, seeded). Every GEMM has its
own operands, so a step touches about 1.5 GB and no launch finds its inputs in L2. The steps are timed on the device
with one CUDA-event pair around all of them, each step being one replay of a CUDA graph of the 18 launches; a second
pass with one event pair per launch gives the per-shape table and the roofline figures.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload dense|grouped|masked|mixed|fp4|bf16|quant]

Prints one JSON line (rank 0). `value` is whole-job TFLOP/s with operands resident in HBM; `e2e` is the same metric
through the public Python API with pinned host buffers, host<->device copies inside the timed region.
With N > 1 (torchrun, one rank per GPU) the dense shapes are sharded along N: the global problem has N_global =
ranks x N columns and each rank owns one N-wide slab, so per-GPU work is fixed (weak scaling) and no collective is
needed. `--workload grouped` shards experts across ranks instead and reports the optional NCCL gather separately.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
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
FP8_MAX = 448.0


def peaks() -> dict:
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        p = json.load(open(path))
        return {'hbm_gbs': p['hbm_gbs'], 'bf16_tflops': p['bf16_tflops'],
                'bf16_tflops_sustained': p.get('bf16_tflops_sustained', p['bf16_tflops']), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0, 'source': 'fallback'}


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


class DenseCase:
    """One (M, N, K) problem with operands on the device, canonical scale factors, and a prepared C-ABI call."""

    def __init__(self, m, n, k, device, seed):
        import deep_gemm
        from deep_gemm import _api
        g = torch.Generator(device=device).manual_seed(seed)
        self.m, self.n, self.k = m, n, k
        self.a, self.sfa32 = quantize_fp8(torch.randn(m, k, device=device, generator=g), (1, 128))
        self.b, self.sfb32 = quantize_fp8(torch.randn(n, k, device=device, generator=g), (128, 128))
        self.d = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        # scale factors already in the required layout: the kernel-only number excludes the relayout
        self.sfa = deep_gemm.transform_sf_into_required_layout(self.sfa32, m, k, (1, 128, 128), is_sfa=True)
        self.sfb = deep_gemm.transform_sf_into_required_layout(self.sfb32, n, k, (1, 128, 128), is_sfa=False)
        self.desc = _api._run_gemm(_api.L.GEMM_NORMAL, self.a, self.b, self.d, None, _api.Identity(), self.sfa, self.sfb,
                                   (1, 1, 32), None, None, None, 'nk', False)
        self.flops = 2.0 * m * n * k
        k64 = -(-k // 64)
        self.bytes = m * k + n * k + (m + n) * k64 * 2 + m * n * 2
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
def cpu_oracle_sample(shapes, repeats=1):
    """Times oracle.gemm_ref (dequantise + FP32 matmul + BF16 cast) on `shapes`; returns (TFLOP/s, seconds)."""
    import oracle
    torch.manual_seed(0)
    total_flops, total_s = 0.0, 0.0
    for (m, n, k) in shapes:
        a, sfa, _ = oracle.quantize_e4m3(torch.randn(m, k), (1, 128))
        b, sfb, _ = oracle.quantize_e4m3(torch.randn(n, k), (128, 128))
        for _ in range(repeats):
            t0 = time.perf_counter()
            a_deq = oracle.dequantize(oracle.decode_e4m3(a), sfa, 1, 128)
            b_deq = oracle.dequantize(oracle.decode_e4m3(b), sfb, 128, 128)
            oracle.gemm_ref(a_deq, b_deq, torch.bfloat16)
            total_s += time.perf_counter() - t0
            total_flops += 2.0 * m * n * k
    return total_flops / total_s / 1e12, total_s


CPU_SAMPLE = [(128, n, k) for n, k in NK_LIST] + [(4096, 7168, 2048)]
CPU_SAMPLE_TEXT = 'dequantise + FP32 matmul + BF16 cast of the six M=128 shapes and 4096x7168x2048, torch CPU'


def run_reference(args, rank, world):
    """The reference's CPU implementation of the path (its test oracle) on this box's host cores."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(args.warmup):
        cpu_oracle_sample(CPU_SAMPLE[:2])
    t0 = time.perf_counter()
    flops = 0.0
    for _ in range(args.steps):
        tf, s = cpu_oracle_sample(CPU_SAMPLE)
        flops += tf * s * 1e12
    elapsed = time.perf_counter() - t0
    value = flops / elapsed / 1e12
    line = {
        'impl': 'reference', 'metric': 'fp8_block_scaled_gemm_tflops', 'value': value, 'unit': 'TFLOP/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': elapsed / args.steps * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'dense FP8 NT sweep, M in {64,128,4096} x 6 (N,K), BF16 out', 'sample': CPU_SAMPLE_TEXT},
        'cpu_baseline': {'value': value, 'unit': 'TFLOP/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                         'sample': CPU_SAMPLE_TEXT},
        'e2e': {'value': value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    emit(line)


# ----------------------------------------------------------------------------------------------------------------
# Main arm
# ----------------------------------------------------------------------------------------------------------------
def run_dense(args, rank, world, device):
    import deep_gemm
    from deep_gemm import _lib as L
    lib = L.lib()
    pk = peaks()
    stream = torch.cuda.current_stream(device)
    sptr = stream.cuda_stream
    cases = [DenseCase(m, n, k, device, seed=1000 * rank + i)
             for i, (m, (n, k)) in enumerate((m, nk) for m in M_LIST for nk in NK_LIST)]
    torch.cuda.synchronize(device)

    # One step = the 18 GEMMs back to back. Every GEMM has its own operands and the sweep touches far more than the
    # L2 holds between two uses of the same buffer (`footprint` below), so every launch finds its inputs in HBM
    # without a flush kernel in between.
    footprint = sum(c.bytes for c in cases)
    l2_bytes = torch.cuda.get_device_properties(device).L2_cache_size
    assert footprint > 4 * l2_bytes, 'the sweep must not fit in L2'

    def sweep(stream_ptr, record=None):
        for ci, c in enumerate(cases):
            if record is not None:
                record[ci][0].record(stream)
            c.launch(lib, stream_ptr)
            if record is not None:
                record[ci][1].record(stream)

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

    # Second pass, same sweep with one CUDA-event pair around every launch: the per-shape table and the roofline
    # figures (a launch timed this way includes the gap to its neighbours, so these are upper bounds on kernel time).
    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in cases]
              for _ in range(args.steps)]
    for s in range(args.steps):
        sweep(sptr, events[s])
    barrier()
    clocks = sampler.stop() if sampler else None
    status = deep_gemm.device_status()

    per_case_us = [sum(events[s][ci][0].elapsed_time(events[s][ci][1]) for s in range(args.steps)) / args.steps * 1e3
                   for ci in range(len(cases))]
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
                deep_gemm.fp8_gemm_nt((c.a, c.sfa32), (c.b, c.sfb32), c.d, recipe=(1, 128, 128))
                done_mm[i] = torch.cuda.Event()
                done_mm[i].record(s_mm)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done_mm[i])
                c.h_d.copy_(c.d, non_blocking=True)
                done_out[i] = torch.cuda.Event()
                done_out[i].record(s_out)

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = torch.tensor([(time.perf_counter() - t0) / e2e_steps], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(e2e_s, op=torch.distributed.ReduceOp.MAX)
    e2e_value = world * flops_step / float(e2e_s.item()) / 1e12

    if rank != 0:
        return
    # ---- roofline of the dominant kernel (the GEMM kernel on the tensor-bound M = 4096 shapes) and of the
    #      HBM-bound small-M launches
    big = [i for i, c in enumerate(cases) if c.m == 4096]
    small = [i for i, c in enumerate(cases) if c.m <= 128]
    tf_big = sum(cases[i].flops for i in big) / sum(per_case_us[i] for i in big) / 1e6
    gbs_small = sum(cases[i].bytes for i in small) / sum(per_case_us[i] for i in small) / 1e3
    fp8_peak = 2.0 * pk['bf16_tflops']
    shapes = [{'m': c.m, 'n': c.n, 'k': c.k, 'us': round(per_case_us[i], 2),
               'tflops': round(c.flops / per_case_us[i] / 1e6, 1), 'gbs': round(c.bytes / per_case_us[i] / 1e3, 1),
               'block_n': c.config['block_n'], 'cta_group': c.config['cta_group'], 'split_k': c.config['split_k'],
               'split_in_cluster': bool(c.config['cluster_split']),
               'stages': c.config['num_stages']} for i, c in enumerate(cases)]
    cpu_tf, cpu_s = cpu_oracle_sample(CPU_SAMPLE) if world == 1 else (None, None)
    line = {
        'metric': 'fp8_block_scaled_gemm_tflops', 'value': value, 'unit': 'TFLOP/s', 'n_gpus': world,
        'steps': args.steps, 'warmup': max(args.warmup, 3), 'ms_per_step': step_ms_max, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp8_e4m3 x ue8m0, fp32 accumulate', 'data': 'synthetic',
        'config': {'workload': 'dense FP8 NT sweep: M in {64,128,4096} x (N,K) in ' + str(NK_LIST) +
                               ', BF16 out, A scaled per 1x128, B per 128x128 (UE8M0)',
                   'l2': 'inputs larger than L2: every GEMM has its own operands, %d MB per step against %d MB of L2'
                         % (footprint // 10**6, l2_bytes // 10**6),
                   'sharding': 'none' if world == 1 else 'N-slabs, one per rank, no collective',
                   'timing': ('one CUDA-event pair around the %d steps, each step one replay of a CUDA graph of the 18 launches'
                              % args.steps if graph is not None else 'one CUDA-event pair around the steps, plain stream launches')
                             + '; per-shape and roofline figures from a second pass with one event pair per launch'},
        'roofline': {'bound': 'tensor', 'achieved': tf_big, 'peak': fp8_peak, 'unit': 'TFLOP/s', 'frac': tf_big / fp8_peak,
                     'traffic': 489.5e6, 'traffic_of': 'dram__bytes_read.sum + dram__bytes_write.sum of the 4096x7168x16384 launch '
                     '(ncu capture in profiles/mx_gemm_wide_tile_pair.md; algorithmic 249.0 MB)',
                     'kernel': 'mx_gemm_kernel on the six M=4096 launches',
                     'peak_source': '2 x bf16 burst of MEASURED_PEAKS.json (%s)' % pk['source']},
        'roofline_small_m': {'bound': 'hbm', 'achieved': gbs_small, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
                             'frac': gbs_small / pk['hbm_gbs'], 'kernel': 'mx_gemm_kernel (+ split-K finalisation) on the twelve M<=128 launches'},
        'e2e': {'value': e2e_value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': sum(c.h2d for c in cases),
                'd2h_bytes_per_step': sum(c.d2h for c in cases), 'steps': e2e_steps},
        'gpu_launches': int(launches),
        'clocks': clocks,
        'device_status': status,
        'shapes': shapes,
    }
    if cpu_tf is not None:
        line['cpu_baseline'] = {'value': cpu_tf, 'unit': 'TFLOP/s', 'cores': torch.get_num_threads(), 'kind': 'port',
                                'sample': CPU_SAMPLE_TEXT + ' (%.1f s)' % cpu_s}
    emit(line)


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
    ap.add_argument('--workload', default='dense', choices=['dense', 'grouped', 'masked', 'mixed', 'fp4', 'bf16', 'quant'])
    ap.add_argument('--experts-per-gpu', type=int, default=0, help='grouped / masked workloads (default 8 / 32)')
    ap.add_argument('--no-graph', action='store_true',
                    help='dense workload: plain stream launches instead of a CUDA graph (for profilers that cannot follow a capture)')
    ap.add_argument('--gather', action='store_true', help='grouped workload, N > 1: also time an NCCL all-gather of D')
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
    try:
        if args.workload == 'dense':
            run_dense(args, rank, world, device)
        else:
            from deep_gemm.testing import moe_bench
            moe_bench.run(args, rank, world, device, emit)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == '__main__':
    main()
