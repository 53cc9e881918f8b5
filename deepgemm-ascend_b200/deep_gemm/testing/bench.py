"""CUDA-event benchmarking with a cold L2.

Follows the reference's `bench_msprof` (deep_gemm/testing/bench.py:284-400): warm-up iterations, then timed
iterations that each start by overwriting a buffer larger than L2 (:263-268,342-351). The profile object
answers `dur_us`, `tflops()` and `gbps()` like the reference's KernelProfile (:27-71).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib as L

_flush_buffers: dict = {}


def l2_flush_buffer(device: torch.device) -> torch.Tensor:
    """A buffer of twice the L2 size (at least 256 MiB), allocated once per device."""
    key = device.index
    if key not in _flush_buffers:
        l2 = torch.cuda.get_device_properties(device).L2_cache_size
        _flush_buffers[key] = torch.empty(max(2 * l2, 256 << 20), dtype=torch.uint8, device=device)
    return _flush_buffers[key]


@dataclass
class KernelProfile:
    dur_us: float          # mean over the timed iterations
    min_us: float
    max_us: float
    iters: int

    @property
    def dur_ns(self) -> float:
        return self.dur_us * 1000

    def tflops(self, flops: float) -> float:
        return flops / self.dur_us / 1e6

    def gbps(self, nbytes: float) -> float:
        return nbytes / self.dur_us / 1e3


def bench_events(fn, num_warmups: int = 10, num_tests: int = 30, flush_l2: bool = True) -> KernelProfile:
    """Time `fn` (which enqueues work on the current stream) with one CUDA-event pair per iteration."""
    device = torch.device('cuda', torch.cuda.current_device())
    stream = torch.cuda.current_stream(device)
    buf = l2_flush_buffer(device) if flush_l2 else None

    def flush():
        if buf is not None:
            L.check(L.lib().dg_l2_flush_launch(buf.data_ptr(), buf.numel(), stream.cuda_stream))

    for _ in range(num_warmups):
        flush()
        fn()
    torch.cuda.synchronize(device)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    for i in range(num_tests):
        flush()
        starts[i].record(stream)
        fn()
        ends[i].record(stream)
    torch.cuda.synchronize(device)
    times = [s.elapsed_time(e) * 1e3 for s, e in zip(starts, ends)]
    return KernelProfile(sum(times) / len(times), min(times), max(times), num_tests)


def bench_graph(launchers, num_warmups: int = 3, num_tests: int = 10) -> KernelProfile:
    """Time a sequence of launches as one CUDA graph replayed `num_tests` times between one CUDA-event pair, and
    return the mean duration per launch.

    `launchers` are callables taking a raw stream pointer; each must work on operands of its own, and together they
    must touch several times the L2 capacity, so that no launch finds its inputs cached (inputs larger than L2
    instead of a flush kernel between launches). Timing a stream of launches this way leaves out the CUDA-event
    records between kernels that `bench_events` pays per launch and lets consecutive kernels overlap their launch
    latencies exactly as they do in an application that enqueues them back to back."""
    device = torch.device('cuda', torch.cuda.current_device())
    for fn in launchers:                                   # loads kernels, sets attributes: not capturable work
        fn(torch.cuda.current_stream(device).cuda_stream)
    torch.cuda.synchronize(device)
    side = torch.cuda.Stream(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        sptr = torch.cuda.current_stream(device).cuda_stream
        for fn in launchers:
            fn(sptr)
    stream = torch.cuda.current_stream(device)
    for _ in range(num_warmups):
        graph.replay()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(num_tests):
        graph.replay()
    end.record(stream)
    torch.cuda.synchronize(device)
    per_launch = start.elapsed_time(end) * 1e3 / (num_tests * len(launchers))
    return KernelProfile(per_launch, per_launch, per_launch, num_tests * len(launchers))


def _select_profiles(profiles: dict, kernel_names, return_all_kernels: bool):
    # deep_gemm/testing/bench.py:271-281
    if return_all_kernels:
        return profiles
    if isinstance(kernel_names, str):
        matched = {name: profile for name, profile in profiles.items() if kernel_names in name}
        if len(matched) != 1:
            summary = '\n'.join(f'  - {name}' for name in profiles) or '  (none)'
            raise RuntimeError(f"No unique kernel matching '{kernel_names}':\n{summary}")
        return next(iter(matched.values()))
    return [next((profile for name, profile in profiles.items() if query in name), None) for query in kernel_names]


def bench_msprof(fn, kernel_names=None, num_warmups: int = 10, num_tests: int = 30, flush_l2: bool = True,
                 barrier_comm_profiling: bool = False, barrier=None, return_all_kernels: bool = False,
                 suppress_verbose_output: bool = True, backend: str = 'persistent'):
    """Per-kernel device time of the kernels `fn` launches, by name: the interface of the reference's profiler-based timer
    (deep_gemm/testing/bench.py:284-400; same arguments, same three return forms, names matched by substring, template
    arguments of instantiations with the same base name pooled), here over the CUDA activity trace of `torch.profiler`. Every timed iteration starts with
    an L2 flush and, with `barrier_comm_profiling`, a long `npu_sleep` and the barrier, as in the reference. `backend`
    is accepted for compatibility: there is one trace source. The durations come from a tracing profiler: use them to
    compare kernels, and CUDA events (`bench_events`, `bench_graph`) for numbers that are reported."""
    if kernel_names is None and not return_all_kernels:
        raise ValueError('kernel_names is required unless return_all_kernels=True')
    if backend not in ('slow', 'fast', 'persistent'):
        raise ValueError(f'Unsupported profiler backend: {backend}')
    if num_warmups < 0 or num_tests <= 0:
        raise ValueError('num_warmups must be non-negative and num_tests must be positive')
    from .. import _api
    device = torch.device('cuda', torch.cuda.current_device())
    stream = torch.cuda.current_stream(device)
    _api.npu_sleep(0)
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize(device)
    buf = l2_flush_buffer(device) if flush_l2 else None
    profile_barrier = barrier if barrier_comm_profiling else None
    if barrier_comm_profiling and profile_barrier is None:
        import torch.distributed as dist
        dummy = torch.ones(1, dtype=torch.float, device=device)
        profile_barrier = lambda: dist.all_reduce(dummy)            # noqa: E731
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(num_tests):
            if buf is not None:
                L.check(L.lib().dg_l2_flush_launch(buf.data_ptr(), buf.numel(), stream.cuda_stream))
            if profile_barrier is not None:
                _api.npu_sleep(int(2e7))        # keep the device busy so that the barrier, not launch gaps, dominates
                profile_barrier()
            fn()
        torch.cuda.synchronize(device)
    samples: dict = {}
    for event in prof.events():
        if 'cuda' not in str(getattr(event, 'device_type', '')).lower():
            continue
        us = float(getattr(event, 'device_time', 0.0) or getattr(event, 'cuda_time', 0.0) or 0.0)
        samples.setdefault(event.name.split('<')[0].split('(')[0].strip(), []).append(us)
    profiles = {name: KernelProfile(sum(v) / len(v), min(v), max(v), len(v)) for name, v in samples.items() if v}
    return _select_profiles(profiles, kernel_names, return_all_kernels)


def close_persistent_profiler() -> None:
    """Kept for callers of the reference's interface (deep_gemm/testing/bench.py:923-930): there is no resident session."""
