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
