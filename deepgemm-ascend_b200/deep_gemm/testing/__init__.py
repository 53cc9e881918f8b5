"""Timing helpers: the CUDA counterpart of deep_gemm/testing/bench.py:284-400 (bench_msprof)."""

from .bench import KernelProfile, bench_events, bench_graph, l2_flush_buffer  # noqa: F401
