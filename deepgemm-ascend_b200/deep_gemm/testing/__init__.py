"""Timing helpers: the CUDA counterpart of deep_gemm/testing/bench.py:284-400 (bench_msprof)."""

from .bench import (KernelProfile, bench_events, bench_graph, bench_msprof, close_persistent_profiler,  # noqa: F401
                    l2_flush_buffer)
