"""The allocation-free split-K entry point, dg_gemm_launch_static_scratch.

Who needs it: a host that must not allocate device memory around a GEMM (a runtime that owns all device memory in
its own pool, a plugin that is only ever handed pointers, code inside a no-allocation region). The ordinary entry
point asks such a caller for a zeroed workspace whenever K is split; this one keeps the partial sums in a fixed array
inside the library. The test drives both entry points through the C ABI on the same operands and compares the
outputs, twice in a row because the array is shared and keeps the previous call's contents. It is collected last on
purpose and does not depend on any other test having run.
"""

import ctypes as C

import pytest
import torch

import deep_gemm
import oracle
from deep_gemm import _api
from deep_gemm import _lib as L
from helpers import assert_close, seed_all, uniform_fp8

pytestmark = pytest.mark.gpu


def _split_k_config(split: int, block_n: int) -> L.GemmConfig:
    cfg = L.GemmConfig()
    cfg.block_n, cfg.cta_group, cfg.split_k = block_n, 1, split
    return cfg


def _case(m, n, k, seed):
    seed_all(seed)
    a, sfa, a_ref = uniform_fp8((m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
    ref = oracle.gemm_ref(a_ref, b_ref, torch.bfloat16)
    a, b = a.cuda(), b.cuda()
    sfa = deep_gemm.transform_sf_into_required_layout(sfa.cuda(), m, k, (1, 1, 32), is_sfa=True)
    sfb = deep_gemm.transform_sf_into_required_layout(sfb.cuda(), n, k, (1, 1, 32), is_sfa=False)
    return a, sfa, b, sfb, ref


def test_static_scratch_matches_workspace_entry_point_twice():
    """Two calls in a row (the array is shared and keeps the first call's contents), each compared with the ordinary
    entry point and with the CPU oracle. Free device memory as the driver reports it (which sees every allocation,
    not only torch's) must not move across a call once the kernels are loaded."""
    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (m, n, k, split, bn) in enumerate([(128, 640, 4096, 4, 128), (96, 1000, 2048, 8, 96)]):
        a, sfa, b, sfb, ref = _case(m, n, k, seed=10 + call)
        d_ref = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        d_new = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        config = {'block_n': bn, 'cta_group': 1, 'split_k': split}
        # existing entry point: workspace supplied by the caller
        desc = _api._run_gemm(L.GEMM_NORMAL, a, b, d_ref, None, _api.Identity(), sfa, sfb, (1, 1, 32), None, None,
                              None, 'nk', False, config=config)
        # new entry point: same descriptor, other output, no workspace argument at all
        desc.d = d_new.data_ptr()
        cfg = _split_k_config(split, bn)
        L.check(lib.dg_gemm_launch_static_scratch(C.byref(desc), C.byref(cfg), stream))      # loads what it needs
        torch.cuda.synchronize()
        d_new.fill_(float('nan'))
        free_before, torch_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        L.check(lib.dg_gemm_launch_static_scratch(C.byref(desc), C.byref(cfg), stream))
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == torch_before
        assert deep_gemm.device_status() == 0
        assert_close(d_new, d_ref, f'static scratch against the workspace entry point, call {call}')
        assert_close(d_new, ref, f'static scratch against the oracle, call {call}')


def test_static_scratch_with_the_heuristic_and_with_the_cluster_reduction():
    """`config = NULL` (the library picks the tiling) on a few-rows, long-K shape, and an explicit cluster split-K
    (which needs no scratch at all): both must go through and match the oracle."""
    lib = L.lib()
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = 64, 512, 8192
    a, sfa, b, sfb, ref = _case(m, n, k, seed=21)
    d = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    desc = _api._run_gemm(L.GEMM_NORMAL, a, b, d, None, _api.Identity(), sfa, sfb, (1, 1, 32), None, None,
                          None, 'nk', False)
    assert_close(d, ref, 'ordinary entry point')
    d.fill_(float('nan'))
    L.check(lib.dg_gemm_launch_static_scratch(C.byref(desc), None, stream))
    assert_close(d, ref, 'static scratch, heuristic tiling')
    cfg = _split_k_config(4, 128)
    cfg.reserved[3] = 1
    d.fill_(float('nan'))
    L.check(lib.dg_gemm_launch_static_scratch(C.byref(desc), C.byref(cfg), stream))
    assert_close(d, ref, 'static scratch entry point, cluster reduction')
    assert deep_gemm.device_status() == 0


def test_static_scratch_rejects_problems_beyond_its_size():
    lib = L.lib()
    m, n, k = 128, 16384, 1024                      # 128 x 16384 x 4 bytes = 8 MiB of partial sums > 4 MiB
    a, sfa, b, sfb, _ = _case(m, n, k, seed=3)
    d = torch.zeros(m, n, dtype=torch.bfloat16, device='cuda')
    desc = _api._run_gemm(L.GEMM_NORMAL, a, b, d, None, _api.Identity(), sfa, sfb, (1, 1, 32), None, None,
                          None, 'nk', False, config={'block_n': 128, 'cta_group': 1, 'split_k': 1})
    cfg = _split_k_config(2, 128)
    rc = lib.dg_gemm_launch_static_scratch(C.byref(desc), C.byref(cfg), torch.cuda.current_stream().cuda_stream)
    assert rc == L.DG_ERR_WORKSPACE
    assert 'exceeds the built-in' in L.last_error() and str(L.STATIC_SCRATCH_BYTES) in L.last_error()
    # without split-K no scratch is needed and the same problem goes through
    cfg = _split_k_config(1, 128)
    L.check(lib.dg_gemm_launch_static_scratch(C.byref(desc), C.byref(cfg), torch.cuda.current_stream().cuda_stream))
    assert deep_gemm.device_status() == 0
