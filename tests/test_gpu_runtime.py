"""Runtime behaviour around the GEMM on the GPU: invalid scale factors, the sleep marker kernel, deterministic mode,
the launch-plan cache, operands and outputs that are column slices of wider tensors, launch overlap on and off."""

import ctypes as C

import pytest
import torch

import deep_gemm
import oracle
from deep_gemm import _lib as L
from helpers import assert_close, seed_all, uniform_fp8, with_major

pytestmark = pytest.mark.gpu


def test_invalid_fp32_scale_factor_is_reported_not_trapped():
    """The reference asserts on the device when an FP32 scale is negative or not a power of two
    (deep_gemm/include/deep_gemm/transform_sf.hpp:13-21). Here the transform records it and `device_status()`
    reports code 201 once; the context stays usable."""
    assert deep_gemm.device_status() == 0
    mn, k = 256, 512
    sf = torch.ones(mn, k // 32, device='cuda')
    deep_gemm.transform_sf_into_required_layout(sf, mn, k, (1, 1, 32), is_sfa=True)
    assert deep_gemm.device_status() == 0
    for bad in (1.5, -1.0):
        sf2 = sf.clone()
        sf2[17, 3] = bad
        deep_gemm.transform_sf_into_required_layout(sf2, mn, k, (1, 1, 32), is_sfa=True)
        assert deep_gemm.device_status() == deep_gemm._api.STATUS_INVALID_SCALE_FACTOR
        assert deep_gemm.device_status() == 0                # reported once
    # the same through a GEMM call that is handed FP32 scales
    seed_all(1)
    a, sfa, _ = uniform_fp8((128, 512), (1, 32))
    b, sfb, _ = uniform_fp8((256, 512), (1, 32))
    sfa[5, 2] = 3.0
    d = torch.empty(128, 256, dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d)
    assert deep_gemm.device_status() == deep_gemm._api.STATUS_INVALID_SCALE_FACTOR
    # and the library still works afterwards
    sfa[5, 2] = 0.5
    deep_gemm.fp8_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d)
    assert deep_gemm.device_status() == 0


def test_npu_sleep_runs_and_takes_about_the_requested_time():
    """csrc/apis/runtime.hpp:64-79: one block per SM spinning for the given number of cycles."""
    deep_gemm.npu_sleep(0)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    deep_gemm.npu_sleep(2_000_000, marker=1)                # about 1 ms at 1.9 GHz
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    assert 0.5 < ms < 20.0, ms
    with pytest.raises(RuntimeError, match='sleep_cycles'):
        deep_gemm.npu_sleep(10 ** 10)
    assert deep_gemm.device_status() == 0


def test_deterministic_mode_gives_the_same_bits_every_time():
    """MN-major B with few rows and a long K is where the heuristic otherwise splits K through the FP32 workspace
    (partial sums added in arrival order). With use_deterministic_algorithms(True) repeated runs agree bit for bit
    and still match the oracle."""
    seed_all(5)
    m, n, k = 128, 512, 16384
    a, sfa, a_ref = uniform_fp8((m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
    ref = oracle.gemm_ref(a_ref, b_ref, torch.float32)
    b_dev = with_major(b, True).cuda()
    a_arg, b_arg = (a.cuda(), sfa.cuda()), (b_dev.transpose(0, 1), sfb.cuda().transpose(0, 1))
    deep_gemm.use_deterministic_algorithms(True)
    try:
        outs = []
        for _ in range(4):
            d = torch.empty(m, n, dtype=torch.float32, device='cuda')
            deep_gemm.fp8_gemm_nn(a_arg, b_arg, d)
            outs.append(d)
        assert deep_gemm.device_status() == 0
        assert all(torch.equal(outs[0], o) for o in outs[1:])
        assert_close(outs[0], ref, 'deterministic nn')
        # K-major B takes the cluster reduction (rank order), with or without the flag
        outs = []
        for _ in range(3):
            d = torch.empty(m, n, dtype=torch.float32, device='cuda')
            deep_gemm.fp8_gemm_nt(a_arg, (b.cuda(), sfb.cuda()), d)
            outs.append(d)
        assert all(torch.equal(outs[0], o) for o in outs[1:])
        assert_close(outs[0], ref, 'deterministic nt')
    finally:
        deep_gemm.use_deterministic_algorithms(False)


def test_repeated_calls_reuse_the_launch_plan():
    seed_all(2)
    a, sfa, a_ref = uniform_fp8((256, 1024), (1, 32))
    b, sfb, b_ref = uniform_fp8((384, 1024), (1, 32))
    a_dev, b_dev = a.cuda(), b.cuda()
    sfa_dev = deep_gemm.transform_sf_into_required_layout(sfa.cuda(), 256, 1024, (1, 1, 32), is_sfa=True)
    sfb_dev = deep_gemm.transform_sf_into_required_layout(sfb.cuda(), 384, 1024, (1, 1, 32), is_sfa=False)
    d = torch.empty(256, 384, dtype=torch.bfloat16, device='cuda')
    hits, misses = C.c_uint64(), C.c_uint64()
    lib = L.lib()
    deep_gemm.fp8_gemm_nt((a_dev, sfa_dev), (b_dev, sfb_dev), d)
    lib.dg_plan_cache_stats(C.byref(hits), C.byref(misses))
    h0, m0 = hits.value, misses.value
    for _ in range(5):
        d.fill_(float('nan'))
        deep_gemm.fp8_gemm_nt((a_dev, sfa_dev), (b_dev, sfb_dev), d)
    lib.dg_plan_cache_stats(C.byref(hits), C.byref(misses))
    assert hits.value == h0 + 5 and misses.value == m0
    assert_close(d, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16), 'cached plan')
    # another output buffer is another plan
    d2 = torch.empty(256, 384, dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nt((a_dev, sfa_dev), (b_dev, sfb_dev), d2)
    lib.dg_plan_cache_stats(C.byref(hits), C.byref(misses))
    assert misses.value == m0 + 1
    assert torch.equal(d.view(torch.int16), d2.view(torch.int16))
    assert deep_gemm.device_status() == 0


@pytest.mark.parametrize('m,n,k,out', [(128, 512, 2048, torch.bfloat16), (4096, 1024, 1024, torch.bfloat16),
                                       (300, 520, 1024, torch.float32)])
def test_output_and_operands_as_column_slices_of_wider_tensors(m, n, k, out):
    """Dense N-sharding writes D[:, n0:n1] of a wider D (outer_stride_d > n; csrc/jit_kernels/gemm_config.hpp:68-75);
    A and B may be K-slices of wider tensors. Columns outside the slice must stay untouched."""
    seed_all(m + n)
    a, sfa, a_ref = uniform_fp8((m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
    ref = oracle.gemm_ref(a_ref, b_ref, out)
    # D as columns [n0, n0 + n) of a tensor three slabs wide
    n0 = n + 64
    wide_d = torch.full((m, 3 * n + 128), 7.0, dtype=out, device='cuda')
    d = wide_d[:, n0:n0 + n]
    # A and B as column ranges of wider byte tensors
    wide_a = torch.zeros(m, k + 256, dtype=torch.uint8, device='cuda')
    wide_a[:, 128:128 + k] = a.view(torch.uint8).cuda()
    wide_b = torch.zeros(n, 2 * k, dtype=torch.uint8, device='cuda')
    wide_b[:, k:] = b.view(torch.uint8).cuda()
    a_arg = (wide_a[:, 128:128 + k].view(torch.float8_e4m3fn), sfa.cuda())
    b_arg = (wide_b[:, k:].view(torch.float8_e4m3fn), sfb.cuda())
    deep_gemm.fp8_gemm_nt(a_arg, b_arg, d)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref, f'column slices {m}x{n}x{k}')
    assert bool((wide_d[:, :n0] == 7.0).all()) and bool((wide_d[:, n0 + n:] == 7.0).all()), 'columns outside the slab were written'
    # accumulate into the slab
    if out == torch.float32:
        c = torch.randn(m, n)
        d.copy_(c)
        deep_gemm.fp8_gemm_nt(a_arg, b_arg, d, c=d)
        assert_close(d, oracle.gemm_ref(a_ref, b_ref, out, c=c), 'column slab accumulate')
        assert bool((wide_d[:, :n0] == 7.0).all()) and bool((wide_d[:, n0 + n:] == 7.0).all())


def test_results_do_not_depend_on_launch_overlap():
    """GEMMs queued back to back, each reading the previous one's output as its A operand: with programmatic
    dependent launch (the default) a kernel starts before its predecessor has finished and must still see all of
    its output. Same bits with the overlap switched off."""
    seed_all(9)
    m, n, k = 128, 512, 512
    x, sfx, _ = uniform_fp8((m, k), (1, 32))
    ws = [uniform_fp8((n, k), (1, 32)) for _ in range(6)]
    lib = L.lib()

    def chain():
        cur = (x.cuda(), sfx.cuda())
        outs = []
        for w, sfw, _ in ws:
            d = torch.empty(m, n, dtype=torch.bfloat16, device='cuda')
            deep_gemm.fp8_gemm_nt(cur, (w.cuda(), sfw.cuda()), d)
            outs.append(d)
            # next A: the output's bytes reinterpreted as E4M3 codes (NaN codes masked), unit scales
            codes = d.view(torch.uint8).reshape(m, 2 * n)[:, :k] & 0x77
            cur = (codes.view(torch.float8_e4m3fn), torch.ones(m, k // 32, device='cuda'))
        torch.cuda.synchronize()
        return outs

    assert lib.dg_get_overlap_launches() == 1
    first = chain()
    try:
        lib.dg_set_overlap_launches(0)
        second = chain()
    finally:
        lib.dg_set_overlap_launches(1)
    assert deep_gemm.device_status() == 0
    for x1, x2 in zip(first, second):
        assert torch.equal(x1.view(torch.int16), x2.view(torch.int16))


def test_lean_gemm_after_kernels_that_dirty_shared_memory():
    """A small-M GEMM (one tile per CTA, warps 0..3 join the epilogue) launched straight behind kernels that leave other
    contents in shared memory: every warp must take the accumulator's TMEM address from this CTA's own allocation, never
    from whatever the previous kernel left at that shared-memory word. Same bits as the first, undisturbed, call."""
    seed_all(10)
    m, n, k = 128, 7168, 2048
    a, sfa, _ = uniform_fp8((m, k), (1, 128))
    b, sfb, _ = uniform_fp8((n, k), (128, 128))
    a, sfa, b, sfb = a.cuda(), sfa.cuda(), b.cuda(), sfb.cuda()
    sfa_t = deep_gemm.transform_sf_into_required_layout(sfa, m, k, (1, 128), None)
    sfb_t = deep_gemm.transform_sf_into_required_layout(sfb, n, k, (128, 128), None)
    want = torch.empty(m, n, dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nt((a, sfa_t), (b, sfb_t), want)
    torch.cuda.synchronize()
    noise = torch.randn(148 * 8, 4096, device='cuda')
    for i in range(40):
        got = torch.empty_like(want)
        # softmax, sort and a small matmul keep data in shared memory on every SM
        torch.softmax(noise, dim=-1)
        torch.sort(noise, dim=-1)
        noise[:512, :512] @ noise[:512, :512]
        deep_gemm.fp8_gemm_nt((a, sfa_t), (b, sfb_t), got)
        torch.cuda.synchronize()
        assert deep_gemm.device_status() == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f'iteration {i}'


def test_bench_msprof_reports_the_gemm_kernel_by_name():
    """The reference's profiler-based timer (deep_gemm/testing/bench.py:284-400) with its three return forms."""
    from deep_gemm.testing import bench_msprof
    seed_all(11)
    m, n, k = 256, 512, 1024
    a, sfa, _ = uniform_fp8((m, k), (1, 32))
    b, sfb, _ = uniform_fp8((n, k), (1, 32))
    a, sfa, b, sfb = a.cuda(), sfa.cuda(), b.cuda(), sfb.cuda()
    d = torch.empty(m, n, dtype=torch.bfloat16, device='cuda')

    def fn():
        deep_gemm.fp8_gemm_nt((a, sfa), (b, sfb), d)
    one = bench_msprof(fn, kernel_names='mx_gemm_kernel', num_warmups=2, num_tests=5)
    assert one.iters == 5 and 0.5 < one.dur_us < 1000 and one.tflops(2.0 * m * n * k) > 0
    both = bench_msprof(fn, kernel_names=['mx_gemm_kernel', 'transform_sf', 'no_such_kernel'], num_warmups=1, num_tests=3)
    assert both[0] is not None and both[1] is not None and both[2] is None
    everything = bench_msprof(fn, return_all_kernels=True, num_warmups=1, num_tests=3)
    assert any('mx_gemm_kernel' in name for name in everything) and any('l2_flush' in name for name in everything)
    with pytest.raises(RuntimeError, match='No unique kernel'):
        bench_msprof(fn, kernel_names='kernel', num_warmups=0, num_tests=1)
    with pytest.raises(ValueError):
        bench_msprof(fn)


@pytest.mark.parametrize('m,n,k', [(256, 384, 1024), (130, 200, 512), (4096, 512, 2048), (64, 2112, 7168)])
def test_bf16_accumulation_rounds_once(m, n, k):
    """D (BF16) = A B + D is the FP32 sum rounded once: bit for bit the BF16 cast of the FP32-accumulated result, also
    where product and addend nearly cancel (a reduce-add of a BF16-rounded product would be off by several ulps there)."""
    seed_all(12)
    a, sfa, a_ref = uniform_fp8((m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
    prod = a_ref @ b_ref.T
    c = (-prod * (1.0 + 0.01 * torch.randn(m, n))).to(torch.bfloat16)           # nearly cancels the product
    a_arg, b_arg = (a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda())
    d32 = c.float().cuda()
    deep_gemm.fp8_gemm_nt(a_arg, b_arg, d32, c=d32)
    d16 = c.cuda()
    deep_gemm.fp8_gemm_nt(a_arg, b_arg, d16, c=d16)
    assert deep_gemm.device_status() == 0
    assert torch.equal(d16.view(torch.int16), d32.to(torch.bfloat16).view(torch.int16))
    assert_close(d16, (prod + c.float()).to(torch.bfloat16), f'bf16 accumulate {m}x{n}x{k}')


def _runtime_cases():
    seed_all(21)
    cases = []
    for (m, n, k) in [(128, 2112, 7168), (64, 512, 8192), (1000, 1500, 1024), (4096, 1024, 512)]:
        a, sfa, a_ref = uniform_fp8((m, k), (1, 32))
        b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
        cases.append(((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), oracle.gemm_ref(a_ref, b_ref, torch.bfloat16), (m, n, k)))
    return cases


def test_sm_limit_from_all_sms_down_to_one():
    """`set_num_sms` (csrc/apis/runtime.hpp:12-24): grids, cluster splits and waves follow the limit; results do not change."""
    cases = _runtime_cases()
    try:
        for sms in (148, 132, 100, 33, 8, 2, 1):
            deep_gemm.set_num_sms(sms)
            for a, b, ref, shape in cases:
                d = torch.full(ref.shape, float('nan'), dtype=torch.bfloat16, device='cuda')
                deep_gemm.fp8_gemm_nt(a, b, d)
                assert deep_gemm.device_status() == 0
                assert_close(d, ref, f'num_sms={sms} {shape}')
    finally:
        deep_gemm.set_num_sms(torch.cuda.get_device_properties(0).multi_processor_count)


def test_threads_on_streams_of_their_own():
    """Three host threads, each on its own stream, alternating the heuristic's tiling and a split through the FP32 scratch
    (one scratch per stream): the ABI is thread-safe and the launches of different streams do not share state."""
    import threading
    cases = _runtime_cases()[:3]
    errors = []

    def worker(tid):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                for it in range(20):
                    for a, b, ref, shape in cases:
                        d = torch.full(ref.shape, float('nan'), dtype=torch.bfloat16, device='cuda')
                        cfg = {'block_n': 128, 'cta_group': 1, 'split_k': 4} if (it + tid) % 2 else None
                        deep_gemm.fp8_gemm_nt(a, b, d, config=cfg)
                        stream.synchronize()
                        assert_close(d, ref, f'thread {tid} iteration {it} {shape}')
        except Exception as exc:        # noqa: BLE001 - collected and reported by the main thread
            errors.append((tid, repr(exc)[:300]))
    threads = [threading.Thread(target=worker, args=(t,)) for t in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert errors == [] and deep_gemm.device_status() == 0


def test_api_calls_inside_a_cuda_graph():
    """Calls with FP32 scales (two relayout kernels each) and a K split through the scratch, captured once (after a
    first plain call, as the header asks) and replayed: same results at every replay."""
    a, b, ref, _ = _runtime_cases()[1]
    split = {'block_n': 128, 'cta_group': 1, 'split_k': 4}
    d = torch.empty(ref.shape, dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nt(a, b, d)
    deep_gemm.fp8_gemm_nt(a, b, d, config=split)
    torch.cuda.synchronize()
    d1, d2 = torch.empty_like(d), torch.empty_like(d)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        deep_gemm.fp8_gemm_nt(a, b, d1)
        deep_gemm.fp8_gemm_nt(a, b, d2, config=split)
    for _ in range(3):
        d1.fill_(float('nan'))
        d2.fill_(float('nan'))
        graph.replay()
        torch.cuda.synchronize()
        assert_close(d1, ref, 'replayed, heuristic tiling')
        assert_close(d2, ref, 'replayed, split through the scratch')
    assert deep_gemm.device_status() == 0
