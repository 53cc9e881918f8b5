"""The reference's own FP8 case matrix at its full sizes, for the cases the benchmark-configuration tests leave out.

tests/generators.py:544-576 (dense): forward M in {1, 128, 4096} over seven (N, K), and for 4096 tokens the dgrad
(K-major x MN-major, BF16) and wgrad (MN-major x MN-major, FP32 accumulate and BF16) problems of every (N, K).
tests/generators.py:579-603 (m-grouped contiguous): (groups, expected rows per group) in {(4, 1), (4, 8192),
(8, 4096)} over four (N, K), B K-major and MN-major.

Inputs follow the reference's generator for these cases (tests/generators.py:137-153): every non-NaN E4M3 code equally
likely, one power-of-two scale from {2^-9, 2^-8, 2^-7} per 1 x 32 block, recipe (1, 1, 32). Every call goes through
the public API with the tiling the heuristic picks. The whole output is compared with the CPU oracle except for the
two large m-grouped settings, where the oracle checks each group's first, last and one random 256-row block; padding
rows of D must be exactly zero everywhere. Tolerance: tests/helpers.py (1 - cosine <= 1e-3, max relative error <= 2e-2).
"""

import random

import pytest
import torch

import deep_gemm
import oracle
from helpers import assert_close, assert_close_device, pow2_scales, seed_all, uniform_codes, uniform_fp8, with_major

pytestmark = pytest.mark.gpu

NK_ALL = [(2112, 7168), (576, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]
# (2112, 7168) and (7168, 2048) at 4096 rows are in test_gpu_baseline_configs.py
NK_BACKWARD = [(576, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168)]


@pytest.mark.parametrize('n,k', NK_ALL)
def test_forward_single_row(n, k):
    """M = 1: one row of A against the whole weight (a 128-row tile with 127 rows out of bounds)."""
    seed_all(n ^ k)
    a, sfa, a_ref = uniform_fp8((1, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
    d = torch.full((1, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d)
    assert deep_gemm.device_status() == 0
    assert_close(d, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16), f'fwd 1x{n}x{k}')


@pytest.mark.parametrize('m', [128, 4096])
def test_forward_576_columns(m):
    """(N, K) = (576, 7168), the forward shape of the reference's list that the benchmark sweep does not contain."""
    n, k = 576, 7168
    seed_all(m)
    a, sfa, a_ref = uniform_fp8((m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
    d = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d)
    assert deep_gemm.device_status() == 0
    assert_close_device(d, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16), f'fwd {m}x{n}x{k}')


@pytest.mark.parametrize('n,k', NK_BACKWARD)
def test_backward_problems_of_4096_tokens(n, k):
    m = 4096
    seed_all(2 * n + k)
    # dgrad, problem (m, k, n): D [m, k] = A [m, n] @ B [k, n]^T, B stored with its MN axis (k) contiguous
    a, sfa, a_ref = uniform_fp8((m, n), (1, 32))
    b, sfb, b_ref = uniform_fp8((k, n), (1, 32))
    b_dev = with_major(b, True).cuda()
    d = torch.full((m, k), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nn((a.cuda(), sfa.cuda()), (b_dev.transpose(0, 1), sfb.cuda().transpose(0, 1)), d)
    assert_close_device(d, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16), f'dgrad {m}x{k}x{n}')
    del a, b, a_ref, b_ref, b_dev, d
    # wgrad, problem (n, m, k): D [n, m] = A [n, k] @ B [m, k]^T, both operands stored with MN contiguous
    a, sfa, a_ref = uniform_fp8((n, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((m, k), (1, 32))
    a_arg = (with_major(a, True).cuda().transpose(0, 1), sfa.cuda().transpose(0, 1))
    b_arg = (with_major(b, True).cuda().transpose(0, 1), sfb.cuda().transpose(0, 1))
    prod = a_ref @ b_ref.T
    d = torch.full((n, m), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_tn(a_arg, b_arg, d)
    assert_close_device(d, prod.to(torch.bfloat16), f'wgrad {n}x{m}x{k}')
    c = torch.randn(n, m)
    d = c.cuda()
    deep_gemm.fp8_gemm_tn(a_arg, b_arg, d, c=d)
    assert_close_device(d, prod + c, f'wgrad {n}x{m}x{k} accumulate')
    assert deep_gemm.device_status() == 0


def _group_sizes(num_groups: int, expected_m: int) -> list[int]:
    # tests/generators.py:212-220: every group draws its row count around the expected one
    return [int(expected_m * random.uniform(0.7, 1.3)) for _ in range(num_groups)]


@pytest.mark.parametrize('n,k', [(6144, 7168), (7168, 3072), (4096, 4096), (4096, 2048)])
@pytest.mark.parametrize('num_groups,expected_m', [(4, 1), (4, 8192), (8, 4096)])
def test_m_grouped_contiguous_reference_settings(num_groups, expected_m, n, k):
    random.seed(num_groups * 100003 + expected_m + n)
    sizes = _group_sizes(num_groups, expected_m)
    if expected_m == 1:
        sizes[0], sizes[-1] = 1, 0                       # a one-row group and an empty one are always among them
    total, psum = oracle.make_psum_layout(sizes, 256)
    seed_all(n + k + num_groups)
    a, sfa = uniform_codes((total, k)), pow2_scales((total, k // 32))
    for span in oracle.psum_padding_spans(psum, 256):
        a[span] = 0                                      # padding rows of A are zero, those of the scales are not
        sfa[span] = torch.randn_like(sfa[span])
    b, sfb = uniform_codes((num_groups, n, k)).view(torch.float8_e4m3fn), pow2_scales((num_groups, n, k // 32))
    # the oracle's answer for the blocks to check: the whole group when it is small, three 256-row blocks otherwise
    refs = []
    for gi, span in enumerate(oracle.psum_valid_spans(psum, 256)):
        if span.stop == span.start:
            continue
        if expected_m == 1:
            starts = [span.start]
        else:
            last = (span.stop - 1) // 256 * 256
            starts = sorted({span.start, last, random.randrange(span.start, last + 1, 256)})
        b_ref = oracle.dequantize(b[gi].float(), sfb[gi], 1, 32)
        for r0 in starts:
            rows = slice(r0, min(r0 + 256, span.stop))
            a_blk = oracle.dequantize(a[rows].view(torch.float8_e4m3fn).float(), sfa[rows], 1, 32)
            refs.append((rows, (a_blk @ b_ref.T).to(torch.bfloat16)))
    a_arg = (a.view(torch.float8_e4m3fn).cuda(), sfa.cuda())
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    for trans_b in (False, True):
        if trans_b:
            b_arg = (with_major(b, True).cuda().transpose(1, 2), sfb.cuda().transpose(1, 2))
            fn = deep_gemm.m_grouped_fp8_gemm_nn_contiguous
        else:
            b_arg = (b.cuda(), sfb.cuda())
            fn = deep_gemm.m_grouped_fp8_gemm_nt_contiguous
        d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        fn(a_arg, b_arg, d, layout)
        assert deep_gemm.device_status() == 0
        for rows, ref in refs:
            assert_close(d[rows], ref, f'm-grouped {num_groups} x {expected_m} n={n} k={k} trans_b={trans_b} rows {rows.start}')
        for span in oracle.psum_padding_spans(psum, 256):
            assert bool((d[span] == 0).all()), 'padding rows of D must be exactly zero'
        del d, b_arg


# tests/generators.py:620-627: (groups, M, N, expected K per group) of the weight-gradient GEMM at its EP64 / EP32 / EP16
# sizes; A [K, M] and B [K, N] hold the groups along K on the 256-row psum layout
K_GROUPED = [(4, 4096, 7168, 8192), (4, 7168, 2048, 8192), (8, 4096, 7168, 4096), (8, 7168, 2048, 4096),
             (16, 4096, 7168, 2048), (16, 7168, 2048, 2048)]


@pytest.mark.parametrize('num_groups,m,n,expected_k', K_GROUPED)
def test_k_grouped_reference_settings(num_groups, m, n, expected_k):
    """Group sizes as the reference draws them (`max(1, int(expected_k * U(0.7, 1.3)))`), then its three variants
    (tests/generators.py:606-613): all groups, a quarter of them empty (the first always, the last never), and a single
    non-empty group in the middle: all three with four groups (FP32 accumulation, direct BF16, BF16 accumulation), the
    second with eight and the first with sixteen. The whole [G, M, N] output is compared with the oracle (an empty group
    leaves zeros, or C untouched when accumulating)."""
    from test_gpu_k_grouped import _run
    random.seed(num_groups + m)
    real = [max(1, int(expected_k * random.uniform(0.7, 1.3))) for _ in range(num_groups)]
    empty = [0 if random.random() < 0.25 else s for s in real]
    empty[0], empty[-1] = 0, real[-1]
    single = [s if g == num_groups // 2 else 0 for g, s in enumerate(real)]
    if num_groups == 4:
        _run(m, n, tuple(real), out=torch.float32, acc=True, ks_hint='list', seed=1)
        _run(m, n, tuple(empty), out=torch.bfloat16, acc=False, ks_hint='none', seed=2)
        _run(m, n, tuple(single), out=torch.bfloat16, acc=True, ks_hint='empty', seed=3)
    else:                                       # 8 and 16 groups: one variant each, to keep the oracle's share short
        _run(m, n, tuple(empty if num_groups == 8 else real), out=torch.bfloat16, acc=False, ks_hint='list', seed=1)
