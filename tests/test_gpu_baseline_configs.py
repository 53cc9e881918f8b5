"""Parity at the sizes the five benchmark configurations name, with the tiling the heuristic itself picks.

Every case goes through the public API (and so through the C ABI) without a `config=` override, on operands
generated on the CPU with a fixed seed, and is compared with the CPU oracle: the whole output where the oracle
finishes in seconds, whole 256-row blocks of every group where it would not (the 32-expert grouped GEMM). The
tolerance is the one of tests/helpers.py (1 - cosine <= 1e-3, max relative error <= 2e-2); padding rows and the two
spellings of the mixed-precision recipe are compared bit for bit.

Case lists follow the reference's tests/generators.py:544-576 (forward shapes, dgrad / wgrad majors) and :579-603
(m-grouped), at the shapes of the benchmark sweep.
"""

import random

import pytest
import torch

import deep_gemm
import oracle
from helpers import (assert_close, assert_close_device, pow2_scales, seed_all, uniform_codes, uniform_fp4, uniform_fp8,
                     with_major)

pytestmark = pytest.mark.gpu

NK_LIST = [(2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]


# ----------------------------------------------------------------------------------------------------------------
# Configurations 1 and 2: the dense NT sweep, plain / [1, N] bias / FP32 accumulate into D
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('n,k', NK_LIST)
def test_dense_sweep_shapes_all_variants(n, k):
    """M in {64, 128, 4096} for one (N, K) of the sweep: N(0,1) data, A scaled per 1x128 and B per 128x128, scales
    handed over as FP32 with recipe (1, 128, 128) exactly as the benchmark's end-to-end leg does."""
    seed_all(n + k)
    b, sfb, b_ref = oracle.quantize_e4m3(torch.randn(n, k), (128, 128))
    b_dev, sfb_dev = b.cuda(), sfb.cuda()
    for m in (64, 128, 4096):
        a, sfa, a_ref = oracle.quantize_e4m3(torch.randn(m, k), (1, 128))
        prod = a_ref @ b_ref.T                                   # the oracle's FP32 product, shared by the variants
        a_arg, b_arg = (a.cuda(), sfa.cuda()), (b_dev, sfb_dev)
        # plain BF16 output
        d = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.fp8_gemm_nt(a_arg, b_arg, d, recipe=(1, 128, 128))
        assert_close_device(d, prod.to(torch.bfloat16), f'dense {m}x{n}x{k}')
        # [1, N] BF16 bias
        bias = torch.randn(1, n).to(torch.bfloat16)
        d = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.fp8_gemm_nt(a_arg, b_arg, d, c=bias.cuda(), recipe=(1, 128, 128))
        assert_close_device(d, (prod + bias.float()).to(torch.bfloat16), f'dense {m}x{n}x{k} + bias')
        # FP32 D pre-filled, accumulated into (c is d)
        c = torch.randn(m, n)
        d = c.cuda()
        deep_gemm.fp8_gemm_nt(a_arg, b_arg, d, c=d, recipe=(1, 128, 128))
        assert_close_device(d, prod + c, f'dense {m}x{n}x{k} accumulate')
        del prod, c, d
    assert deep_gemm.device_status() == 0


@pytest.mark.parametrize('n,k', [(2112, 7168), (7168, 2048)])
def test_dense_backward_majors_at_4096_rows(n, k):
    """tests/generators.py:571-576 for a forward weight [n, k] and 4096 tokens: dgrad = K-major A times MN-major B
    (4096 x k x n, BF16 out); wgrad = both operands MN-major (n x 4096 x k), FP32 accumulate and plain BF16."""
    m = 4096
    seed_all(n * 3 + k)
    # dgrad: problem (m, k, n): D [m, k] = A [m, n] @ B [k, n]^T with B stored [n, k] (MN-major)
    a, sfa, a_ref = uniform_fp8((m, n), (1, 32))
    b, sfb, b_ref = uniform_fp8((k, n), (1, 32))
    b_dev = with_major(b, True).cuda()
    d = torch.full((m, k), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nn((a.cuda(), sfa.cuda()), (b_dev.transpose(0, 1), sfb.cuda().transpose(0, 1)), d)
    assert_close_device(d, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16), f'dgrad {m}x{k}x{n}')
    # wgrad: problem (n, m, k): D [n, m] = A [n, k] @ B [m, k]^T, both stored with MN contiguous
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


# ----------------------------------------------------------------------------------------------------------------
# Configuration 3: FP8 x packed FP4, NN, 4096 x 7168 x 2048, A per 128 and B per 32
# ----------------------------------------------------------------------------------------------------------------
def test_mixed_fp8_fp4_nn_at_benchmark_size_both_recipe_spellings():
    m, n, k = 4096, 7168, 2048
    seed_all(3)
    a, sfa, a_ref = oracle.quantize_e4m3(torch.randn(m, k), (1, 128))
    b, sfb, b_ref = uniform_fp4(n, k, (1, 32), mn_major=True)                  # storage [K, N/2], scales from {.25, .5, 1}
    ref = oracle.gemm_ref(a_ref, b_ref, torch.bfloat16)
    a_dev, b_dev = a.cuda(), b.cuda()
    b_arg = (b_dev.transpose(0, 1), sfb.cuda().transpose(0, 1))
    # the spelling the benchmark uses: per-128 scales on A next to per-32 scales on B
    d1 = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_fp4_gemm_nn((a_dev, sfa.cuda()), b_arg, d1, recipe_a=(1, 128), recipe_b=(1, 32))
    assert_close_device(d1, ref, 'fp8xfp4 nn 4096x7168x2048, recipe_a=(1,128) recipe_b=(1,32)')
    # the spelling the reference accepts: A's scales repeated over the four 32-blocks they cover, recipe (1, 1, 32)
    sfa32 = sfa.repeat_interleave(4, dim=1).contiguous()
    d2 = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_fp4_gemm_nn((a_dev, sfa32.cuda()), b_arg, d2, recipe=(1, 1, 32))
    assert deep_gemm.device_status() == 0
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16)), 'the two recipe spellings must give the same bits'


# ----------------------------------------------------------------------------------------------------------------
# Configuration 4: m-grouped contiguous, per-expert M ~ U(0.7, 1.3) x 8192 on the 256-row psum layout
# ----------------------------------------------------------------------------------------------------------------
def _expert_sizes(num_groups: int, seed: int) -> list[int]:
    random.seed(seed)
    return [int(random.uniform(0.7, 1.3) * 8192) for _ in range(num_groups)]


@pytest.mark.parametrize('n,k,trans_b', [(4096, 7168, False), (7168, 2048, True)])
def test_m_grouped_contiguous_8_experts_full_tensor(n, k, trans_b):
    """Eight experts, the whole D against the oracle. N(0,1) data quantised per 1x128 / 128x128; padding rows of A
    are zero, padding rows of the scales are garbage (tests/generators.py:338-346)."""
    g = 8
    sizes = _expert_sizes(g, seed=8)
    total, psum = oracle.make_psum_layout(sizes, 256)
    seed_all(n + g)
    a = torch.zeros(total, k, dtype=torch.uint8)
    sfa = torch.randn(total, k // 128)                        # garbage wherever no valid row overwrites it
    ref = torch.zeros(total, n, dtype=torch.bfloat16)
    bs, sfbs = [], []
    for gi, span in enumerate(oracle.psum_valid_spans(psum, 256)):
        aq, asf, a_ref = oracle.quantize_e4m3(torch.randn(span.stop - span.start, k), (1, 128))
        bq, bsf, b_ref = oracle.quantize_e4m3(torch.randn(n, k), (128, 128))
        a[span] = aq.view(torch.uint8)
        sfa[span] = asf
        ref[span] = (a_ref @ b_ref.T).to(torch.bfloat16)
        bs.append(bq.view(torch.uint8)); sfbs.append(bsf)
    b = torch.stack(bs).view(torch.float8_e4m3fn)
    sfb = torch.stack(sfbs)
    b_dev = with_major(b, trans_b).cuda()
    b_arg = (b_dev.transpose(1, 2), sfb.cuda().transpose(1, 2)) if trans_b else (b_dev, sfb.cuda())
    d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    fn = deep_gemm.m_grouped_fp8_gemm_nn_contiguous if trans_b else deep_gemm.m_grouped_fp8_gemm_nt_contiguous
    fn((a.view(torch.float8_e4m3fn).cuda(), sfa.cuda()), b_arg, d, layout, recipe=(1, 128, 128))
    assert deep_gemm.device_status() == 0
    assert_close_device(d, ref, f'm-grouped 8 experts n={n} k={k} trans_b={trans_b}')
    for span in oracle.psum_padding_spans(psum, 256):
        assert bool((d[span] == 0).all()), 'padding rows of D must be exactly zero'


@pytest.mark.parametrize('n,k', [(4096, 7168), (7168, 2048)])
def test_m_grouped_contiguous_32_experts_sampled_blocks(n, k):
    """Thirty-two experts (about 262 000 rows): the oracle checks every group's first and last 256-row block and one
    random block of each group, for K-major and MN-major B; every padding row of D must be exactly zero. Uniform
    E4M3 codes with per-1x32 power-of-two scales, the distribution of the reference's own m-grouped test."""
    g = 32
    sizes = _expert_sizes(g, seed=32)
    total, psum = oracle.make_psum_layout(sizes, 256)
    seed_all(k + g)
    a = uniform_codes((total, k))
    sfa = pow2_scales((total, k // 32))
    for span in oracle.psum_padding_spans(psum, 256):
        a[span] = 0
        sfa[span] = torch.randn_like(sfa[span])
    b = uniform_codes((g, n, k))
    sfb = pow2_scales((g, n, k // 32))
    a_dev, sfa_dev = a.view(torch.float8_e4m3fn).cuda(), sfa.cuda()
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    # blocks to check: (group, first row)
    blocks = []
    for gi, span in enumerate(oracle.psum_valid_spans(psum, 256)):
        first, last = span.start, (span.stop - 1) // 256 * 256
        blocks += [(gi, first), (gi, last), (gi, random.randrange(first, last + 1, 256))]
    refs = {}
    for gi in range(g):
        b_ref = oracle.dequantize(b[gi].view(torch.float8_e4m3fn).float(), sfb[gi], 1, 32)
        for (gj, r0) in blocks:
            if gj == gi and (gi, r0) not in refs:
                rows = slice(r0, r0 + 256)
                a_blk = oracle.dequantize(a[rows].view(torch.float8_e4m3fn).float(), sfa[rows], 1, 32)
                a_blk[max(0, psum[gi] - r0):] = 0                 # padding rows inside the group's last block
                refs[(gi, r0)] = (a_blk @ b_ref.T).to(torch.bfloat16)
    for trans_b in (False, True):
        b8 = b.view(torch.float8_e4m3fn)
        if trans_b:
            b_dev = b8.cuda().view(torch.uint8).transpose(1, 2).contiguous().transpose(1, 2).view(torch.float8_e4m3fn)
            b_arg = (b_dev.transpose(1, 2), sfb.cuda().transpose(1, 2))
            fn = deep_gemm.m_grouped_fp8_gemm_nn_contiguous
        else:
            b_arg = (b8.cuda(), sfb.cuda())
            fn = deep_gemm.m_grouped_fp8_gemm_nt_contiguous
        d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        fn((a_dev, sfa_dev), b_arg, d, layout)
        assert deep_gemm.device_status() == 0
        for (gi, r0), ref in refs.items():
            assert_close(d[r0:r0 + 256], ref, f'm-grouped 32 experts n={n} k={k} trans_b={trans_b} group {gi} rows {r0}')
        for span in oracle.psum_padding_spans(psum, 256):
            assert bool((d[span] == 0).all()), 'padding rows of D must be exactly zero'
        del d, b_arg


# ----------------------------------------------------------------------------------------------------------------
# Configuration 5: m-grouped masked, 32 experts x 256 rows, valid rows ~ U[0, 256]
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('n,k', [(4096, 7168), (7168, 2048)])
def test_m_grouped_masked_32_experts_at_benchmark_size(n, k):
    g, max_m = 32, 256
    random.seed(5)
    masked = [random.randint(0, max_m) for _ in range(g)]
    masked[3], masked[7] = 0, max_m                       # an empty and a full expert are always among them
    seed_all(n)
    a = uniform_codes((g, max_m, k))
    sfa = pow2_scales((g, max_m, k // 32))
    b = uniform_codes((g, n, k))
    sfb = pow2_scales((g, n, k // 32))
    d = torch.full((g, max_m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    mask = torch.tensor(masked, dtype=torch.int32, device='cuda')
    deep_gemm.m_grouped_fp8_gemm_nt_masked((a.view(torch.float8_e4m3fn).cuda(), sfa.cuda()),
                                           (b.view(torch.float8_e4m3fn).cuda(), sfb.cuda()), d, mask,
                                           sum(masked) // g)
    assert deep_gemm.device_status() == 0
    for gi, mg in enumerate(masked):
        if mg == 0:
            continue
        a_ref = oracle.dequantize(a[gi, :mg].view(torch.float8_e4m3fn).float(), sfa[gi, :mg], 1, 32)
        b_ref = oracle.dequantize(b[gi].view(torch.float8_e4m3fn).float(), sfb[gi], 1, 32)
        assert_close(d[gi, :mg], (a_ref @ b_ref.T).to(torch.bfloat16), f'masked n={n} k={k} group {gi} rows {mg}')
