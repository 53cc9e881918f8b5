"""Packed-FP4 operands outside the K-major x K-major kernel: FP4 x FP4 with MN-major operands (the dgrad / wgrad
problems of tests/generators.py:571-576, which the reference's FP4 and dequant tests run like the forward ones),
m-grouped FP4 x FP4 with an MN-major B (tests/generators.py:597-603) and the k-grouped layout with FP8 x FP4 and
FP4 x FP4 operands (csrc/apis/gemm.hpp:325-384: "Supports fp8xfp8, fp4xfp4 and fp8xfp4").

Shapes whose packed operands satisfy the rules of TMA's 4-bit unpacking (32-byte strides, 128-element extents) are read
by the tensor cores as E2M1; the others are first expanded to E4M3, exactly. Both routes are compared with the CPU
oracle with the tolerance of tests/helpers.py.
"""

import pytest
import torch

import deep_gemm
import oracle
from helpers import assert_close, seed_all, uniform_fp4, uniform_fp8

pytestmark = pytest.mark.gpu


def _operand(kind, mn, k, mn_major):
    """(tensor as the API's logical [MN, K] view, scales [MN, K/32], dequantised [MN, K])."""
    if kind == 'fp4':
        return uniform_fp4(mn, k, (1, 32), mn_major=mn_major)
    data, sf, ref = uniform_fp8((mn, k), (1, 32))
    if mn_major:
        data = data.view(torch.uint8).t().contiguous().t().view(torch.float8_e4m3fn)
    return data, sf, ref


def _dense(kinds, m, n, k, trans, *, out=torch.bfloat16, acc=False, config=None, seed=0):
    seed_all(seed)
    a, sfa, a_ref = _operand(kinds[0], m, k, trans[0] == 't')
    b, sfb, b_ref = _operand(kinds[1], n, k, trans[1] == 'n')
    c = torch.randn(m, n).to(out) if acc else None
    ref = oracle.gemm_ref(a_ref, b_ref, out, c=c)
    a_dev, b_dev, sfa_dev, sfb_dev = a.cuda(), b.cuda(), sfa.cuda(), sfb.cuda()
    a_arg = (a_dev.transpose(0, 1), sfa_dev.transpose(0, 1)) if trans[0] == 't' else (a_dev, sfa_dev)
    b_arg = (b_dev.transpose(0, 1), sfb_dev.transpose(0, 1)) if trans[1] == 'n' else (b_dev, sfb_dev)
    d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
    kwargs = {}
    if acc:
        d.copy_(c)
        kwargs['c'] = d
    getattr(deep_gemm, f'fp8_fp4_gemm_{trans}')(a_arg, b_arg, d, recipe_a=(1, 32), recipe_b=(1, 32), config=config, **kwargs)
    assert deep_gemm.device_status() == 0
    return assert_close(d, ref, f'{kinds[0]}x{kinds[1]} {trans} {m}x{n}x{k} out={out} acc={acc} config={config}')


@pytest.mark.parametrize('trans', ['nn', 'tn', 'tt'])
@pytest.mark.parametrize('m,n,k', [(128, 128, 256), (256, 384, 1024), (512, 1280, 2048), (128, 2176, 7168)])
def test_fp4_pair_with_mn_major_operands_read_as_e2m1(trans, m, n, k):
    """Extents that are multiples of 128: TMA expands both packed operands and the MMA reads E2M1 x E2M1."""
    _dense(('fp4', 'fp4'), m, n, k, trans)
    _dense(('fp4', 'fp4'), m, n, k, trans, out=torch.float32, acc=True)


@pytest.mark.parametrize('trans', ['nn', 'tn', 'tt'])
@pytest.mark.parametrize('m,n,k', [(130, 258, 512), (64, 200, 1056), (4, 4, 16384), (16384, 4, 4), (300, 520, 96)])
def test_fp4_pair_with_mn_major_operands_of_any_extent(trans, m, n, k):
    """Extents TMA cannot unpack: the packed operand is expanded to E4M3 first (A), or decoded in shared memory (B)."""
    _dense(('fp4', 'fp4'), m, n, k, trans)


def test_fp4_pair_mn_major_tilings():
    # an MN-major B is fetched in 128-column atoms per CTA
    for cfg in ({'cta_group': 1, 'block_n': 128}, {'cta_group': 1, 'block_n': 256}, {'cta_group': 2, 'block_n': 256}):
        _dense(('fp4', 'fp4'), 512, 1024, 1024, 'tn', config=cfg)
        _dense(('fp4', 'fp4'), 512, 1024, 1024, 'nn', config=cfg)
    for cfg in ({'cta_group': 1, 'block_n': 64}, {'cta_group': 1, 'block_n': 224}, {'cta_group': 2, 'block_n': 128}):
        _dense(('fp4', 'fp4'), 512, 1344, 1024, 'tt', config=cfg)
    _dense(('fp4', 'fp4'), 128, 512, 8192, 'nn', config={'block_n': 128, 'split_k': 4})
    _dense(('fp4', 'fp4'), 4096, 2176, 7168, 'tn')                     # the heuristic's pick for a wgrad-sized problem


def test_benchmark_sized_backward_problems_in_fp4():
    """tests/generators.py:571-576 for (N, K) = (7168, 2048) and 4096 tokens with packed operands."""
    m, n, k = 4096, 7168, 2048
    _dense(('fp4', 'fp4'), m, k, n, 'nn')                               # dgrad: K-major A, MN-major B
    _dense(('fp4', 'fp4'), n, m, k, 'tn', out=torch.float32, acc=True)  # wgrad: both MN-major, FP32 accumulate
    _dense(('fp8', 'fp4'), n, m, k, 'tn')                               # FP8 A (MN-major) next to a packed MN-major B


@pytest.mark.parametrize('n,k', [(384, 1024), (520, 640)])
def test_fp4_pair_m_grouped_with_mn_major_b(n, k):
    seed_all(12)
    sizes = [300, 0, 513, 128]
    total, psum = oracle.make_psum_layout(sizes, 256)
    a, sfa, a_ref = uniform_fp4(total, k, (1, 32), mn_major=False)
    raw = a.clone()
    for span in oracle.psum_padding_spans(psum, 256):
        raw[span] = 0
        a_ref[span] = 0
    bs = [uniform_fp4(n, k, (1, 32), mn_major=True) for _ in sizes]
    # storage [G, K, N/2]; the API takes the transposed view of every group
    b = torch.stack([x[0].transpose(0, 1).contiguous() for x in bs]).cuda().transpose(1, 2)
    sfb = torch.stack([x[1] for x in bs])
    b_ref = torch.stack([x[2] for x in bs])
    ref = oracle.m_grouped_psum_ref(a_ref, b_ref, psum, torch.bfloat16)
    d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    deep_gemm.m_grouped_fp8_fp4_gemm_nn_contiguous((raw.cuda(), sfa.cuda()), (b.transpose(1, 2), sfb.cuda().transpose(1, 2)), d, layout,
                                                   recipe_a=(1, 32), recipe_b=(1, 32))
    assert deep_gemm.device_status() == 0
    out = d.cpu()
    for span in oracle.psum_valid_spans(psum, 256):
        assert_close(out[span], ref[span], f'fp4xfp4 m-grouped, MN-major B, n={n} k={k}')
    for span in oracle.psum_padding_spans(psum, 256):
        assert bool((out[span] == 0).all())


def _k_grouped(kinds, m, n, sizes, *, out=torch.bfloat16, acc=False, seed=0):
    """A [K, M] and B [K, N] with K holding the groups on the 256-row psum layout (tests/generators.py:361-398)."""
    seed_all(seed)
    total_k, psum = oracle.make_psum_layout(list(sizes), 256)
    ops = []
    for kind, mn in zip(kinds, (m, n)):
        data, sf, _ = _operand(kind, mn, total_k, True)                 # logical [MN, K], MN contiguous
        store = data.transpose(0, 1)                                     # [K, MN or MN/2], contiguous rows
        raw = store.contiguous().view(torch.uint8).clone() if kind == 'fp8' else store.contiguous().clone()
        for span in oracle.psum_padding_spans(psum, 256):
            raw[span] = 0
        vals = (raw.view(torch.float8_e4m3fn).float() if kind == 'fp8' else oracle.decode_e2m1_packed(raw, axis=-1))   # [K, MN]
        sf_t = sf.transpose(0, 1).contiguous()                           # [K/32, MN]
        deq = oracle.dequantize(vals, sf_t, 32, 1)
        for span in oracle.psum_padding_spans(psum, 256, 32):
            sf_t[span] = torch.randn_like(sf_t[span])                    # garbage scales inside the padding
        ops.append((raw.view(torch.float8_e4m3fn) if kind == 'fp8' else raw, sf_t, deq))
    (a, sfa, a_deq), (b, sfb, b_deq) = ops
    g = len(sizes)
    c = torch.randn(g, m, n).to(out) if acc else None
    ref = oracle.k_grouped_psum_ref(a_deq, b_deq, psum, out, c=c)
    d = torch.full((g, m, n), float('nan'), dtype=out, device='cuda')
    kwargs = {}
    if acc:
        d.copy_(c)
        kwargs['c'] = d
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    deep_gemm.k_grouped_fp8_gemm_tn_contiguous((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d,
                                               [oracle.align(s, 256) for s in sizes], layout, recipe=(1, 1, 32), **kwargs)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref, f'k-grouped {kinds[0]}x{kinds[1]} {m}x{n} sizes={sizes} out={out} acc={acc}')


@pytest.mark.parametrize('kinds', [('fp8', 'fp4'), ('fp4', 'fp4')])
@pytest.mark.parametrize('m,n,sizes', [(256, 384, (700, 300, 1024, 33)), (128, 128, (0, 512, 0, 640)), (512, 1024, (2048 + 16, 2048 - 16)),
                                       (130, 200, (900, 1300, 512)), (4, 4, (1, 1, 1, 1))])
def test_k_grouped_with_packed_operands(kinds, m, n, sizes):
    _k_grouped(kinds, m, n, sizes)
    _k_grouped(kinds, m, n, sizes, out=torch.float32, acc=True, seed=1)


def test_k_grouped_packed_at_a_benchmark_size():
    _k_grouped(('fp8', 'fp4'), 4096, 7168, (2100, 1900, 0, 2048))
    _k_grouped(('fp4', 'fp4'), 7168, 2048, (2100, 1900, 0, 2048), out=torch.float32, acc=True)


def test_operand_kinds_that_stay_rejected():
    a = torch.zeros(128, 64, dtype=torch.int8, device='cuda')
    b = torch.zeros(128, 128, dtype=torch.float8_e4m3fn, device='cuda')
    sf = torch.ones(128, 4, dtype=torch.float32, device='cuda')
    d = torch.zeros(128, 128, dtype=torch.bfloat16, device='cuda')
    with pytest.raises(RuntimeError, match='Unsupported operand dtypes'):
        deep_gemm.fp8_fp4_gemm_nt((a, sf), (b, sf), d)


# The reference's shape lists for odd extents (tests/generators.py:466-541), which its FP4 and dequant tests run over the
# four major combinations with FP32 accumulation. An odd extent along a packed operand's contiguous axis is doubled,
# as the reference's generator does (two codes share a byte).
EXTRA_SHAPES = [(4, 4, 4), (4, 4, 16384), (4, 16384, 4), (16384, 4, 4), (16384, 4, 16384), (4, 16384, 16384), (128, 128, 128),
                (256, 512, 1024), (1024, 256, 512), (4096, 4096, 4096)]
UNALIGNED_MN = [(4, 4, 64), (17, 4096, 4096), (4096, 17, 4096), (15, 4096, 4096), (4096, 15, 4096), (130, 257, 2048), (513, 257, 4096)]
UNALIGNED_K = [(64, 64, 4), (1024, 2048, 17), (8192, 4096, 15), (128, 128, 234), (2048, 8192, 4095)]


@pytest.mark.parametrize('kinds', [('fp4', 'fp4'), ('fp8', 'fp4')])
@pytest.mark.parametrize('m,n,k', EXTRA_SHAPES + UNALIGNED_MN + UNALIGNED_K)
def test_reference_shape_lists_with_packed_operands_all_majors(kinds, m, n, k):
    if kinds[0] == 'fp8' and m * n * k == 4 * 16384 * 16384:
        pytest.skip('the two 268M-element operands are generated once, for the FP4 x FP4 kind')
    for trans in ('nt', 'nn', 'tn', 'tt'):
        mm = m * 2 if (kinds[0] == 'fp4' and trans[0] == 't' and m % 2) else m
        nn = n * 2 if (trans[1] == 'n' and n % 2) else n
        kk = k * 2 if k % 2 else k
        _dense(kinds, mm, nn, kk, trans, out=torch.float32, acc=True)
