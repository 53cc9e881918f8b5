"""Parity of the BF16 GEMM family (kind::f16 MMAs, no scale factors) with the CPU oracle.

Same tolerance as the FP8 tests (tests/helpers.py); products of BF16 values are exact in FP32, so the only difference
from the oracle is the order of the FP32 additions."""

import pytest
import torch

import deep_gemm
import oracle
from helpers import assert_close, seed_all, with_major

pytestmark = pytest.mark.gpu


def _dense(m, n, k, trans='nt', out=torch.bfloat16, acc=False, bias=False, alpha=None, config=None, seed=0):
    seed_all(seed)
    a, b = torch.randn(m, k).bfloat16(), torch.randn(n, k).bfloat16()
    c = torch.randn(1 if bias else m, n).to(out) if (acc or bias) else None
    ref = oracle.gemm_ref(a.float(), b.float(), out, c=c if acc else None, bias=c if bias else None, alpha=alpha)
    a_dev, b_dev = with_major(a, trans[0] == 't').cuda(), with_major(b, trans[1] == 'n').cuda()
    a_arg = a_dev.transpose(0, 1) if trans[0] == 't' else a_dev
    b_arg = b_dev.transpose(0, 1) if trans[1] == 'n' else b_dev
    d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
    kwargs = {}
    if acc:
        d.copy_(c)
        kwargs['c'] = d
    elif bias:
        kwargs['c'] = c.cuda()
    getattr(deep_gemm, f'bf16_gemm_{trans}')(a_arg, b_arg, d, alpha=alpha, config=config, **kwargs)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref, f'bf16 {trans} {m}x{n}x{k} out={out} acc={acc} bias={bias} config={config}')


@pytest.mark.parametrize('trans', ['nt', 'nn', 'tn', 'tt'])
def test_dense_all_majors(trans):
    _dense(128, 128, 64, trans)
    _dense(256, 384, 512, trans)
    _dense(384, 256, 1024, trans, out=torch.float32, acc=True)
    _dense(4096, 512, 2048, trans)


def test_dense_shapes_and_epilogues():
    for m, n, k in ((64, 2112, 7168), (1, 576, 512), (130, 264, 2048), (513, 264, 1000), (128, 128, 72)):
        _dense(m, n, k)
        _dense(m, n, k, out=torch.float32, acc=True)
    _dense(256, 384, 512, bias=True)
    _dense(256, 384, 512, alpha=-0.375)
    _dense(256, 384, 512, out=torch.float32, bias=True)


def test_dense_tilings():
    for bn in (32, 64, 96, 128, 160, 192, 224, 256):
        _dense(384, 768, 1024, config={'block_n': bn})
        _dense(512, 768, 1024, config={'cta_group': 2, 'block_n': bn})
    _dense(512, 512, 1024, trans='nn', config={'cta_group': 2, 'block_n': 128})
    _dense(512, 512, 1024, trans='tn', config={'cta_group': 1, 'block_n': 64})
    _dense(128, 512, 4096, config={'block_n': 128, 'split_k': 4})
    _dense(128, 512, 4096, config={'block_n': 128, 'split_k': 4, 'cluster_split': 1})
    # wide tiles: two column halves per K step sharing the A tile; without scale columns TMEM holds 2 x 256
    for bn in (320, 384, 448, 512):
        _dense(512, 1100, 1024, config={'cta_group': 2, 'block_n': bn})
        _dense(300, 2 * bn + 8, 512, config={'cta_group': 2, 'block_n': bn}, out=torch.float32, acc=True)
    with pytest.raises(RuntimeError):
        _dense(512, 1024, 1024, trans='nn', config={'cta_group': 2, 'block_n': 320})


def test_golden_fixtures(golden):
    for name, trans in (('bf16_dense_nt', 'nt'), ('bf16_dense_tn_acc_f32', 'tn'), ('bf16_dense_nn_bias', 'nn')):
        c = golden[name]
        a_dev, b_dev = with_major(c['a'], trans[0] == 't').cuda(), with_major(c['b'], trans[1] == 'n').cuda()
        a_arg = a_dev.transpose(0, 1) if trans[0] == 't' else a_dev
        b_arg = b_dev.transpose(0, 1) if trans[1] == 'n' else b_dev
        d = torch.zeros_like(c['d']).cuda()
        kwargs = {}
        if c['accumulate']:
            d.copy_(c['c'])
            kwargs['c'] = d
        elif c['with_bias']:
            kwargs['c'] = c['c'].cuda()
        getattr(deep_gemm, f'bf16_gemm_{trans}')(a_arg, b_arg, d, **kwargs)
        assert_close(d, c['d'], name)
    c = golden['bf16_mgrouped_nt']
    d = torch.full(c['d'].shape, float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.m_grouped_bf16_gemm_nt_contiguous(c['a'].cuda(), c['b'].cuda(), d, torch.tensor(c['psum'], dtype=torch.int32, device='cuda'))
    assert_close(d, c['d'], 'bf16_mgrouped_nt')
    pad = torch.ones(c['d'].size(0), dtype=torch.bool)
    for span in oracle.psum_valid_spans(c['psum'], 256):
        pad[span] = False
    assert d.cpu()[pad].abs().max().item() == 0                      # padding rows of A are zero, so D is zero there
    c = golden['bf16_kgrouped_acc_f32']
    d = c['c'].clone().cuda()
    deep_gemm.k_grouped_bf16_gemm_tn_contiguous(c['a'].cuda(), c['b'].cuda(), d, None,
                                                torch.tensor(c['psum'], dtype=torch.int32, device='cuda'), c=d)
    assert_close(d, c['d'], 'bf16_kgrouped_acc_f32')


@pytest.mark.parametrize('trans_b', [False, True])
def test_m_grouped(trans_b):
    seed_all(2)
    sizes = [300, 0, 513, 128, 1]
    total, psum = oracle.make_psum_layout(sizes, 256)
    n, k = 384, 1024
    a = torch.randn(total, k).bfloat16()
    for span in oracle.psum_padding_spans(psum, 256):
        a[span] = 0
    b = torch.randn(len(sizes), n, k).bfloat16()
    ref = oracle.m_grouped_psum_ref(a.float(), b.float(), psum, torch.bfloat16)
    d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    if trans_b:
        deep_gemm.m_grouped_bf16_gemm_nn_contiguous(a.cuda(), b.transpose(1, 2).contiguous().cuda(), d, layout)
    else:
        deep_gemm.m_grouped_bf16_gemm_nt_contiguous(a.cuda(), b.cuda(), d, layout)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref, f'bf16 m-grouped trans_b={trans_b}')


@pytest.mark.parametrize('out,acc', [(torch.float32, True), (torch.bfloat16, False)])
def test_k_grouped(out, acc):
    seed_all(3)
    sizes = [700, 0, 1024, 33]
    total_k, psum = oracle.make_psum_layout(sizes, 256)
    m, n = 256, 384
    a, b = torch.randn(total_k, m).bfloat16(), torch.randn(total_k, n).bfloat16()
    for span in oracle.psum_padding_spans(psum, 256):
        a[span] = 0
        b[span] = 0
    c = torch.randn(len(sizes), m, n).to(out) if acc else None
    ref = oracle.k_grouped_psum_ref(a.float(), b.float(), psum, out, c=c)
    d = torch.full((len(sizes), m, n), float('nan'), dtype=out, device='cuda')
    kwargs = {}
    if acc:
        d.copy_(c)
        kwargs['c'] = d
    deep_gemm.k_grouped_bf16_gemm_tn_contiguous(a.cuda(), b.cuda(), d, [oracle.align(s, 256) for s in sizes],
                                                torch.tensor(psum, dtype=torch.int32, device='cuda'), **kwargs)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref, f'bf16 k-grouped out={out} acc={acc}')
    if not acc:
        assert d[1].abs().max().item() == 0


def test_argument_checks():
    a = torch.zeros(128, 64, dtype=torch.bfloat16, device='cuda')
    d = torch.zeros(128, 128, dtype=torch.bfloat16, device='cuda')
    with pytest.raises(RuntimeError):
        deep_gemm.bf16_gemm_nt(a, a.to(torch.float8_e4m3fn), d)
    b = torch.zeros(128, 60, dtype=torch.bfloat16, device='cuda')
    deep_gemm.bf16_gemm_nt(b, b, d)              # rows 120 bytes apart are repacked to a 16-byte pitch by the host layer
    deep_gemm.bf16_gemm_nt(a[:, :60], a[:, :60], d)
    assert d.abs().max().item() == 0


# tests/generators.py:491-541 through tests/test_bf16_gemm.py: extents that are not multiples of 16 bytes, every major pair
@pytest.mark.parametrize('m,n,k', [(4, 4, 64), (17, 4096, 4096), (4096, 15, 4096), (130, 257, 2048), (513, 257, 4096),
                                   (64, 64, 4), (1024, 2048, 17), (8192, 4096, 15), (128, 128, 234), (2048, 8192, 4095)])
def test_reference_odd_extent_lists_all_majors(m, n, k):
    for trans in ('nt', 'nn', 'tn', 'tt'):
        _dense(m, n, k, trans, out=torch.float32, acc=True)


@pytest.mark.parametrize('batch,m,n,k', [(4, 128, 256, 512), (3, 130, 200, 1000), (8, 64, 64, 64)])
def test_bf16_bmm(batch, m, n, k):
    seed_all(batch)
    a, b = torch.randn(batch, m, k).bfloat16(), torch.randn(batch, n, k).bfloat16()
    prod = torch.einsum('bmk,bnk->bmn', a.float(), b.float())
    d = torch.full((batch, m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.bf16_bmm(a.cuda(), b.cuda(), d)
    assert_close(d, prod.to(torch.bfloat16), f'bf16_bmm {batch}x{m}x{n}x{k}')
    c = torch.randn(batch, m, n)
    d32 = c.cuda()
    deep_gemm.bf16_bmm(a.cuda(), b.cuda(), d32, c=d32)
    assert deep_gemm.device_status() == 0
    assert_close(d32, prod + c, f'bf16_bmm accumulate {batch}x{m}x{n}x{k}')


@pytest.mark.parametrize('expr', ['bhr,hdr->bhd', 'bhd,hdr->bhr', 'bhd,bhr->hdr'])
@pytest.mark.parametrize('b_,h,r,d_', [(4, 2, 2, 2), (32, 128, 512, 128), (128, 8, 4096, 1024), (4096, 8, 512, 128)])
def test_bf16_einsum(expr, b_, h, r, d_):
    """csrc/apis/einsum.hpp:102-145 on sizes of tests/generators.py:778-786 (inputs N(0, 0.1), the weight-gradient
    expression accumulates into FP32, the other two write BF16)."""
    seed_all(b_ + h)
    shapes = {'bhr,hdr->bhd': ((b_, h, r), (h, d_, r), (b_, h, d_)), 'bhd,hdr->bhr': ((b_, h, d_), (h, d_, r), (b_, h, r)),
              'bhd,bhr->hdr': ((b_, h, d_), (b_, h, r), (h, d_, r))}[expr]
    a = (torch.randn(shapes[0]) * 0.1).bfloat16()
    b = (torch.randn(shapes[1]) * 0.1).bfloat16()
    ref = torch.einsum(expr, a.float(), b.float())
    if expr == 'bhd,bhr->hdr':
        c = torch.randn(shapes[2]) * 0.1
        d = c.cuda()
        deep_gemm.einsum(expr, a.cuda(), b.cuda(), d, c=d)
        ref = ref + c
    else:
        d = torch.full(shapes[2], float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.einsum(expr, a.cuda(), b.cuda(), d)
        ref = ref.to(torch.bfloat16)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref, f'einsum {expr} b={b_} h={h} r={r} d={d_}')
    with pytest.raises(RuntimeError, match='Unsupported einsum expression'):
        deep_gemm.einsum('bh,hd->bd', a.cuda(), b.cuda(), d)
