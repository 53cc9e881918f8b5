"""Parity of the CUDA GEMM path (through the Python API and the C ABI) with the CPU oracle.

Tolerance on the output: 1 - cosine <= 1e-3 and max relative error <= 2e-2 (see tests/helpers.py); padding rows,
group handling and scale-factor layouts are compared bit-exactly.
"""

import pytest
import torch

import deep_gemm
import oracle
from helpers import assert_close, normal_fp8, seed_all, uniform_fp4, uniform_fp8, with_major

pytestmark = pytest.mark.gpu


def _dense(m, n, k, *, trans='nt', recipe=(1, 1, 32), dist='uniform', out=torch.bfloat16, acc=False, bias=False,
           alpha=None, config=None, seed=0):
    seed_all(seed)
    gm, gn, gk = recipe
    gen = uniform_fp8 if dist == 'uniform' else normal_fp8
    a, sfa, a_ref = gen((m, k), (gm, gk))
    b, sfb, b_ref = gen((n, k), (gn, gk))
    c = torch.randn(1 if bias else m, n).to(out) if (acc or bias) else None
    ref = oracle.gemm_ref(a_ref, b_ref, out, c=c if acc else None, bias=c if bias else None, alpha=alpha)
    a_dev = with_major(a, trans[0] == 't').cuda()
    b_dev = with_major(b, trans[1] == 'n').cuda()
    a_arg = (a_dev.transpose(0, 1), sfa.cuda().transpose(0, 1)) if trans[0] == 't' else (a_dev, sfa.cuda())
    b_arg = (b_dev.transpose(0, 1), sfb.cuda().transpose(0, 1)) if trans[1] == 'n' else (b_dev, sfb.cuda())
    d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
    kwargs = {}
    if acc:
        d.copy_(c)
        kwargs['c'] = d
    elif bias:
        kwargs['c'] = c.cuda()
    getattr(deep_gemm, f'fp8_gemm_{trans}')(a_arg, b_arg, d, recipe=recipe, alpha=alpha, config=config, **kwargs)
    assert deep_gemm.device_status() == 0
    return assert_close(d, ref, f'{trans} {m}x{n}x{k} recipe={recipe} {dist} out={out} acc={acc} bias={bias} alpha={alpha}')


@pytest.mark.parametrize('m,n,k', [(128, 128, 128), (128, 256, 512), (256, 192, 1024), (64, 2112, 7168),
                                   (1, 576, 512), (384, 7168, 256)])
def test_dense_nt_bf16(m, n, k):
    _dense(m, n, k)


def test_dense_nt_baseline_distribution_and_recipe():
    """N(0,1) data, per-1x128 scales on A and 128x128 on B: the distribution the benchmark uses."""
    _dense(128, 2112, 7168, recipe=(1, 128, 128), dist='normal')
    _dense(320, 512, 1024, recipe=(1, 128, 128), dist='normal', out=torch.float32)


@pytest.mark.parametrize('recipe', [(1, 32, 32), (32, 1, 32), (32, 32, 32), (128, 128, 32)])
def test_dense_recipes(recipe):
    _dense(200, 328, 640, recipe=recipe, out=torch.float32, acc=True)


@pytest.mark.parametrize('m,n,k', [(4, 4, 64), (17, 512, 1024), (512, 17, 1024), (15, 1024, 512), (130, 257, 2048),
                                   (513, 257, 1024)])
def test_dense_unaligned_mn(m, n, k):
    _dense(m, n, k, out=torch.float32, acc=True)
    _dense(m, n, k, out=torch.bfloat16)


@pytest.mark.parametrize('m,n,k', [(64, 64, 4), (256, 512, 17), (512, 256, 15), (128, 128, 234), (256, 384, 4095)])
def test_dense_unaligned_k(m, n, k):
    _dense(m, n, k, out=torch.float32, acc=True)


@pytest.mark.parametrize('out', [torch.bfloat16, torch.float32])
def test_dense_epilogues(out):
    _dense(256, 384, 512, out=out, bias=True)
    _dense(256, 384, 512, out=out, alpha=-0.375)
    _dense(256, 384, 512, out=out, acc=True)
    _dense(256, 384, 512, out=out, acc=True, alpha=0.625)


@pytest.mark.parametrize('trans', ['nn', 'tn', 'tt'])
def test_dense_majors(trans):
    _dense(256, 384, 512, trans=trans)
    _dense(384, 256, 1024, trans=trans, out=torch.float32, acc=True)


def test_dense_forced_tilings():
    for bn in (64, 128, 192, 256):
        _dense(384, 768, 1024, config={'block_n': bn})
    for stages in (1, 2, 3):
        _dense(256, 256, 2048, config={'block_n': 128, 'num_stages': stages})
    for split in (2, 4, 7):
        _dense(128, 512, 4096, config={'block_n': 128, 'split_k': split})
        _dense(128, 512, 4096, config={'block_n': 128, 'split_k': split}, bias=True)
        _dense(100, 500, 4096, config={'block_n': 96, 'split_k': split}, out=torch.float32, acc=True)
    # a second split-K launch must find the workspace zeroed by the first one
    _dense(128, 512, 4096, config={'block_n': 128, 'split_k': 4}, seed=1)


@pytest.mark.parametrize('bn,split', [(32, 2), (64, 3), (64, 8), (96, 3), (96, 5), (128, 2), (128, 4), (128, 5),
                                      (160, 2), (160, 3), (192, 2)])
def test_dense_cluster_split_k(bn, split):
    """The K splits of one tile run as one thread-block cluster: every rank pushes its partial sums of the
    32-column chunks it does not own into the owner's shared memory; the owner adds them in rank order."""
    cfg = {'block_n': bn, 'split_k': split, 'cluster_split': 1}
    _dense(128, 512, 4096, config=cfg)
    _dense(128, 512, 4096, config=cfg, bias=True)
    _dense(100, 500, 4096, config=cfg, out=torch.float32, acc=True)
    _dense(64, 2112, 7168, config=cfg, out=torch.float32)


def test_dense_cluster_split_k_variants():
    cfg = {'block_n': 128, 'split_k': 4, 'cluster_split': 1}
    _dense(300, 640, 2048, config=cfg)                                  # three row blocks, each its own clusters
    _dense(128, 4096, 7168, config=cfg, dist='normal', recipe=(1, 128, 128), alpha=0.5)
    _dense(128, 516, 2000, config=cfg, out=torch.bfloat16, acc=True)    # K tail, odd N: plain stores / atomics
    _dense(128, 1000, 4096, config={'block_n': 96, 'split_k': 3, 'cluster_split': 1}, trans='tt')    # MN-major A
    # the result is the sum of the partials in rank order: two runs agree bit for bit
    seed_all(7)
    a, sfa, _ = uniform_fp8((128, 4096), (1, 32))
    b, sfb, _ = uniform_fp8((1024, 4096), (1, 32))
    outs = []
    for _ in range(2):
        d = torch.empty(128, 1024, dtype=torch.float32, device='cuda')
        deep_gemm.fp8_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, config=cfg)
        outs.append(d)
    assert torch.equal(outs[0], outs[1])
    # heuristic choice for a decode shape (prints nothing; must simply be right)
    _dense(128, 2112, 7168, dist='normal', recipe=(1, 128, 128))
    _dense(64, 4096, 7168, dist='normal', recipe=(1, 128, 128), bias=True)
    with pytest.raises(RuntimeError):
        _dense(512, 512, 1024, config={'cta_group': 2, 'block_n': 128, 'split_k': 2, 'cluster_split': 1})
    with pytest.raises(RuntimeError):
        _dense(128, 512, 4096, config={'block_n': 128, 'split_k': 9, 'cluster_split': 1})


@pytest.mark.parametrize('bn', [32, 64, 96, 128, 160, 224, 256])
def test_dense_cta_pair(bn):
    """Two CTAs of a cluster share one 256-row UMMA; each loads its own A rows and half of the B tile."""
    _dense(512, 768, 1024, config={'cta_group': 2, 'block_n': bn})
    _dense(300, 500, 640, config={'cta_group': 2, 'block_n': bn}, out=torch.float32, acc=True)


def test_dense_cta_pair_variants():
    _dense(1024, 2048, 2048, config={'cta_group': 2, 'block_n': 224}, bias=True)
    _dense(130, 257, 2048, config={'cta_group': 2, 'block_n': 96}, out=torch.float32)
    _dense(512, 512, 1024, trans='nn', config={'cta_group': 2, 'block_n': 256})
    _dense(512, 512, 1024, trans='tn', config={'cta_group': 2, 'block_n': 256})
    _dense(512, 512, 1024, trans='tt', config={'cta_group': 2, 'block_n': 128})
    _dense(4096, 2112, 1024, dist='normal', recipe=(1, 128, 128))      # heuristic picks the CTA pair here


def _mixed(m, n, k, *, trans='nn', recipe_a=(1, 32), out=torch.bfloat16, config=None, bias=False, seed=0):
    """FP8 A times packed-FP4 B. 'nn': B is given as [K, N/2] (MN-major codes); 'nt': B is [N, K/2]."""
    seed_all(seed)
    a, sfa, a_ref = uniform_fp8((m, k), recipe_a)
    b, sfb, b_ref = uniform_fp4(n, k, (1, 32), mn_major=trans[1] == 'n')
    c = torch.randn(1, n).to(out) if bias else None
    ref = oracle.gemm_ref(a_ref, b_ref, out, bias=c)
    b_dev, sfb_dev = b.cuda(), sfb.cuda()
    b_arg = (b_dev.transpose(0, 1), sfb_dev.transpose(0, 1)) if trans[1] == 'n' else (b_dev, sfb_dev)
    d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
    getattr(deep_gemm, f'fp8_fp4_gemm_{trans}')((a.cuda(), sfa.cuda()), b_arg, d, c=c.cuda() if bias else None,
                                                recipe_a=recipe_a, recipe_b=(1, 32), config=config)
    assert deep_gemm.device_status() == 0
    return assert_close(d, ref, f'fp8xfp4 {trans} {m}x{n}x{k} recipe_a={recipe_a} config={config}')


@pytest.mark.parametrize('trans', ['nn', 'nt'])
def test_mixed_fp8_fp4(trans):
    _mixed(128, 256, 512, trans=trans)
    _mixed(384, 768, 1024, trans=trans, out=torch.float32)
    _mixed(300, 520, 640, trans=trans, bias=True)
    _mixed(512, 512, 2048, trans=trans, recipe_a=(1, 128))       # per-128 scales on A, per-32 on B (BASELINE config 3)
    _mixed(512, 512, 1024, trans=trans, config={'cta_group': 2, 'block_n': 256})
    _mixed(512, 1024, 1024, trans=trans, config={'cta_group': 1, 'block_n': 128})


def test_mixed_fp8_fp4_nt_narrow_tiles():
    for bn in (32, 96, 224):
        _mixed(256, 672, 768, trans='nt', config={'cta_group': 1, 'block_n': bn})
    _mixed(512, 448, 768, trans='nt', config={'cta_group': 2, 'block_n': 224})


def test_mixed_golden(golden):
    for name, trans in (('dense_fp8fp4_nn', 'nn'), ('dense_fp8fp4_nt', 'nt')):
        c = golden[name]
        a = c['a'].view(torch.float8_e4m3fn).cuda()
        if trans == 'nn':      # fixture holds the logical [N/2, K] view made contiguous; storage is [K, N/2]
            b_arg = (c['b'].transpose(0, 1).contiguous().cuda(), c['sfb'].cuda().transpose(0, 1))
        else:
            b_arg = (c['b'].cuda(), c['sfb'].cuda())
        d = torch.zeros_like(c['d']).cuda()
        getattr(deep_gemm, f'fp8_fp4_gemm_{trans}')((a, c['sfa'].cuda()), b_arg, d)
        assert_close(d, c['d'], name)


def _fp4_pair(m, n, k, *, out=torch.bfloat16, acc=False, bias=False, config=None, seed=0):
    """Both operands packed E2M1, K-major ([MN, K/2] int8), per-32 UE8M0 scales: the kind::mxf4 path."""
    seed_all(seed)
    a, sfa, a_ref = uniform_fp4(m, k, (1, 32), mn_major=False)
    b, sfb, b_ref = uniform_fp4(n, k, (1, 32), mn_major=False)
    c = torch.randn(1 if bias else m, n).to(out) if (acc or bias) else None
    ref = oracle.gemm_ref(a_ref, b_ref, out, c=c if acc else None, bias=c if bias else None)
    d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
    kwargs = {}
    if acc:
        d.copy_(c)
        kwargs['c'] = d
    elif bias:
        kwargs['c'] = c.cuda()
    deep_gemm.fp8_fp4_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, recipe_a=(1, 32), recipe_b=(1, 32),
                              config=config, **kwargs)
    assert deep_gemm.device_status() == 0
    return assert_close(d, ref, f'fp4xfp4 {m}x{n}x{k} out={out} acc={acc} bias={bias} config={config}')


@pytest.mark.parametrize('m,n,k', [(128, 128, 256), (128, 256, 1024), (256, 192, 2048), (64, 2112, 7168), (4096, 512, 4096),
                                   (130, 257, 2048), (17, 512, 4096), (64, 64, 64), (256, 512, 96), (128, 128, 468)])
def test_fp4_pair_dense(m, n, k):
    _fp4_pair(m, n, k)
    _fp4_pair(m, n, k, out=torch.float32, acc=True)


def test_fp4_pair_tilings_and_epilogues():
    for bn in (32, 64, 96, 128, 160, 192, 224, 256):
        _fp4_pair(384, 768, 2048, config={'block_n': bn})
        _fp4_pair(512, 768, 2048, config={'cta_group': 2, 'block_n': bn})
    _fp4_pair(256, 384, 1024, bias=True)
    _fp4_pair(128, 512, 8192, config={'block_n': 128, 'split_k': 4})
    _fp4_pair(128, 512, 8192, config={'block_n': 128, 'split_k': 4, 'cluster_split': 1})
    _fp4_pair(4096, 2112, 7168)                         # heuristic: CTA pairs


def test_fp4_pair_golden(golden):
    for name in ('dense_fp4fp4_nt', 'dense_fp4fp4_nt_acc_f32'):
        c = golden[name]
        d = torch.zeros_like(c['d']).cuda()
        kwargs = {}
        if c['accumulate']:
            d.copy_(c['c'])
            kwargs['c'] = d
        deep_gemm.fp8_fp4_gemm_nt((c['a'].cuda(), c['sfa'].cuda()), (c['b'].cuda(), c['sfb'].cuda()), d, **kwargs)
        assert deep_gemm.device_status() == 0
        assert_close(d, c['d'], name)


def test_fp4_pair_m_grouped():
    """m-grouped contiguous (psum layout) with both operands packed E2M1."""
    seed_all(11)
    sizes = [300, 0, 513, 128]
    total, psum = oracle.make_psum_layout(sizes, 256)
    n, k = 384, 1024
    a, sfa, a_ref = uniform_fp4(total, k, (1, 32), mn_major=False)
    raw = a.clone()
    for span in oracle.psum_padding_spans(psum, 256):
        raw[span] = 0
        a_ref[span] = 0
    bs = [uniform_fp4(n, k, (1, 32), mn_major=False) for _ in sizes]
    b = torch.stack([x[0] for x in bs]); sfb = torch.stack([x[1] for x in bs]); b_ref = torch.stack([x[2] for x in bs])
    ref = oracle.m_grouped_psum_ref(a_ref, b_ref, psum, torch.bfloat16)
    d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    deep_gemm.m_grouped_fp8_fp4_gemm_nt_contiguous((raw.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, layout,
                                                   recipe_a=(1, 32), recipe_b=(1, 32))
    assert deep_gemm.device_status() == 0
    out = d.cpu()
    for span in oracle.psum_valid_spans(psum, 256):
        assert_close(out[span], ref[span], 'fp4xfp4 m-grouped')


def test_fp4_operand_rules():
    # a packed A next to an E4M3 B stays rejected (csrc/apis/gemm.hpp:22-33); MN-major packed operands: test_gpu_fp4_majors.py
    a = torch.zeros(128, 64, dtype=torch.int8, device='cuda')
    b = torch.zeros(128, 128, dtype=torch.float8_e4m3fn, device='cuda')
    sf = torch.ones(128, 4, dtype=torch.float32, device='cuda')
    d = torch.zeros(128, 128, dtype=torch.bfloat16, device='cuda')
    with pytest.raises(RuntimeError, match='Unsupported operand dtypes'):
        deep_gemm.fp8_fp4_gemm_nt((a, sf), (b, sf), d)


@pytest.mark.parametrize('m,n,k', [(4, 4, 4), (4, 4, 16384), (4, 16384, 4), (16384, 4, 4), (16384, 4, 16384),
                                   (4, 16384, 16384), (128, 128, 128), (256, 512, 1024), (1024, 256, 512)])
def test_reference_extra_shape_list_all_majors(m, n, k):
    """The shape list of tests/generators.py:466-488 with every major combination, FP32 accumulate."""
    for trans in ('nt', 'nn', 'tn', 'tt'):
        _dense(m, n, k, trans=trans, out=torch.float32, acc=True)


def test_m_grouped_minimal_case():
    """tests/generators.py:594: 128 groups of about one row, N = K = 4."""
    import random
    random.seed(0)
    sizes = [max(int(random.uniform(0.7, 1.3) * 1), 0) for _ in range(128)]
    _grouped_case(sizes, 4, 4)


@pytest.mark.parametrize('m,n,k,trans', [(256, 384, 512, 'nt'), (130, 257, 1024, 'nt'), (384, 224, 768, 'nn'),
                                         (1024, 2112, 2048, 'nt'), (64, 100, 256, 'tn')])
def test_stochastic_rounding_is_bit_exact(m, n, k, trans):
    """BF16 output with the BF16StochasticRounding epilogue equals the reference's hash model applied to the FP32
    output of the same GEMM, bit for bit (tests/utils.py:70-92, tests/common.py:215-221)."""
    seed_all(m + n)
    a, sfa, _ = uniform_fp8((m, k), (1, 32))
    b, sfb, _ = uniform_fp8((n, k), (1, 32))
    a_dev = with_major(a, trans[0] == 't').cuda()
    b_dev = with_major(b, trans[1] == 'n').cuda()
    a_arg = (a_dev.transpose(0, 1), sfa.cuda().transpose(0, 1)) if trans[0] == 't' else (a_dev, sfa.cuda())
    b_arg = (b_dev.transpose(0, 1), sfb.cuda().transpose(0, 1)) if trans[1] == 'n' else (b_dev, sfb.cuda())
    fn = getattr(deep_gemm, f'fp8_gemm_{trans}')
    d32 = torch.empty(m, n, dtype=torch.float32, device='cuda')
    fn(a_arg, b_arg, d32)
    d16 = torch.empty(m, n, dtype=torch.bfloat16, device='cuda')
    fn(a_arg, b_arg, d16, epilogue=deep_gemm.epilogue.BF16StochasticRounding())
    assert deep_gemm.device_status() == 0
    expected = oracle.stochastic_round_bf16(d32)
    assert torch.equal(d16.cpu().view(torch.int16), expected.view(torch.int16))
    with pytest.raises(RuntimeError, match='Stochastic rounding requires a direct BF16 output'):
        fn(a_arg, b_arg, d32, epilogue=deep_gemm.epilogue.BF16StochasticRounding())


def test_golden_fixtures_through_the_api(golden):
    for name in ('dense_fp8_nt_bf16', 'dense_fp8_nt_acc_f32', 'dense_fp8_unaligned_k', 'dense_fp8_recipe_32_32',
                 'dense_fp8_nn_bias', 'dense_fp8_tn_alpha'):
        c = golden[name]
        a = c['a'].view(torch.float8_e4m3fn)
        b = c['b'].view(torch.float8_e4m3fn)
        a_dev = with_major(a, c['a_major'] == 'MN').cuda()
        b_dev = with_major(b, c['b_major'] == 'MN').cuda()
        d = torch.zeros_like(c['d']).cuda()
        kwargs = {}
        if c['accumulate']:
            d.copy_(c['c'])
            kwargs['c'] = d
        elif c['with_bias']:
            kwargs['c'] = c['c'].cuda()
        gm, gn, gk = c['recipe']
        deep_gemm.fp8_gemm_nt((a_dev, c['sfa'].cuda()), (b_dev, c['sfb'].cuda()), d, recipe_a=(gm, gk),
                              recipe_b=(gn, gk), alpha=c['alpha'], **kwargs)
        assert_close(d, c['d'], name)


def _grouped_case(sizes, n, k, trans_b=False, out=torch.bfloat16, seed=0, config=None):
    seed_all(seed)
    total, psum = oracle.make_psum_layout(sizes, 256)
    g = len(sizes)
    a, sfa, a_ref = uniform_fp8((total, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((g, n, k), (1, 32))
    for span in oracle.psum_padding_spans(psum, 256):
        a.view(torch.uint8)[span] = 0
        a_ref[span] = 0
        sfa[span] = torch.randn_like(sfa[span])          # garbage on purpose (tests/generators.py:342-346)
    ref = oracle.m_grouped_psum_ref(a_ref, b_ref, psum, out)
    b_dev = with_major(b, trans_b).cuda()
    b_arg = (b_dev.transpose(1, 2), sfb.cuda().transpose(1, 2)) if trans_b else (b_dev, sfb.cuda())
    d = torch.full((total, n), float('nan'), dtype=out, device='cuda')
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    fn = deep_gemm.m_grouped_fp8_gemm_nn_contiguous if trans_b else deep_gemm.m_grouped_fp8_gemm_nt_contiguous
    fn((a.cuda(), sfa.cuda()), b_arg, d, layout, config=config)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref, f'm-grouped sizes={sizes} n={n} k={k} trans_b={trans_b} config={config}')
    # padding rows are computed from zero rows of A and must be exactly zero
    for span in oracle.psum_padding_spans(psum, 256):
        assert (d[span] == 0).all(), 'padding rows of D must be exactly zero'


@pytest.mark.parametrize('sizes', [[300, 200, 513], [1, 0, 255, 256, 257], [700]])
def test_m_grouped_contiguous(sizes):
    _grouped_case(sizes, 384, 512)
    _grouped_case(sizes, 256, 768, trans_b=True, out=torch.float32)
    _grouped_case(sizes, 384, 512, config={'cta_group': 1, 'block_n': 128})
    _grouped_case(sizes, 384, 512, config={'cta_group': 2, 'block_n': 224})


def test_m_grouped_golden(golden):
    for name, trans_b in (('mgrouped_fp8_nt', False), ('mgrouped_fp8_nn', True)):
        c = golden[name]
        a = c['a'].view(torch.float8_e4m3fn).cuda()
        b = with_major(c['b'].view(torch.float8_e4m3fn), trans_b).cuda()
        sfb = c['sfb'].cuda()
        b_arg = (b.transpose(1, 2), sfb.transpose(1, 2)) if trans_b else (b, sfb)
        d = torch.full(tuple(c['d'].shape), float('nan'), dtype=torch.bfloat16, device='cuda')
        layout = torch.tensor(c['psum'], dtype=torch.int32, device='cuda')
        fn = deep_gemm.m_grouped_fp8_gemm_nn_contiguous if trans_b else deep_gemm.m_grouped_fp8_gemm_nt_contiguous
        fn((a, c['sfa'].cuda()), b_arg, d, layout)
        assert_close(d, c['d'], name)


@pytest.mark.parametrize('max_m,masked', [(256, [0, 256, 1, 130, 77]), (128, [128, 5, 0]), (200, [200, 13, 129])])
def test_m_grouped_masked(max_m, masked):
    seed_all(7)
    g, n, k = len(masked), 384, 640
    a, sfa, a_ref = uniform_fp8((g, max_m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((g, n, k), (1, 32))
    ref = oracle.m_grouped_masked_ref(a_ref, b_ref, masked, torch.bfloat16)
    d = torch.full((g, max_m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    mask = torch.tensor(masked, dtype=torch.int32, device='cuda')
    deep_gemm.m_grouped_fp8_gemm_nt_masked((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, mask, max(masked))
    assert deep_gemm.device_status() == 0
    for i, mg in enumerate(masked):
        if mg:
            assert_close(d[i, :mg], ref[i, :mg], f'masked group {i} rows {mg}')


def test_dense_eight_epilogue_warps():
    """Warps 8..11 as a second set of epilogue warps (every other 64-column group of a tile)."""
    for bn in (32, 64, 96, 128, 160, 192, 224, 256):
        _dense(384, 768, 512, config={'block_n': bn, 'epilogue_warps': 8})
        _dense(512, 768, 512, config={'cta_group': 2, 'block_n': bn, 'epilogue_warps': 8}, out=torch.float32, acc=True)
    _dense(1024, 2048, 256, config={'cta_group': 2, 'block_n': 224, 'epilogue_warps': 8}, bias=True)
    _dense(300, 500, 384, config={'block_n': 96, 'epilogue_warps': 8}, alpha=0.5)
    _dense(4096, 4096, 512)            # the heuristic takes eight warps here
    with pytest.raises(RuntimeError):
        _dense(256, 256, 512, trans='nn', config={'block_n': 128, 'epilogue_warps': 8})


@pytest.mark.parametrize('bn', [320, 384, 448])
def test_dense_wide_tiles(bn):
    """block_n > 256 (CTA pairs): two column halves per K step that share the A tile, one accumulator of block_n columns."""
    _dense(512, 1024, 1024, config={'cta_group': 2, 'block_n': bn})
    _dense(300, 1000, 640, config={'cta_group': 2, 'block_n': bn}, out=torch.float32, acc=True)
    _dense(130, 257, 384, config={'cta_group': 2, 'block_n': bn}, bias=True)                  # one ragged tile
    _dense(256, 2 * bn + 40, 512, config={'cta_group': 2, 'block_n': bn}, alpha=0.25)
    _dense(1024, 3 * bn, 2048, config={'cta_group': 2, 'block_n': bn, 'num_stages': 2})


def test_dense_wide_tile_variants():
    _dense(4096, 4096, 7168, dist='normal', recipe=(1, 128, 128))      # the heuristic takes a wide pair tile here
    _dense(1024, 900, 2048, config={'cta_group': 2, 'block_n': 448}, acc=True)               # BF16 reduce-add
    # same accumulation order as the narrow tiling: bit-identical results
    seed_all(7)
    a, sfa, _ = uniform_fp8((512, 1024), (1, 32))
    b, sfb, _ = uniform_fp8((1344, 1024), (1, 32))
    outs = []
    for cfg in ({'cta_group': 2, 'block_n': 224}, {'cta_group': 2, 'block_n': 448}, {'cta_group': 2, 'block_n': 320}):
        d = torch.full((512, 1344), float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.fp8_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, config=cfg)
        outs.append(d)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[0].view(torch.int16), outs[2].view(torch.int16))
    for bad in ({'cta_group': 2, 'block_n': 288}, {'cta_group': 2, 'block_n': 512}, {'cta_group': 1, 'block_n': 320},
                {'cta_group': 2, 'block_n': 320, 'epilogue_warps': 8}):
        with pytest.raises(RuntimeError):
            _dense(256, 1024, 1024, config=bad)
    with pytest.raises(RuntimeError):                                                          # MN-major B
        _dense(256, 1024, 1024, trans='nn', config={'cta_group': 2, 'block_n': 320})


def test_m_grouped_wide_tiles():
    total, psum = oracle.make_psum_layout([300, 0, 513, 256], 256)
    seed_all(3)
    a, sfa, a_ref = uniform_fp8((total, 768), (1, 32))
    b, sfb, b_ref = uniform_fp8((4, 1000, 768), (1, 32))
    for span in oracle.psum_padding_spans(psum):
        a.view(torch.uint8)[span] = 0
        a_ref[span] = 0
    ref = oracle.m_grouped_psum_ref(a_ref, b_ref, psum, torch.bfloat16)
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    for cfg in ({'cta_group': 2, 'block_n': 384}, {'cta_group': 2, 'block_n': 448}):
        d = torch.full((total, 1000), float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.m_grouped_fp8_gemm_nt_contiguous((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, layout, config=cfg)
        assert deep_gemm.device_status() == 0
        assert_close(d, ref, f'm-grouped wide {cfg}')


def test_fp4_pair_wide_tiles():
    """Both operands packed E2M1 with block_n > 256: two column halves per K step, two scale words per row and stage."""
    for bn in (320, 448):
        _fp4_pair(512, 1024, 1024, config={'cta_group': 2, 'block_n': bn})
        _fp4_pair(300, 1000, 768, config={'cta_group': 2, 'block_n': bn}, out=torch.float32)
    _fp4_pair(4096, 7168, 4096)          # the heuristic takes a wide tile here


@pytest.mark.parametrize('bn,n', [(448, 7168), (320, 6080), (384, 5376)])
def test_dense_wide_tiles_last_wave_in_halves(bn, n):
    """A wide-tile launch whose last wave fills at most half of the CTA pairs (16 x n / bn tiles on 74 pairs) hands
    that wave's tiles out as single column halves: same results, bit for bit, as with whole tiles."""
    cfg = {'cta_group': 2, 'block_n': bn}
    _dense(4096, n, 256, config=cfg)
    _dense(4096, n - 24, 384, config=cfg, out=torch.float32, acc=True)
    _dense(4096, n, 128, config=cfg, bias=True)
    seed_all(11)
    a, sfa, _ = uniform_fp8((4096, 512), (1, 32))
    b, sfb, _ = uniform_fp8((n, 512), (1, 32))
    outs = []
    for c in (cfg, {'cta_group': 2, 'block_n': 224}):
        d = torch.full((4096, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.fp8_gemm_nt((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, config=c)
        outs.append(d)
    assert deep_gemm.device_status() == 0
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


@pytest.mark.parametrize('trans_b', [False, True])
def test_m_grouped_mixed_fp8_fp4(trans_b):
    """m-grouped contiguous and masked GEMM with a packed-FP4 B: [G, N, K/2] (K-major) or [G, K, N/2] (MN-major codes).
    N and K are multiples of 128, so the tensor cores read B as E2M1 (one 3-D tensor map over all groups); a second
    problem with N = 392 takes the decoder warps instead."""
    seed_all(21)
    sizes = [300, 0, 513]
    total, psum = oracle.make_psum_layout(sizes, 256)
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    for n, k in ((384, 512), (392, 640)):
        a, sfa, a_ref = uniform_fp8((total, k), (1, 32))
        for span in oracle.psum_padding_spans(psum):
            a.view(torch.uint8)[span] = 0
            a_ref[span] = 0
        parts = [uniform_fp4(n, k, (1, 32), mn_major=trans_b) for _ in sizes]
        b_ref = torch.stack([p[2] for p in parts])
        sfb = torch.stack([p[1] for p in parts])
        if trans_b:      # storage [G, K, N/2]; the API takes the [G, K, N/2] tensor and transposes it itself
            b_store = torch.stack([p[0].transpose(0, 1).contiguous() for p in parts]).cuda()
            b_arg = (b_store, sfb.cuda().transpose(1, 2))
            fn = deep_gemm.m_grouped_fp8_fp4_gemm_nn_contiguous
        else:
            b_arg = (torch.stack([p[0] for p in parts]).cuda(), sfb.cuda())
            fn = deep_gemm.m_grouped_fp8_fp4_gemm_nt_contiguous
        d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        fn((a.cuda(), sfa.cuda()), b_arg, d, layout, recipe_a=(1, 32), recipe_b=(1, 32))
        assert deep_gemm.device_status() == 0
        ref = oracle.m_grouped_psum_ref(a_ref, b_ref, psum, torch.bfloat16)
        for span in oracle.psum_valid_spans(psum, 256):
            if span.stop > span.start:
                assert_close(d[span], ref[span], f'm-grouped fp8xfp4 n={n} k={k} trans_b={trans_b}')
    if not trans_b:
        masked = [200, 0, 77]
        n, k = 384, 512
        am, sfam, am_ref = uniform_fp8((3, 256, k), (1, 32))
        parts = [uniform_fp4(n, k, (1, 32), mn_major=False) for _ in masked]
        d = torch.zeros((3, 256, n), dtype=torch.bfloat16, device='cuda')
        deep_gemm.m_grouped_fp8_fp4_gemm_nt_masked((am.cuda(), sfam.cuda()),
                                                   (torch.stack([p[0] for p in parts]).cuda(), torch.stack([p[1] for p in parts]).cuda()),
                                                   d, torch.tensor(masked, dtype=torch.int32, device='cuda'), 100,
                                                   recipe_a=(1, 32), recipe_b=(1, 32))
        assert deep_gemm.device_status() == 0
        ref = oracle.m_grouped_masked_ref(am_ref, torch.stack([p[2] for p in parts]), masked, torch.bfloat16)
        for g, mg in enumerate(masked):
            if mg:
                assert_close(d[g, :mg], ref[g, :mg], f'masked fp8xfp4 group {g}')


@pytest.mark.parametrize('m,n,k,config', [(1152, 2742, 1408, {'block_n': 64, 'cta_group': 1}),
                                          (1152, 2742, 1425, {'block_n': 32, 'cta_group': 1}),
                                          (384, 32766, 512, None), (1000, 4098, 640, {'block_n': 128, 'cta_group': 1})])
def test_dense_plain_stores_with_several_tiles_per_cta(m, n, k, config):
    """A D whose rows TMA cannot write (N * element size not a multiple of 16 bytes) goes out through plain stores; with
    single CTAs and three or more tiles per CTA that must not take the one-tile-per-CTA kernel."""
    _dense(m, n, k, config=config)
    _dense(m, n, k, config=config, out=torch.float32, acc=True)


def test_cluster_split_that_shrinks_to_fewer_splits():
    """K = 551 has five K blocks: four requested splits become three (two blocks each), whose reduce buffers are larger
    than those of four; the pipeline depth must be sized for the split count that runs."""
    cfg = {'block_n': 128, 'cta_group': 1, 'split_k': 4, 'cluster_split': 1, 'num_stages': 6}
    _dense(33, 128, 551, trans='tn', config=cfg, acc=True)
    _dense(33, 128, 551, trans='nt', config=cfg)
    _dense(128, 192, 640, config={'block_n': 64, 'cta_group': 1, 'split_k': 4, 'cluster_split': 1})
