"""The two host layers over the C ABI, the compiled `_C` extension (csrc/python_api.cpp) and the Python module
`_api`, must produce the same bits on the GPU for the same calls: dense (all majors, bias, accumulate, alpha),
m-grouped contiguous, masked, k-grouped, batched with FP8 output, and the scale-factor transform."""

import pytest
import torch

import deep_gemm
import oracle
from deep_gemm import _api
from helpers import assert_close, seed_all, uniform_fp8, with_major

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(_api._C is None, reason='the _C extension has not been built')]


def _both(name):
    return getattr(_api._C, name), getattr(_api, name)


@pytest.mark.parametrize('trans', ['nt', 'nn', 'tn', 'tt'])
def test_dense_same_bits_through_both_host_layers(trans):
    seed_all(4)
    m, n, k = 300, 520, 1024
    a, sfa, a_ref = uniform_fp8((m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((n, k), (1, 32))
    a_dev = with_major(a, trans[0] == 't').cuda()
    b_dev = with_major(b, trans[1] == 'n').cuda()
    a_arg = (a_dev.transpose(0, 1), sfa.cuda().transpose(0, 1)) if trans[0] == 't' else (a_dev, sfa.cuda())
    b_arg = (b_dev.transpose(0, 1), sfb.cuda().transpose(0, 1)) if trans[1] == 'n' else (b_dev, sfb.cuda())
    bias = torch.randn(1, n).to(torch.bfloat16)
    c32 = torch.randn(m, n)
    variants = [
        (torch.bfloat16, {}, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16)),
        (torch.bfloat16, {'c': bias.cuda()}, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16, bias=bias)),
        (torch.bfloat16, {'alpha': -0.375}, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16, alpha=-0.375)),
        (torch.float32, {'acc': True}, oracle.gemm_ref(a_ref, b_ref, torch.float32, c=c32)),
        (torch.bfloat16, {'config': {'block_n': 128, 'cta_group': 1}}, oracle.gemm_ref(a_ref, b_ref, torch.bfloat16)),
    ]
    for out, kwargs, ref in variants:
        results = []
        for fn in _both(f'fp8_gemm_{trans}'):
            kw = dict(kwargs)
            d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
            if kw.pop('acc', False):
                d.copy_(c32)
                kw['c'] = d
            fn(a_arg, b_arg, d, **kw)
            results.append(d)
        assert deep_gemm.device_status() == 0
        assert torch.equal(results[0].view(torch.int32 if out == torch.float32 else torch.int16),
                           results[1].view(torch.int32 if out == torch.float32 else torch.int16))
        assert_close(results[0], ref, f'{trans} {kwargs}')


def test_grouped_layouts_same_bits_through_both_host_layers():
    seed_all(6)
    sizes = [300, 0, 513]
    total, psum = oracle.make_psum_layout(sizes, 256)
    n, k = 384, 512
    a, sfa, a_ref = uniform_fp8((total, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((3, n, k), (1, 32))
    for span in oracle.psum_padding_spans(psum):
        a.view(torch.uint8)[span] = 0
        a_ref[span] = 0
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    outs = []
    for fn in _both('m_grouped_fp8_gemm_nt_contiguous'):
        d = torch.full((total, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        fn((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, layout)
        outs.append(d)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert_close(outs[0], oracle.m_grouped_psum_ref(a_ref, b_ref, psum, torch.bfloat16), 'm-grouped')
    # masked
    masked = [200, 0, 77]
    am, sfam, am_ref = uniform_fp8((3, 256, k), (1, 32))
    mask = torch.tensor(masked, dtype=torch.int32, device='cuda')
    outs = []
    for fn in _both('m_grouped_fp8_gemm_nt_masked'):
        d = torch.zeros((3, 256, n), dtype=torch.bfloat16, device='cuda')
        fn((am.cuda(), sfam.cuda()), (b.cuda(), sfb.cuda()), d, mask, 100)
        outs.append(d)
    ref = oracle.m_grouped_masked_ref(am_ref, b_ref, masked, torch.bfloat16)
    for g, mg in enumerate(masked):
        assert torch.equal(outs[0][g, :mg].view(torch.int16), outs[1][g, :mg].view(torch.int16))
        if mg:
            assert_close(outs[0][g, :mg], ref[g, :mg], 'masked')
    assert deep_gemm.device_status() == 0


def test_transform_and_fp8_output_same_bits_through_both_host_layers():
    seed_all(8)
    sf = (torch.randint(1, 255, (3, 200, 23), dtype=torch.int32) << 23).view(torch.float32).cuda()
    outs = [fn(sf, 200, 23 * 32, (1, 1, 32), 3, True) for fn in _both('transform_sf_into_required_layout')]
    assert torch.equal(outs[0], outs[1]) and outs[0].stride() == outs[1].stride()
    assert torch.equal(outs[0].cpu(), oracle.required_sf_layout(sf.cpu(), 200, 23 * 32, 1))
    # batched GEMM with E4M3 output and its scale tensor
    bsz, m, n, k = 2, 128, 256, 512
    a, sfa, _ = uniform_fp8((bsz, m, k), (1, 32))
    b, sfb, _ = uniform_fp8((bsz, n, k), (1, 32))
    results = []
    for fn in _both('fp8_bmm'):
        d = torch.zeros(m, bsz * n, dtype=torch.uint8, device='cuda').view(torch.float8_e4m3fn)
        d3 = d.view(m, bsz, n).permute(1, 0, 2)
        sfd = torch.zeros(bsz * n // 64, m, dtype=torch.int16, device='cuda').transpose(0, 1)
        fn((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), (d3, sfd))
        results.append((d.view(torch.uint8).clone(), sfd.clone()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    assert deep_gemm.device_status() == 0


@pytest.mark.parametrize('m,n,k', [(256, 384, 1024), (130, 258, 512)])
def test_packed_fp4_with_mn_major_operands_same_bits_through_both_host_layers(m, n, k):
    """FP4 x FP4 "tn" (both operands MN-major): read as E2M1 when TMA can unpack them, expanded to E4M3 by the host layer
    when it cannot (the second shape); k-grouped FP8 x FP4 likewise."""
    from helpers import uniform_fp4
    seed_all(8)
    a, sfa, a_ref = uniform_fp4(m, k, (1, 32), mn_major=True)
    b, sfb, b_ref = uniform_fp4(n, k, (1, 32), mn_major=True)
    a_arg = (a.cuda().transpose(0, 1), sfa.cuda().transpose(0, 1))
    b_arg = (b.cuda().transpose(0, 1), sfb.cuda().transpose(0, 1))
    outs = []
    for fn in _both('fp8_fp4_gemm_tn'):
        d = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        fn(a_arg, b_arg, d, recipe_a=(1, 32), recipe_b=(1, 32))
        outs.append(d)
    assert deep_gemm.device_status() == 0
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert_close(outs[0], oracle.gemm_ref(a_ref, b_ref, torch.bfloat16), f'fp4xfp4 tn {m}x{n}x{k}')
    # k-grouped: A [K, M] E4M3, B [K, N/2] packed, two groups of K
    sizes = (k // 2, k // 2 - 40)
    total_k, psum = oracle.make_psum_layout(list(sizes), 256)
    a8, sfa8, _ = uniform_fp8((total_k, m), (32, 1))
    b4, sfb4, _ = uniform_fp4(n, total_k, (1, 32), mn_major=True)
    b4 = b4.transpose(0, 1).contiguous()                                  # [K, N/2]
    sfb4 = sfb4.transpose(0, 1).contiguous()                              # [K/32, N]
    for span in oracle.psum_padding_spans(psum, 256):
        a8.view(torch.uint8)[span] = 0
        b4[span] = 0
    ref = oracle.k_grouped_psum_ref(oracle.dequantize(a8.float(), sfa8, 32, 1),
                                    oracle.dequantize(oracle.decode_e2m1_packed(b4, axis=-1), sfb4, 32, 1), psum, torch.float32)
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    outs = []
    for fn in _both('k_grouped_fp8_gemm_tn_contiguous'):
        d = torch.full((2, m, n), float('nan'), dtype=torch.float32, device='cuda')
        fn((a8.cuda(), sfa8.cuda()), (b4.cuda(), sfb4.cuda()), d, None, layout, recipe=(1, 1, 32))
        outs.append(d)
    assert deep_gemm.device_status() == 0
    assert torch.equal(outs[0].view(torch.int32), outs[1].view(torch.int32))
    assert_close(outs[0], ref, f'k-grouped fp8xfp4 {m}x{n}')
