"""Batched GEMM, the FP8 einsum forms and the FP8-quantised output epilogue against the oracle
(modelled on the reference's tests/test_einsum.py:30-110)."""

import pytest
import torch

import deep_gemm
import oracle
from helpers import assert_close, seed_all, uniform_fp8, with_major

pytestmark = pytest.mark.gpu


def _batched_operands(batch, m, n, k, seed=0):
    seed_all(seed)
    a, sfa, a_ref = uniform_fp8((batch, m, k), (1, 32))
    b, sfb, b_ref = uniform_fp8((batch, n, k), (1, 32))
    return (a, sfa, a_ref), (b, sfb, b_ref)


@pytest.mark.parametrize('batch,m,n,k', [(3, 200, 256, 512), (8, 128, 384, 1024), (2, 520, 130, 256)])
def test_fp8_bmm(batch, m, n, k):
    (a, sfa, a_ref), (b, sfb, b_ref) = _batched_operands(batch, m, n, k)
    ref = torch.einsum('bmk,bnk->bmn', a_ref, b_ref)
    for a_mn, b_mn in ((False, False), (True, False), (False, True), (True, True)):
        d = torch.full((batch, m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.fp8_bmm((with_major(a, a_mn).cuda(), sfa.cuda()), (with_major(b, b_mn).cuda(), sfb.cuda()), d)
        assert deep_gemm.device_status() == 0
        assert_close(d, ref.bfloat16(), f'bmm majors {a_mn},{b_mn}')
    # accumulate into FP32: C aliases D
    c = torch.randn(batch, m, n)
    d = c.clone().cuda()
    deep_gemm.fp8_bmm((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, c=d)
    assert_close(d, ref + c, 'bmm accumulate')


@pytest.mark.parametrize('expr', ['bhr,hdr->bhd', 'bhd,hdr->bhr', 'bhd,bhr->hdr'])
@pytest.mark.parametrize('b_,h,r,d_', [(32, 4, 256, 128), (128, 8, 512, 128), (4, 2, 64, 64)])
def test_fp8_einsum(expr, b_, h, r, d_):
    seed_all(b_ + h)
    # build the batched [B, M, K] / [B, N, K] problem, then hand it over in the einsum's own axis order
    if expr == 'bhr,hdr->bhd':
        (a, sfa, a_ref), (b, sfb, b_ref) = _batched_operands(h, b_, d_, r)           # (B,M,N,K) = (h,b,d,r)
        a_arg = (a.permute(1, 0, 2).cuda(), sfa.permute(1, 0, 2).cuda())              # [b,h,r]
        b_arg = (b.cuda(), sfb.cuda())                                                # [h,d,r]
        ref = torch.einsum('hbr,hdr->bhd', a_ref, b_ref)
        out_shape = (b_, h, d_)
    elif expr == 'bhd,hdr->bhr':
        (a, sfa, a_ref), (b, sfb, b_ref) = _batched_operands(h, b_, r, d_)           # (h,b,r,d)
        a_arg = (a.permute(1, 0, 2).cuda(), sfa.permute(1, 0, 2).cuda())              # [b,h,d]
        b_arg = (b.permute(0, 2, 1).cuda(), sfb.permute(0, 2, 1).cuda())              # [h,d,r]
        ref = torch.einsum('hbd,hrd->bhr', a_ref, b_ref)
        out_shape = (b_, h, r)
    else:
        (a, sfa, a_ref), (b, sfb, b_ref) = _batched_operands(h, d_, r, b_)           # (h,d,r,b), K = b
        a_arg = (a.permute(2, 0, 1).cuda(), sfa.permute(2, 0, 1).cuda())              # [b,h,d]
        b_arg = (b.permute(2, 0, 1).cuda(), sfb.permute(2, 0, 1).cuda())              # [b,h,r]
        ref = torch.einsum('hdb,hrb->hdr', a_ref, b_ref)
        out_shape = (h, d_, r)
    d = torch.full(out_shape, float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_einsum(expr, a_arg, b_arg, d)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref.bfloat16(), f'einsum {expr}')
    if expr == 'bhd,bhr->hdr':
        c = torch.randn(out_shape)
        acc = c.clone().cuda()
        deep_gemm.fp8_einsum(expr, a_arg, b_arg, acc, c=acc)
        assert_close(acc, ref + c, f'einsum {expr} accumulate')

    if expr == 'bhr,hdr->bhd' and d_ % 128 == 0:
        # E4M3 output with per-(row, 32) UE8M0 scales: bit-exact against quantising the BF16 result on the CPU
        out8 = torch.zeros(out_shape, dtype=torch.float8_e4m3fn, device='cuda')
        sfd = torch.empty_strided((b_, h * d_ // 64), (1, b_), dtype=torch.int16, device='cuda')
        deep_gemm.fp8_einsum(expr, a_arg, b_arg, (out8, sfd))
        assert deep_gemm.device_status() == 0
        q, sf, _ = oracle.quantize_e4m3(d.cpu().float().reshape(b_, h * d_), (1, 32))
        sf_bytes = ((sf.view(torch.int32) >> 23) & 0xFF).reshape(b_, -1, 2)
        ref_sfd = (sf_bytes[..., 0] + sf_bytes[..., 1] * 256).to(torch.int16)
        assert torch.equal(out8.cpu().view(torch.uint8).reshape(b_, h * d_), q.view(torch.uint8))
        assert torch.equal(sfd.contiguous().cpu(), ref_sfd)


def test_fp8_output_rules():
    (a, sfa, _), (b, sfb, _) = _batched_operands(2, 128, 128, 128)
    d = torch.zeros(2, 128, 128, dtype=torch.float8_e4m3fn, device='cuda')
    sfd = torch.empty_strided((128, 4), (1, 128), dtype=torch.int16, device='cuda')
    with pytest.raises(RuntimeError, match='hold the batches side by side'):
        deep_gemm.fp8_bmm((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), (d, sfd))
    with pytest.raises(RuntimeError, match='Unsupported einsum expression'):
        deep_gemm.fp8_einsum('bhr,hrd->bhd', (a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d)


def test_wide_tiles_batched_quantised_and_stochastic():
    """block_n > 256 (two column halves per K step) under the batched scheduler and the two epilogues that work on
    32-column chunks: FP8-quantised output (bit-exact against quantising the BF16 result) and stochastic rounding
    (bit-exact against the hash model applied to the FP32 result)."""
    cfg = {'cta_group': 2, 'block_n': 384}
    (a, sfa, a_ref), (b, sfb, b_ref) = _batched_operands(3, 300, 800, 512, seed=2)
    ref = torch.einsum('bmk,bnk->bmn', a_ref, b_ref)
    d = torch.full((3, 300, 800), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_bmm((a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda()), d, config=cfg)
    assert deep_gemm.device_status() == 0
    assert_close(d, ref.bfloat16(), 'bmm wide tile')

    b_, h, r, d_ = 64, 4, 256, 256                                                   # 'bhr,hdr->bhd': N = d_ per head
    (a, sfa, _), (b, sfb, _) = _batched_operands(h, b_, d_, r, seed=4)
    a_arg = (a.permute(1, 0, 2).cuda(), sfa.permute(1, 0, 2).cuda())
    b_arg = (b.cuda(), sfb.cuda())
    d16 = torch.full((b_, h, d_), float('nan'), dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_einsum('bhr,hdr->bhd', a_arg, b_arg, d16)
    out8 = torch.zeros((b_, h, d_), dtype=torch.float8_e4m3fn, device='cuda')
    sfd = torch.empty_strided((b_, h * d_ // 64), (1, b_), dtype=torch.int16, device='cuda')
    deep_gemm.fp8_einsum('bhr,hdr->bhd', a_arg, b_arg, (out8, sfd), config={'cta_group': 2, 'block_n': 320})
    assert deep_gemm.device_status() == 0
    q, sf, _ = oracle.quantize_e4m3(d16.cpu().float().reshape(b_, h * d_), (1, 32))
    sf_bytes = ((sf.view(torch.int32) >> 23) & 0xFF).reshape(b_, -1, 2)
    assert torch.equal(out8.cpu().view(torch.uint8).reshape(b_, h * d_), q.view(torch.uint8))
    assert torch.equal(sfd.contiguous().cpu(), (sf_bytes[..., 0] + sf_bytes[..., 1] * 256).to(torch.int16))

    seed_all(9)
    a, sfa, _ = uniform_fp8((384, 768), (1, 32))
    b, sfb, _ = uniform_fp8((900, 768), (1, 32))
    a_arg, b_arg = (a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda())
    d32 = torch.empty(384, 900, dtype=torch.float32, device='cuda')
    deep_gemm.fp8_gemm_nt(a_arg, b_arg, d32, config={'cta_group': 2, 'block_n': 448})
    d16 = torch.empty(384, 900, dtype=torch.bfloat16, device='cuda')
    deep_gemm.fp8_gemm_nt(a_arg, b_arg, d16, epilogue=deep_gemm.epilogue.BF16StochasticRounding(),
                          config={'cta_group': 2, 'block_n': 448})
    assert deep_gemm.device_status() == 0
    assert torch.equal(d16.cpu().view(torch.int16), oracle.stochastic_round_bf16(d32).view(torch.int16))
