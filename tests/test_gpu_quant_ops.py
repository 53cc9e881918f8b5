"""SwiGLU / cast -> FP8 producer against the CPU oracle, and its output fed straight into the GEMM.

exp() differs in the last bit between the CPU and the GPU, so a value that sits on a rounding boundary of E4M3 (or an
amax on a power-of-two boundary) may round the other way: the comparison allows a small fraction of codes to differ by
one step and checks the dequantised values with a tolerance; everything that does not depend on exp() (the plain
cast, the layout of the scales, which rows are written) is compared bit for bit.
"""

import pytest
import torch

import deep_gemm
import oracle
from helpers import assert_close, seed_all, uniform_fp8

pytestmark = pytest.mark.gpu


def _check(out, out_sf, ref_codes, ref_sf, valid, ref_deq, exact):
    tokens, hidden = ref_codes.shape
    assert out.dtype == torch.float8_e4m3fn and out.shape == (tokens, hidden)
    assert out_sf.dtype == torch.int16 and out_sf.shape == ref_sf.shape and out_sf.stride(0) == 1
    codes, sf = out.view(torch.uint8).cpu()[valid], out_sf.cpu()[valid]
    ref_codes, ref_sf, ref_deq = ref_codes[valid], ref_sf[valid], ref_deq[valid]
    if exact:
        assert torch.equal(sf, ref_sf)
        assert torch.equal(codes, ref_codes)
        return
    sf_b, ref_b = sf.contiguous().view(torch.uint8), ref_sf.contiguous().view(torch.uint8)
    assert (sf_b != ref_b).float().mean().item() < 2e-3
    assert (sf_b.int() - ref_b.int()).abs().max().item() <= 1
    same_scale = (sf_b == ref_b).repeat_interleave(32, dim=1)[:, :hidden]
    differ = (codes != ref_codes) & same_scale
    assert differ.float().mean().item() < 5e-3
    assert ((codes.int() - ref_codes.int()).abs()[differ] <= 1).all()          # neighbouring E4M3 codes
    scale = (sf_b.int() << 23).view(torch.float32).repeat_interleave(32, dim=1)[:, :hidden]
    deq = codes.view(torch.float8_e4m3fn).float() * scale
    assert oracle.calc_diff(deq, ref_deq) < 1e-4


@pytest.mark.parametrize('tokens,hidden', [(1, 128), (33, 256), (256, 2048), (1000, 7168), (4096, 1536)])
def test_swiglu_to_fp8(tokens, hidden):
    seed_all(tokens)
    x = (torch.randn(tokens, 2 * hidden) * 2).bfloat16()
    out, out_sf = deep_gemm.swiglu_apply_weight_to_fp8(x.cuda())
    _check(out, out_sf, *oracle.swiglu_quant_ref(x), exact=False)


def test_swiglu_weight_clamp_and_psum_layout():
    seed_all(3)
    sizes = [300, 0, 129, 1]
    total, psum = oracle.make_psum_layout(sizes, 128)
    x = (torch.randn(total, 1024) * 4).bfloat16()
    w = torch.rand(total) * 2
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    out, out_sf = deep_gemm.swiglu_apply_weight_to_fp8(x.cuda(), w.cuda(), layout, clamp_value=3.0, expert_alignment=128)
    ref = oracle.swiglu_quant_ref(x, w, psum, 3.0, 128)
    assert ref[2].sum().item() == sum(sizes)
    _check(out, out_sf, *ref, exact=False)
    # rows in the padding are not written
    marker = torch.full_like(out.view(torch.uint8), 0x5a)
    out2 = marker.clone().view(torch.float8_e4m3fn)
    from deep_gemm import _lib as L
    sf2 = torch.full((out_sf.size(1), total), 0x1111, dtype=torch.int16, device='cuda')
    L.check(L.lib().dg_quant_fp8_launch(x.cuda().data_ptr(), 1024, total, 512, 1, w.cuda().data_ptr(), layout.data_ptr(), 4, 128,
                                        1, 3.0, out2.data_ptr(), 512, sf2.data_ptr(), total, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    pad = ~ref[2]
    assert (out2.view(torch.uint8).cpu()[pad] == 0x5a).all() and (sf2.T.cpu()[pad] == 0x1111).all()


@pytest.mark.parametrize('tokens,hidden', [(5, 32), (77, 96), (512, 7168)])
def test_plain_cast_is_bit_exact(tokens, hidden):
    seed_all(hidden)
    x = (torch.randn(tokens, hidden) * 3).bfloat16()
    x[0, :32] = 0                                         # an all-zero block takes the 1e-4 floor
    out, out_sf = deep_gemm.cast_to_fp8(x.cuda())
    _check(out, out_sf, *oracle.swiglu_quant_ref(x, swiglu=False), exact=True)


def test_output_feeds_the_gemm_without_a_relayout():
    seed_all(9)
    tokens, hidden, n = 512, 2048, 768
    x = torch.randn(tokens, 2 * hidden).bfloat16()
    a, sfa = deep_gemm.swiglu_apply_weight_to_fp8(x.cuda())
    b, sfb, b_ref = uniform_fp8((n, hidden), (1, 32))
    d = torch.empty(tokens, n, dtype=torch.bfloat16, device='cuda')
    launches = deep_gemm._lib.lib().dg_kernel_launch_count()
    deep_gemm.fp8_gemm_nt((a, sfa), (b.cuda(), deep_gemm.transform_sf_into_required_layout(sfb.cuda(), n, hidden, (1, 1, 32), is_sfa=False)), d,
                          recipe_a=(1, 32), recipe_b=(1, 32))
    # one transform (for B, issued above) and the GEMM kernel(s): none for A
    assert deep_gemm._lib.lib().dg_kernel_launch_count() - launches <= 3
    a_deq = oracle.dequantize(a.float().cpu(), oracle.unpack_required_sf(sfa.cpu(), hidden), 1, 32)
    assert_close(d, oracle.gemm_ref(a_deq, b_ref, torch.bfloat16), 'gemm on the producer output')


def test_expert_mlp_chain_through_the_public_api():
    """GEMM -> SwiGLU * routing weight -> FP8 -> GEMM on a small psum layout (the unfused expert MLP of
    tests/test_mega_moe.py:139-145), each stage checked by the oracle on the stage's own input."""
    from deep_gemm.testing.moe_bench import ExpertMlpCase
    from oracle import checks
    case = ExpertMlpCase([300, 0, 513, 77], 512, 256, torch.device('cuda', 0), seed=5)
    case.run()
    torch.cuda.synchronize()
    assert deep_gemm.device_status() == 0
    assert checks.moe_mlp_case(case, rows=64)
