"""Parity of the k-grouped (weight-gradient) GEMM and of its scale-factor transform with the CPU oracle.

Operands are A [K, M] and B [K, N] with K holding the groups in psum layout (group g = rows
[align256(psum[g-1]), psum[g])); data is zero inside a group's padding and the scales there are garbage, as the
reference's generator makes them (tests/generators.py:361-398). Output tolerance as in tests/helpers.py; the
direct-output-versus-FP32-accumulation property and the scale-factor layout are bit-exact.
"""

import warnings

import pytest
import torch

import deep_gemm
import oracle
from helpers import assert_close, assert_close_device, seed_all, uniform_fp8

pytestmark = pytest.mark.gpu


def _make(m, n, sizes, seed=0, poison=True):
    """Returns CPU (a [K,M] fp8, sfa [K/32,M] fp32, a_deq [K,M]) and the same for b, plus (total_k, psum)."""
    seed_all(seed)
    total_k, psum = oracle.make_psum_layout(list(sizes), 256)
    out = []
    for mn in (m, n):
        data, sf, _ = uniform_fp8((total_k, mn), (32, 1))
        raw = data.view(torch.uint8).clone()
        for span in oracle.psum_padding_spans(psum, 256):
            raw[span] = 0
        data = raw.view(torch.float8_e4m3fn)
        deq = oracle.dequantize(data.float(), sf, 32, 1)
        if poison:
            for span in oracle.psum_padding_spans(psum, 256, 32):
                sf[span] = torch.randn_like(sf[span])        # not powers of two, negative: must be ignored
        out.append((data, sf, deq))
    return out[0], out[1], total_k, psum


def _run(m, n, sizes, out=torch.bfloat16, acc=False, ks_hint='list', epilogue=None, seed=0, deprecated=False, config=None):
    (a, sfa, a_deq), (b, sfb, b_deq), total_k, psum = _make(m, n, sizes, seed)
    g = len(sizes)
    c = torch.randn(g, m, n).to(out) if acc else None
    ref = oracle.k_grouped_psum_ref(a_deq, b_deq, psum, out, c=c)
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    d = torch.full((g, m, n), float('nan'), dtype=out, device='cuda')
    kwargs = {}
    if acc:
        d.copy_(c)
        kwargs['c'] = d
    ks = {'list': [oracle.align(s, 256) for s in sizes], 'none': None, 'empty': []}[ks_hint]
    a_arg, b_arg = (a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda())
    if deprecated:
        with warnings.catch_warnings(record=True) as seen:
            warnings.simplefilter('always')
            deep_gemm.k_grouped_fp8_gemm_nt_contiguous((a_arg[0].T, a_arg[1].T), (b_arg[0].T, b_arg[1].T), d, ks, layout,
                                                       recipe=(1, 1, 32), **kwargs)
        assert any(issubclass(w.category, DeprecationWarning) for w in seen)
    else:
        deep_gemm.k_grouped_fp8_gemm_tn_contiguous(a_arg, b_arg, d, ks, layout, recipe=(1, 1, 32), epilogue=epilogue,
                                                   config=config, **kwargs)
    assert deep_gemm.device_status() == 0
    (assert_close_device if d.numel() > (1 << 24) else assert_close)(d, ref, f'k-grouped {m}x{n} sizes={sizes} out={out} acc={acc}')
    return d, (a_arg, b_arg, layout, ks)


def test_fixture_from_the_reference_generator(golden):
    for name in ('kgrouped_fp8_bf16', 'kgrouped_fp8_acc_f32'):
        c = golden[name]
        a = (c['a'].view(torch.float8_e4m3fn).cuda(), c['sfa'].cuda())
        b = (c['b'].view(torch.float8_e4m3fn).cuda(), c['sfb'].cuda())
        layout = torch.tensor(c['psum'], dtype=torch.int32, device='cuda')
        d = torch.full(c['d'].shape, float('nan'), dtype=c['d'].dtype, device='cuda')
        kwargs = {}
        if c['c'] is not None:
            d.copy_(c['c'])
            kwargs['c'] = d
        deep_gemm.k_grouped_fp8_gemm_tn_contiguous(a, b, d, None, layout, recipe=c['recipe'], **kwargs)
        assert deep_gemm.device_status() == 0
        assert_close(d, c['d'], name)
        if name == 'kgrouped_fp8_bf16':
            assert d[1].abs().max().item() == 0


@pytest.mark.parametrize('out,acc', [(torch.float32, True), (torch.float32, False), (torch.bfloat16, False),
                                     (torch.bfloat16, True)])
@pytest.mark.parametrize('ks_hint', ['list', 'none', 'empty'])
def test_output_modes_and_host_hints(out, acc, ks_hint):
    _run(256, 384, (700, 300, 1024, 33), out=out, acc=acc, ks_hint=ks_hint)


@pytest.mark.parametrize('sizes', [(0, 512, 0, 640), (0, 0, 384, 0, 0), (1, 1, 1, 1), (256,), (2048 + 16, 2048 - 16)])
def test_empty_single_and_tiny_groups(sizes):
    d, _ = _run(320, 200, sizes, out=torch.bfloat16)
    for g, s in enumerate(sizes):
        if s == 0:
            assert d[g].abs().max().item() == 0
    # with accumulation an empty group keeps C
    _run(320, 200, sizes, out=torch.float32, acc=True, seed=1)


@pytest.mark.parametrize('m,n', [(4, 4), (4096, 1024), (1000, 7168), (130, 2050)])
def test_shapes(m, n):
    _run(m, n, (900, 1300, 512), out=torch.bfloat16)


def test_pair_and_single_cta_tilings_agree():
    sizes = (1500, 900, 0, 2048)
    d1, _ = _run(512, 512, sizes, out=torch.float32, config=dict(cta_group=1, block_n=128))
    d2, _ = _run(512, 512, sizes, out=torch.float32, config=dict(cta_group=2, block_n=256))
    assert torch.equal(d1, d2)


def test_direct_output_equals_fp32_accumulation_then_cast():
    """tests/utils.py:61-67: the BF16 (or FP32) result written directly is, bit for bit, the FP32
    accumulation onto zeros followed by one cast."""
    for out in (torch.bfloat16, torch.float32):
        d, (a, b, layout, ks) = _run(384, 640, (1000, 0, 700, 2300), out=out)
        fp32 = torch.zeros(d.shape, dtype=torch.float32, device='cuda')
        deep_gemm.k_grouped_fp8_gemm_tn_contiguous(a, b, fp32, ks, layout, c=fp32)
        bits = torch.int16 if out == torch.bfloat16 else torch.int32
        assert torch.equal(d.view(bits), fp32.to(out).view(bits))


def test_stochastic_rounding_matches_the_hash_model():
    sizes = (800, 0, 1200)
    (a, sfa, _), (b, sfb, _), _, psum = _make(256, 264, sizes, seed=3)
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    a, b = (a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda())
    d = torch.empty(3, 256, 264, dtype=torch.bfloat16, device='cuda')
    deep_gemm.k_grouped_fp8_gemm_tn_contiguous(a, b, d, None, layout, epilogue=deep_gemm.epilogue.BF16StochasticRounding())
    fp32 = torch.zeros(3, 256, 264, dtype=torch.float32, device='cuda')
    deep_gemm.k_grouped_fp8_gemm_tn_contiguous(a, b, fp32, None, layout, c=fp32)
    expected = oracle.stochastic_round_bf16(fp32.cpu())
    assert torch.equal(d.cpu().view(torch.int16), expected.view(torch.int16))


def test_deprecated_nt_entry_point():
    _run(256, 256, (512, 300), deprecated=True)


def test_argument_checks():
    (a, sfa, _), (b, sfb, _), _, psum = _make(128, 128, (256, 256), poison=False)
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    d = torch.empty(2, 128, 128, dtype=torch.bfloat16, device='cuda')
    a, b = (a.cuda(), sfa.cuda()), (b.cuda(), sfb.cuda())
    with pytest.raises(RuntimeError):        # operands must be MN-major, i.e. [K, M] row-major
        deep_gemm.k_grouped_fp8_gemm_tn_contiguous((a[0].T.contiguous().T, a[1]), b, d, None, layout)
    with pytest.raises(RuntimeError):
        deep_gemm.k_grouped_fp8_gemm_tn_contiguous(a, b, d, None, layout, use_psum_layout=False)
    with pytest.raises(RuntimeError):        # D must carry the group dimension
        deep_gemm.k_grouped_fp8_gemm_tn_contiguous(a, b, d[0], None, layout)


# ---------------------------------------------------------------------------------------------------------
# transform_k_grouped_sf_into_required_layout
# ---------------------------------------------------------------------------------------------------------
def test_sf_fixtures_from_the_reference_layout_model(golden):
    for name, c in golden['sf_layout_k_grouped'].items():
        sf = c['sf'].cuda()
        if c['mn_major']:
            sf = sf.T.contiguous().T
        layout = torch.tensor(c['psum'], dtype=torch.int32, device='cuda')
        recipe = (c['gran'], c['gran'], 32)
        out = deep_gemm.transform_k_grouped_sf_into_required_layout(sf, c['mn'], c['k'], recipe, True, layout)
        assert out.dtype == torch.int16 and out.shape == c['expected'].shape, name
        assert out.stride(-2) == 1 and out.stride(-1) == out.size(-2), name
        assert torch.equal(out.cpu(), c['expected']), name


@pytest.mark.parametrize('dtype', [torch.float32, torch.int16])
@pytest.mark.parametrize('gran', [1, 32, 128])
@pytest.mark.parametrize('mn_major', [False, True])
@pytest.mark.parametrize('mn,num_groups,avg_k', [(4096, 16, 2048), (7168, 8, 4096), (4096, 72, 384), (7168, 128, 256)])
def test_sf_random_against_oracle(dtype, gran, mn_major, mn, num_groups, avg_k):
    """The reference's sweep (tests/generators.py:693-722): rows x group configurations, groups whose real size is 16
    short of the alignment on odd indices."""
    seed_all(5)
    sizes = [oracle.align(int(avg_k * (0.7 + 0.6 * torch.rand(()).item())), 256) - (16 if i % 2 else 0) for i in range(num_groups)]
    k, psum = oracle.make_psum_layout(sizes, 256)
    div = 32 if dtype == torch.float32 else 64
    shape = (oracle.ceil_div(mn, gran), oracle.ceil_div(k, div))
    if dtype == torch.float32:
        sf = (torch.randint(1, 255, shape, dtype=torch.int32) * (1 << 23)).view(torch.float32)
    else:
        sf = torch.randint(-32768, 32768, shape, dtype=torch.int16)
    expected = oracle.required_sf_layout(sf, mn, k, gran, k_psum=psum)
    poisoned = sf.clone()
    for span in oracle.psum_padding_spans(psum, 256, div):
        poisoned[..., span] = -1 if dtype == torch.float32 else 0x5a5a
    dev = poisoned.cuda()
    if mn_major:
        dev = dev.T.contiguous().T
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    out = deep_gemm.transform_k_grouped_sf_into_required_layout(dev, mn, k, (gran, gran, 32), True, layout)
    assert out.stride(-2) == 1 and out.stride(-1) == mn
    assert torch.equal(out.cpu(), expected)


def test_sf_already_in_required_layout_is_returned_as_is():
    sf = torch.randint(-32768, 32768, (8, 256), dtype=torch.int16, device='cuda').T      # [256, 8], MN-major
    layout = torch.tensor([500], dtype=torch.int32, device='cuda')
    out = deep_gemm.transform_k_grouped_sf_into_required_layout(sf, 256, 512, (1, 1, 32), False, layout)
    assert out.data_ptr() == sf.data_ptr()
