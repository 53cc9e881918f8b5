"""The CPU oracle against fixtures produced by the reference's own test code."""

import torch

import oracle


def _operand(case, which):
    data, sf = case[which], case['sf' + which]
    is_fp4 = case.get(f'{which}_is_fp4', False)
    major = case.get(f'{which}_major', 'K')
    if is_fp4:
        # two codes per byte along the operand's contiguous axis: K for a K-major
        # operand ([MN, K/2]), MN for an MN-major one (logical [MN/2, K])
        vals = oracle.decode_e2m1_packed(data, axis=-2 if major == 'MN' else -1)
    else:
        vals = oracle.decode_e4m3(data)
    return vals, sf


def test_dense_cases_match_reference_oracle(golden):
    names = [n for n in golden if n.startswith('dense_')]
    assert len(names) >= 8
    for name in names:
        c = golden[name]
        gm, gn, gk = c['recipe']
        a_vals, sfa = _operand(c, 'a')
        b_vals, sfb = _operand(c, 'b')
        a = oracle.dequantize(a_vals, sfa, gm, gk)
        b = oracle.dequantize(b_vals, sfb, gn, gk)
        d = oracle.gemm_ref(a, b, c['d'].dtype,
                            c=c['c'] if c['accumulate'] else None,
                            bias=c['c'] if c['with_bias'] else None,
                            alpha=c['alpha'])
        assert torch.equal(d, c['d']), name


def test_m_grouped_matches_reference_oracle(golden):
    for name in ('mgrouped_fp8_nt', 'mgrouped_fp8_nn'):
        c = golden[name]
        a = oracle.dequantize(oracle.decode_e4m3(c['a']), c['sfa'], 1, 32)
        # scale rows in the group padding hold garbage on purpose; A is zero there
        a = torch.nan_to_num(a, nan=0.0, posinf=0.0, neginf=0.0)
        b = oracle.dequantize(oracle.decode_e4m3(c['b']), c['sfb'], 1, 32)
        d = oracle.m_grouped_psum_ref(a, b, c['psum'], torch.bfloat16)
        assert torch.equal(d, c['d']), name


def _k_grouped_operands(c):
    """Dequantised [K, M] and [K, N]; the generator poisons the scales inside each group's padding,
    where the data is zero."""
    a = oracle.dequantize(oracle.decode_e4m3(c['a']), c['sfa'], 32, 1)
    b = oracle.dequantize(oracle.decode_e4m3(c['b']), c['sfb'], 32, 1)
    return a, b


def test_k_grouped_matches_reference_oracle(golden):
    for name in ('kgrouped_fp8_bf16', 'kgrouped_fp8_acc_f32'):
        c = golden[name]
        a, b = _k_grouped_operands(c)
        d = oracle.k_grouped_psum_ref(a, b, c['psum'], c['d'].dtype, c=c['c'])
        assert d.shape == c['d'].shape == (3, c['m'], c['n'])
        assert torch.equal(d, c['d']), name
    assert golden['kgrouped_fp8_bf16']['d'][1].abs().max() == 0        # the empty group


def test_k_grouped_sf_layout_model(golden):
    cases = golden['sf_layout_k_grouped']
    assert len(cases) == 6
    for name, c in cases.items():
        out = oracle.required_sf_layout(c['sf'], c['mn'], c['k'], c['gran'], k_psum=c['psum'])
        assert out.stride(-2) == 1 and torch.equal(out, c['expected']), name


def test_psum_layout(golden):
    c = golden['psum_layout']
    sizes, last = [], 0
    for p in c['psum']:
        sizes.append(p - last)
        last = oracle.align(p, 256)
    total, psum = oracle.make_psum_layout(sizes, 256)
    assert total == c['total'] and psum == c['psum']
    assert [(s.start, s.stop) for s in oracle.psum_valid_spans(psum)] == c['valid']
    assert [(s.start, s.stop) for s in oracle.psum_padding_spans(psum)] == c['pad']


def test_quantizers(golden):
    for name, gran in (('quant_fp8_1x128', (1, 128)), ('quant_fp8_128x128', (128, 128))):
        c = golden[name]
        q, sf, rep = oracle.quantize_e4m3(c['x'], gran)
        assert torch.equal(q.view(torch.uint8), c['q'])
        assert torch.equal(sf, c['sf']) and torch.equal(rep, c['repr'])
    c = golden['quant_fp4_1x32']
    q, sf, rep = oracle.quantize_e2m1(c['x'], (1, 32))
    assert torch.equal(q.contiguous(), c['q']) and torch.equal(sf, c['sf']) and torch.equal(rep, c['repr'])
    assert torch.equal(oracle.dequantize(oracle.decode_e2m1_packed(q), sf, 1, 32), rep)


def test_sf_layout_model(golden):
    cases = golden['sf_layout']
    assert len(cases) == 12
    for name, c in cases.items():
        out = oracle.required_sf_layout(c['sf'], c['mn'], c['k'], c['gran'])
        assert out.dtype == torch.int16 and out.shape == c['expected'].shape, name
        assert out.stride(-2) == 1 and out.stride(-1) == out.size(-2), name
        assert torch.equal(out, c['expected']), name


def test_sf_gran_k_128_is_replication():
    torch.manual_seed(0)
    mn, k = 24, 640
    e = torch.randint(100, 140, (mn, 5), dtype=torch.int32)
    sf128 = (e << 23).view(torch.float32)
    sf32 = sf128.repeat_interleave(4, dim=1)
    a = oracle.required_sf_layout(sf128, mn, k, 1, gran_k=128)
    b = oracle.required_sf_layout(sf32, mn, k, 1, gran_k=32)
    assert torch.equal(a, b)
    assert torch.equal(oracle.unpack_required_sf(a, k), sf32)


def test_e2m1_to_e4m3_map_is_exact():
    for code in range(16):
        byte = oracle.e2m1_to_e4m3_byte(code)
        val = torch.tensor([byte], dtype=torch.uint8).view(torch.float8_e4m3fn).float().item()
        assert val == oracle.E2M1_VALUES[code] and (val != 0 or code in (0, 8))


def test_metrics():
    x = torch.randn(64, 64)
    assert oracle.calc_diff(x, x) == 0.0
    assert oracle.max_rel_err(x, x) == 0.0
    assert oracle.calc_diff(x, -x) > 1.9


def test_stochastic_rounding_model_properties():
    """The rounding model keeps exactly representable values, only ever picks one of the two neighbours, and is a
    pure function of the row contents (tests/utils.py:70-92)."""
    torch.manual_seed(0)
    x = torch.randn(7, 37) * 3
    r = oracle.stochastic_round_bf16(x)
    assert torch.equal(r, oracle.stochastic_round_bf16(x))
    lo = (x.view(torch.int32) & ~0xFFFF).view(torch.float32)                 # truncation towards zero
    hi = ((x.view(torch.int32) & ~0xFFFF) + 0x10000).view(torch.float32)     # next BF16 away from zero
    assert ((r.float() == lo) | (r.float() == hi)).all()
    exact = torch.randn(5, 8).bfloat16().float()
    assert torch.equal(oracle.stochastic_round_bf16(exact).float(), exact)
    assert oracle.stochastic_round_bf16(torch.tensor([[float('nan'), 1.0]])).view(torch.int16)[0, 0].item() == 0x7fc0
    # rounding is unbiased enough: the mean error over many values is far below one BF16 ulp
    big = torch.rand(64, 4096) + 1.0
    err = (oracle.stochastic_round_bf16(big).float() - big).mean().abs().item()
    assert err < 2.0 ** -7 / 50


def test_stochastic_rounding_model_matches_reference_fixture(golden):
    c = golden['stochastic_bf16']
    assert torch.equal(oracle.stochastic_round_bf16(c['x']).view(torch.int16), c['expected'])


def test_swiglu_quant_model_properties():
    """Scale = max(amax, 1e-4) / 448 rounded up to a power of two (the same rule as tests/generators.py:27-31 states
    for operands), codes times scale reproduce the value within E4M3 precision, rows outside the psum spans invalid."""
    torch.manual_seed(4)
    x = (torch.randn(70, 512) * 3).bfloat16()
    codes, sf, valid, deq = oracle.swiglu_quant_ref(x, swiglu=False)
    assert codes.shape == (70, 512) and sf.shape == (70, 8) and valid.all()
    amax = x.float().reshape(70, 16, 32).abs().amax(-1)
    expected_scale = oracle.ceil_to_ue8m0(amax.clamp(1e-4) * torch.tensor(1.0 / 448.0))
    got_scale = (sf.contiguous().view(torch.uint8).int() << 23).view(torch.float32)
    assert torch.equal(got_scale, expected_scale)
    assert (deq - x.float()).abs().max() <= (x.float().abs().max() / 16)        # 3 mantissa bits
    assert (codes.view(torch.float8_e4m3fn).float().abs() <= 448).all()
    # SwiGLU with weight, clamp and a psum layout
    y = (torch.randn(384, 512) * 2).bfloat16()
    w = torch.rand(384)
    codes, sf, valid, deq = oracle.swiglu_quant_ref(y, w, [100, 256, 300], 1.5, 128)
    assert valid.sum().item() == 100 + 128 + 44
    assert valid[:100].all() and not valid[100:128].any() and valid[128:300].all() and not valid[300:].any()
    xl, xr = y.float()[:, :256].clamp(max=1.5), y.float()[:, 256:].clamp(-1.5, 1.5)
    ref = torch.nn.functional.silu(xl) * xr * w[:, None]
    assert oracle.calc_diff(deq[valid], ref[valid]) < 2e-3


def test_bf16_family_matches_reference_oracle(golden):
    """BF16 operands carry no scale factors: the same dequantise-free FP32 matmul (tests/generators.py:316-322)."""
    for name in ('bf16_dense_nt', 'bf16_dense_tn_acc_f32', 'bf16_dense_nn_bias'):
        c = golden[name]
        d = oracle.gemm_ref(c['a'].float(), c['b'].float(), c['d'].dtype, c=c['c'] if c['accumulate'] else None,
                            bias=c['c'] if c['with_bias'] else None)
        assert torch.equal(d, c['d']), name
    c = golden['bf16_mgrouped_nt']
    d = oracle.m_grouped_psum_ref(c['a'].float(), c['b'].float(), c['psum'], torch.bfloat16)
    # the reference multiplies in BF16 here (tests/generators.py:351-353): equal up to the last BF16 bit
    assert oracle.calc_diff(d, c['d']) < 1e-5 and oracle.max_rel_err(d, c['d']) < 1e-2
    c = golden['bf16_kgrouped_acc_f32']
    d = oracle.k_grouped_psum_ref(c['a'].float(), c['b'].float(), c['psum'], torch.float32, c=c['c'])
    assert torch.allclose(d, c['d'], rtol=1e-5, atol=1e-4)
