"""Scale-factor relayout on the GPU against the oracle and the reference-generated fixtures: bit-exact."""

import pytest
import torch

import deep_gemm
import oracle

pytestmark = pytest.mark.gpu


def _check(out: torch.Tensor, expected: torch.Tensor, name: str) -> None:
    assert out.dtype == torch.int16 and out.shape == expected.shape, name
    assert out.stride(-2) == 1 and out.stride(-1) == out.size(-2), name
    assert torch.equal(out.cpu(), expected), name


def test_fixtures_from_the_reference_layout_model(golden):
    for name, c in golden['sf_layout'].items():
        for mn_major in (False, True):
            sf = c['sf']
            if mn_major and sf.size(-1) > 1 and sf.size(-2) > 1:
                sf = sf.transpose(-2, -1).contiguous().transpose(-2, -1)
            kwargs = {'num_groups': sf.size(0)} if sf.dim() == 3 else {}
            out = deep_gemm.transform_sf_into_required_layout(
                sf.cuda(), c['mn'], c['k'], (c['gran'], c['gran'], 32), is_sfa=True, **kwargs)
            _check(out, c['expected'], f'{name} mn_major={mn_major}')


@pytest.mark.parametrize('dtype', [torch.float32, torch.int16])
@pytest.mark.parametrize('gran', [1, 32, 128])
@pytest.mark.parametrize('mn,k', [(4096, 7168), (4097, 7296), (300, 128)])
def test_random_against_oracle(dtype, gran, mn, k):
    torch.manual_seed(mn + k + gran)
    div = 32 if dtype == torch.float32 else 64
    shape = (oracle.ceil_div(mn, gran), oracle.ceil_div(k, div))
    if dtype == torch.float32:
        sf = (torch.randint(1, 255, shape, dtype=torch.int32) << 23).view(torch.float32)
    else:
        sf = torch.randint(-32768, 32768, shape, dtype=torch.int16)
    out = deep_gemm.transform_sf_into_required_layout(sf.cuda(), mn, k, (gran, gran, 32), is_sfa=False)
    _check(out, oracle.required_sf_layout(sf, mn, k, gran), f'{dtype} gran={gran} mn={mn} k={k}')


def test_identity_fast_path_on_device():
    sf = torch.randint(-32768, 32768, (112, 4096), dtype=torch.int16, device='cuda').transpose(0, 1)
    assert deep_gemm.transform_sf_into_required_layout(sf, 4096, 7168, (1, 1, 32), is_sfa=True) is sf


@pytest.mark.parametrize('dtype', [torch.float32, torch.int16])
@pytest.mark.parametrize('gran', [1, 32])
def test_group_padding_is_zeroed_even_when_poisoned(dtype, gran):
    """tests/test_layout.py:91-97: padding rows hold -1 (an invalid float) / arbitrary bits and come out as 0."""
    torch.manual_seed(3)
    sizes = [300, 0, 513, 255, 256, 1]
    total, psum = oracle.make_psum_layout(sizes, 256)
    k = 704
    div = 32 if dtype == torch.float32 else 64
    shape = (total // gran, oracle.ceil_div(k, div))
    if dtype == torch.float32:
        sf = (torch.randint(1, 255, shape, dtype=torch.int32) << 23).view(torch.float32)
        poison = -1.0
    else:
        sf = torch.randint(-32768, 32768, shape, dtype=torch.int16)
        poison = 0x7FFF
    expected = oracle.required_sf_layout(sf, total, k, gran, psum=psum)
    poisoned = sf.clone()
    for span in oracle.psum_padding_spans(psum, 256, gran):
        poisoned[span] = poison
    layout = torch.tensor(psum, dtype=torch.int32, device='cuda')
    out = deep_gemm.transform_sf_into_required_layout(poisoned.cuda(), total, k, (gran, gran, 32), is_sfa=True,
                                                      psum_layout=layout)
    _check(out, expected, f'psum {dtype} gran={gran}')
    # the same source with the row axis contiguous (its own kernel for per-row scales); no invalid-scale report from padding
    src = poisoned.cuda().t().contiguous().t()
    out = deep_gemm.transform_sf_into_required_layout(src, total, k, (gran, gran, 32), is_sfa=True, psum_layout=layout)
    if dtype == torch.int16 and gran == 1:
        # packed per-row scales that already have the required layout come back untouched, padding included
        # (csrc/apis/layout.hpp:37-62 decides before it looks at the psum layout)
        assert out.data_ptr() == src.data_ptr()
    else:
        _check(out, expected, f'psum {dtype} gran={gran} MN-major source')
    assert deep_gemm.device_status() == 0


def test_gran_k_128_expands_to_four_blocks():
    torch.manual_seed(5)
    mn, k = 520, 7168 + 128
    for gran in (1, 128):
        rows = oracle.ceil_div(mn, gran)
        sf = (torch.randint(90, 140, (rows, oracle.ceil_div(k, 128)), dtype=torch.int32) << 23).view(torch.float32)
        out = deep_gemm.transform_sf_into_required_layout(sf.cuda(), mn, k, (gran, gran, 128), is_sfa=True)
        _check(out, oracle.required_sf_layout(sf, mn, k, gran, gran_k=128), f'gran_k=128 gran_mn={gran}')
        # the same scales stored with the row axis contiguous, dense and with rows that end off the 8-row vector width
        for rows_used in (mn, mn - 3):
            src = sf[:oracle.ceil_div(rows_used, gran)].cuda().t().contiguous().t()
            out = deep_gemm.transform_sf_into_required_layout(src, rows_used, k, (gran, gran, 128), is_sfa=True)
            _check(out, oracle.required_sf_layout(sf[:oracle.ceil_div(rows_used, gran)], rows_used, k, gran, gran_k=128),
                   f'gran_k=128 gran_mn={gran} MN-major rows={rows_used}')


@pytest.mark.parametrize('dtype', [torch.float32, torch.int16])
@pytest.mark.parametrize('mn_major', [False, True])
@pytest.mark.parametrize('num_batches', [1, 2, 4])
def test_reference_layout_product(dtype, mn_major, num_batches):
    """tests/generators.py:682-690: (4096, 4097, 8192) rows x (128, 7168, 7296) columns of K x the three row
    granularities, dense and batched, K-major and MN-major sources, FP32 and packed int16 sources."""
    for mn in (4096, 4097, 8192):
        for k in (128, 7168, 7296):
            for gran in (1, 32, 128):
                torch.manual_seed(mn * 7 + k + gran + num_batches)
                div = 32 if dtype == torch.float32 else 64
                shape = (oracle.ceil_div(mn, gran), oracle.ceil_div(k, div))
                if num_batches > 1:
                    shape = (num_batches, *shape)
                if dtype == torch.float32:
                    sf = (torch.randint(1, 255, shape, dtype=torch.int32) << 23).view(torch.float32)
                else:
                    sf = torch.randint(-32768, 32768, shape, dtype=torch.int16)
                expected = oracle.required_sf_layout(sf, mn, k, gran)
                src = sf.cuda()
                if mn_major and shape[-1] > 1 and shape[-2] > 1:
                    src = src.transpose(-2, -1).contiguous().transpose(-2, -1)
                kwargs = {'num_groups': num_batches} if num_batches > 1 else {}
                out = deep_gemm.transform_sf_into_required_layout(src, mn, k, (gran, gran, 32), is_sfa=True, **kwargs)
                _check(out, expected, f'{dtype} mn_major={mn_major} batches={num_batches} mn={mn} k={k} gran={gran}')
    assert deep_gemm.device_status() == 0
