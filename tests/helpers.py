"""Seeded input generators and comparison helpers shared by the parity tests.

Inputs follow the two distributions the reference uses (tests/generators.py:124-166 uniform codes with
power-of-two scales; :61-95 N(0,1) block quantisation) and are built on the CPU so that the oracle and the
CUDA path see identical bytes.
"""

from __future__ import annotations

import random

import torch

import oracle

# Tolerances on BF16 / FP32 output: 1 - cosine <= 1e-3 and max relative error <= 2e-2.
COS_TOL = 1e-3
REL_TOL = 2e-2


def seed_all(seed: int = 0) -> None:
    random.seed(seed)
    torch.manual_seed(seed)


def uniform_fp8(shape, gran, sf_choices=(2.0 ** -9, 2.0 ** -8, 2.0 ** -7)):
    """Every non-NaN E4M3 code equally likely; scales drawn from three powers of two.
    Returns (data float8 [..., MN, K], sf fp32, dequantised fp32)."""
    raw = torch.randint(0, 254, shape, dtype=torch.uint8)
    raw += (raw >= 0x7F).to(torch.uint8)
    raw[raw == 0xFF] = 0xFE
    data = raw.view(torch.float8_e4m3fn)
    sf_shape = (*shape[:-2], oracle.ceil_div(shape[-2], gran[0]), oracle.ceil_div(shape[-1], gran[1]))
    table = torch.tensor(sf_choices, dtype=torch.float32)
    sf = table[torch.randint(0, len(sf_choices), sf_shape)].contiguous()
    return data, sf, oracle.dequantize(data.float(), sf, gran[0], gran[1])


def uniform_codes(shape) -> torch.Tensor:
    """Random E4M3 bytes (uint8) without the two NaN codes: the distribution of tests/generators.py:137-153, drawn
    eight bytes at a time because some tensors of the full-size tests hold up to two billion codes."""
    numel = 1
    for s in shape:
        numel *= s
    raw = torch.randint(-2 ** 63, 2 ** 63 - 1, ((numel + 7) // 8,), dtype=torch.int64).view(torch.uint8)[:numel].view(shape)
    raw -= ((raw & 0x7F) == 0x7F).to(torch.uint8)           # 0x7f -> 0x7e, 0xff -> 0xfe
    return raw


def pow2_scales(shape) -> torch.Tensor:
    """One of {2^-9, 2^-8, 2^-7} per element (tests/generators.py:141), FP32."""
    table = torch.tensor([2.0 ** -9, 2.0 ** -8, 2.0 ** -7], dtype=torch.float32)
    return table[torch.randint(0, 3, shape)].contiguous()


def uniform_fp4(mn, k, gran, mn_major: bool, sf_choices=(0.25, 0.5, 1.0)):
    """Uniform random packed E2M1 (tests/generators.py:155-164): returns (packed int8 whose logical shape is
    [MN, K] with two codes per byte along the contiguous axis, sf fp32, dequantised fp32 [MN, K]).
    K-major: tensor [MN, K/2]; MN-major: tensor of shape [MN/2, K] with strides (1, MN/2)."""
    if mn_major:
        storage = torch.randint(-128, 128, (k, mn // 2), dtype=torch.int8)
        data = storage.transpose(0, 1)
        vals = oracle.decode_e2m1_packed(storage, axis=-1).transpose(0, 1)
    else:
        data = torch.randint(-128, 128, (mn, k // 2), dtype=torch.int8)
        vals = oracle.decode_e2m1_packed(data, axis=-1)
    table = torch.tensor(sf_choices, dtype=torch.float32)
    sf = table[torch.randint(0, len(sf_choices), (oracle.ceil_div(mn, gran[0]), oracle.ceil_div(k, gran[1])))].contiguous()
    return data, sf, oracle.dequantize(vals, sf, gran[0], gran[1])


def normal_fp8(shape, gran):
    x = torch.randn(shape, dtype=torch.float32)
    if x.dim() == 2:
        return oracle.quantize_e4m3(x, gran)
    parts = [oracle.quantize_e4m3(x[i], gran) for i in range(x.size(0))]
    return (torch.stack([p[0].view(torch.uint8) for p in parts]).view(torch.float8_e4m3fn),
            torch.stack([p[1] for p in parts]), torch.stack([p[2] for p in parts]))


def with_major(t: torch.Tensor, mn_major: bool) -> torch.Tensor:
    """Same logical [..., MN, K] tensor, stored with MN contiguous when `mn_major`."""
    if not mn_major:
        return t.contiguous()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).transpose(-2, -1).contiguous().transpose(-2, -1).view(torch.float8_e4m3fn)
    return t.transpose(-2, -1).contiguous().transpose(-2, -1)


def assert_close(out: torch.Tensor, ref: torch.Tensor, what: str = '') -> tuple[float, float]:
    out, ref = out.detach().cpu(), ref.detach().cpu()
    assert out.shape == ref.shape, f'{what}: shape {out.shape} vs {ref.shape}'
    assert torch.isfinite(out.float()).all(), f'{what}: non-finite output'
    diff = oracle.calc_diff(out, ref)
    rel = oracle.max_rel_err(out, ref)
    assert diff <= COS_TOL, f'{what}: 1-cos = {diff:.3e}'
    assert rel <= REL_TOL, f'{what}: max rel err = {rel:.3e}'
    return diff, rel


def assert_close_device(out: torch.Tensor, ref: torch.Tensor, what: str = '') -> tuple[float, float]:
    """Same two checks as `assert_close` for tensors too large to compare comfortably on the host: `out` stays on
    its CUDA device, the oracle's `ref` is copied there, and only the metrics (plumbing, not the oracle) are
    evaluated on the device, in row chunks so that the FP64 temporaries stay small."""
    assert out.shape == ref.shape, f'{what}: shape {out.shape} vs {ref.shape}'
    out2, ref2 = out.reshape(-1, out.shape[-1]), ref.reshape(-1, ref.shape[-1])
    rows = max(1, (1 << 24) // max(1, out2.shape[-1]))
    dot = sq = 0.0
    scale = float(ref2.abs().max()) if ref2.numel() else 0.0
    worst = 0.0
    for r0 in range(0, out2.shape[0], rows):
        x = out2[r0:r0 + rows].double()
        y = ref2[r0:r0 + rows].to(out.device).double()
        assert torch.isfinite(x).all(), f'{what}: non-finite output'
        dot += float((x * y).sum())
        sq += float((x * x + y * y).sum())
        den = torch.clamp(y.abs(), min=scale / 64) if scale > 0 else torch.ones_like(y)
        worst = max(worst, float(((x - y).abs() / den).max()))
    diff = 0.0 if sq == 0 else 1 - 2 * dot / sq
    assert diff <= COS_TOL, f'{what}: 1-cos = {diff:.3e}'
    assert worst <= REL_TOL, f'{what}: max rel err = {worst:.3e}'
    return diff, worst
