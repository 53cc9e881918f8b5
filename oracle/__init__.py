"""CPU oracle for the block-scaled FP8 / FP8xFP4 GEMM path.

TEST INFRASTRUCTURE ONLY. Nothing in the shipped package imports this module;
it is the checker used by the tests, by the smoke entry and by the CPU-baseline
leg of the benchmark. The product path is the CUDA library and fails loudly
when that library is missing.

The oracle restates, on the CPU with torch/numpy, what the reference's own test
suite treats as ground truth: dequantise both operands with their UE8M0 block
scales, multiply in FP32, apply alpha / bias / accumulate, cast once.

Pinning: the restatement is checked against fixtures under ``tests/golden``
that were produced by importing the reference's own ``tests/generators.py`` and
``tests/test_layout.py`` (see ``tests/golden/make_golden.py``). The masked
grouped entry point and ``gran_k = 128`` recipes have no reference test at all,
so for those two the oracle is "parity unpinned" by the reference.
"""

from .mxgemm import (  # noqa: F401
    E2M1_VALUES,
    calc_diff,
    ceil_to_ue8m0,
    decode_e2m1_packed,
    decode_e4m3,
    dequantize,
    e2m1_to_e4m3_byte,
    gemm_ref,
    k_grouped_psum_ref,
    m_grouped_masked_ref,
    m_grouped_psum_ref,
    max_rel_err,
    quantize_e2m1,
    quantize_e4m3,
    stochastic_round_bf16,
)
from .quant import swiglu_quant_ref  # noqa: F401
from .sf_layout import (  # noqa: F401
    align,
    ceil_div,
    make_psum_layout,
    psum_padding_spans,
    psum_valid_spans,
    required_sf_layout,
    unpack_required_sf,
)
