"""deep_gemm for NVIDIA B200: block-scaled FP8 / FP8xFP4 GEMM behind the DeepGEMM-Ascend Python API.

The names, arguments and error text of the hot path follow the reference's `deep_gemm/__init__.py:25-81`;
everything else of the reference (attention, MegaMoE, ACLNN wrappers) is out of scope
and not exported. Importing this package never initialises a CUDA context.
"""

__version__ = '0.1.1'

from . import _api, locality_domain  # noqa: F401
from ._api import (  # noqa: F401
    device_status,
    get_deterministic_algorithms,
    get_dry_run,
    get_mk_alignment_for_contiguous_layout,
    get_npu_arch,
    get_num_sms,
    get_theoretical_mk_alignment_for_contiguous_layout,
    init,
    set_dry_run,
    set_mk_alignment_for_contiguous_layout,
    set_npu_arch,
    set_num_sms,
    use_deterministic_algorithms,
)

# The entry points of the hot path come from the compiled `_C` torch extension (csrc/python_api.cpp: the reference's
# csrc/apis surface in C++ over the C ABI) when it has been built, otherwise from the Python host layer `_api`, which
# has the same names, arguments and messages and calls the same C ABI. Either way the kernels are libdg_b200.so.
_HOT_PATH_NAMES = (
    'fp8_fp4_gemm_nt', 'fp8_fp4_gemm_nn', 'fp8_fp4_gemm_tn', 'fp8_fp4_gemm_tt',
    'fp8_gemm_nt', 'fp8_gemm_nn', 'fp8_gemm_tn', 'fp8_gemm_tt',
    'm_grouped_fp8_fp4_gemm_nt_contiguous', 'm_grouped_fp8_fp4_gemm_nn_contiguous',
    'm_grouped_fp8_gemm_nt_contiguous', 'm_grouped_fp8_gemm_nn_contiguous',
    'm_grouped_fp8_fp4_gemm_nt_masked', 'm_grouped_fp8_gemm_nt_masked',
    'k_grouped_fp8_gemm_tn_contiguous', 'k_grouped_fp8_gemm_nt_contiguous',
    'bf16_gemm_nt', 'bf16_gemm_nn', 'bf16_gemm_tn', 'bf16_gemm_tt',
    'm_grouped_bf16_gemm_nt_contiguous', 'm_grouped_bf16_gemm_nn_contiguous', 'k_grouped_bf16_gemm_tn_contiguous',
    'fp8_bmm', 'fp8_einsum', 'bf16_bmm', 'einsum',
    'transform_sf_into_required_layout', 'transform_k_grouped_sf_into_required_layout', 'get_recipe', 'npu_sleep',
)
_C = _api._C
BACKEND = '_C' if _C is not None else 'python'
for _name in _HOT_PATH_NAMES:
    globals()[_name] = getattr(_C if _C is not None else _api, _name)
del _name

from . import epilogue, quant_ops, testing  # noqa: E402,F401
from .quant_ops import cast_to_fp8, swiglu_apply_weight_to_fp8  # noqa: F401
from .locality_domain import (  # noqa: F401
    destroy_localizer,
    get_num_locality_domains,
    is_localization_available,
    is_localized,
    localize,
)


def get_library_root_path() -> str:
    import os
    return os.path.dirname(os.path.realpath(__file__))
