"""ctypes binding of libdg_b200.so (the C ABI declared in include/dg_b200.h).

There is no fallback: if the library is missing, importing any compute entry point raises.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# DG_B200_LIB overrides the location of the library (a differently built libdg_b200.so, for example).
LIB_PATH = os.environ.get('DG_B200_LIB') or os.path.join(_HERE, 'libdg_b200.so')

DG_OK, DG_ERR_INVALID, DG_ERR_UNSUPPORTED, DG_ERR_CUDA, DG_ERR_WORKSPACE = 0, -1, -2, -3, -4
MAJOR_K, MAJOR_MN = 0, 1
GEMM_NORMAL, GEMM_M_GROUPED_PSUM, GEMM_K_GROUPED_PSUM, GEMM_BATCHED, GEMM_M_GROUPED_MASKED = 0, 1, 2, 3, 4
E4M3, E2M1X2, BF16, F32 = 0, 1, 2, 3
EPILOGUE_IDENTITY, EPILOGUE_ALPHA, EPILOGUE_BIAS, EPILOGUE_STOCHASTIC_BF16, EPILOGUE_FP8_QUANT = 0, 1, 2, 3, 4


class GemmDesc(C.Structure):
    _fields_ = [
        ('a', C.c_void_p), ('b', C.c_void_p), ('d', C.c_void_p),
        ('sfa', C.c_void_p), ('sfb', C.c_void_p),
        ('a_dtype', C.c_int32), ('b_dtype', C.c_int32), ('d_dtype', C.c_int32),
        ('m', C.c_uint32), ('n', C.c_uint32), ('k', C.c_uint32),
        ('major_a', C.c_int32), ('major_b', C.c_int32),
        ('outer_stride_a', C.c_uint64), ('outer_stride_b', C.c_uint64), ('outer_stride_d', C.c_uint64),
        ('group_stride_a', C.c_uint64), ('group_stride_b', C.c_uint64), ('group_stride_d', C.c_uint64),
        ('sfa_stride', C.c_uint64), ('sfb_stride', C.c_uint64),
        ('sfa_group_stride', C.c_uint64), ('sfb_group_stride', C.c_uint64),
        ('accumulate', C.c_int32), ('gemm_type', C.c_int32),
        ('grouped_layout', C.c_void_p),
        ('num_groups', C.c_uint32), ('expected_m', C.c_uint32),
        ('epilogue', C.c_int32), ('alpha', C.c_float),
        ('bias', C.c_void_p),
        ('num_sms', C.c_uint32),
        ('sfd', C.c_void_p), ('sfd_stride', C.c_uint64),
        ('deterministic', C.c_int32), ('reserved0', C.c_int32),
    ]


class GemmConfig(C.Structure):
    _fields_ = [
        ('block_m', C.c_uint32), ('block_n', C.c_uint32), ('block_k', C.c_uint32),
        ('num_stages', C.c_uint32), ('cta_group', C.c_uint32), ('split_k', C.c_uint32),
        ('num_ctas', C.c_uint32), ('tmem_cols', C.c_uint32), ('smem_bytes', C.c_uint32),
        ('epilogue_mode', C.c_uint32), ('reserved', C.c_uint32 * 6),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_ if name != 'reserved'} | {
            'accum_stages': self.reserved[0], 'store_bufs': self.reserved[1], 'k_stagger': self.reserved[2],
            'cluster_split': self.reserved[3], 'raster_group': self.reserved[4], 'epilogue_warps': 8 if self.reserved[5] == 2 else 4}


_PROTOTYPES = {
    'dg_select_config': (C.c_int, [C.POINTER(GemmDesc), C.POINTER(GemmConfig)]),
    'dg_gemm_workspace_bytes': (C.c_size_t, [C.POINTER(GemmDesc), C.POINTER(GemmConfig)]),
    'dg_gemm_launch': (C.c_int, [C.POINTER(GemmDesc), C.POINTER(GemmConfig), C.c_void_p, C.c_size_t, C.c_void_p]),
    'dg_gemm_dry_run': (C.c_int, [C.POINTER(GemmDesc), C.POINTER(GemmConfig)]),
    'dg_gemm_launch_static_scratch': (C.c_int, [C.POINTER(GemmDesc), C.POINTER(GemmConfig), C.c_void_p]),
    'dg_quant_fp8_launch': (C.c_int, [
        C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_int, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
        C.c_int, C.c_float, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p]),
    'dg_transform_sf_launch': (C.c_int, [
        C.c_void_p, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32,
        C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
        C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]),
    'dg_pad_rows_launch': (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]),
    'dg_resident_clusters': (C.c_uint32, [C.c_uint32]),
    'dg_expand_fp4_launch': (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]),
    'dg_fp4_expansion_needed': (C.c_int, [C.POINTER(GemmDesc), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    'dg_l2_flush_launch': (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    'dg_device_status': (C.c_int, [C.POINTER(C.c_int32)]),
    'dg_plan_cache_stats': (None, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    'dg_sleep_launch': (C.c_int, [C.c_int64, C.c_uint32, C.c_int, C.c_void_p]),
    'dg_set_overlap_launches': (C.c_int, [C.c_int]),
    'dg_get_overlap_launches': (C.c_int, []),
    'dg_debug_set_trace_buffer': (C.c_int, [C.c_void_p, C.c_size_t]),
    'dg_kernel_launch_count': (C.c_uint64, []),
    'dg_get_num_sms': (C.c_int, []),
    'dg_set_num_sms': (C.c_int, [C.c_int]),
    'dg_get_mk_alignment_for_contiguous_layout': (C.c_int, []),
    'dg_last_error': (C.c_char_p, []),
    'dg_abi_version': (C.c_int, []),
}

STATIC_SCRATCH_BYTES = 4 << 20
ABI_VERSION = 3
EXPORTED_SYMBOLS = tuple(_PROTOTYPES)
_lib = None


def lib() -> C.CDLL:
    """Load the library once. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f'{LIB_PATH} is missing: build it with `python deepgemm-ascend_b200/build.py` '
                '(nvcc, sm_100a). There is no CPU or PyTorch fallback for these kernels.')
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
        if handle.dg_abi_version() != ABI_VERSION:
            raise RuntimeError('libdg_b200.so has an unexpected ABI version')
        _lib = handle
    return _lib


def last_error() -> str:
    msg = lib().dg_last_error()
    return msg.decode() if msg else ''


def check(rc: int) -> None:
    if rc != DG_OK:
        raise RuntimeError(last_error() or f'libdg_b200 error {rc}')
