"""Host layer of deep_gemm for B200: the reference's `csrc/apis` surface over the C ABI.

Mirrors, with the same names, argument meaning and error text:
  * csrc/apis/gemm.hpp:60-197 (get_gemm_desc), :225-256 (fp8_fp4_gemm_*), :289-324 (m-grouped contiguous);
  * csrc/apis/layout.hpp:37-128 (check_sf_layout, transform_sf_into_required_layout, get_recipe);
  * csrc/utils/layout.hpp:37-99,140-219 (majors, early returns, shape inference);
  * csrc/jit_kernels/epilogue_class.hpp:14-128 and csrc/apis/runtime.hpp:12-62.
Tensors are only unpacked here (pointers, sizes, strides); validation of the problem, the tiling
heuristic, TMA descriptors and the launches live in libdg_b200.so.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
import warnings
from typing import Optional

import torch

from . import _lib as L

# The compiled host layer, when it has been built (`python deepgemm-ascend_b200/build.py`); DG_PYTHON_HOST=1 keeps to
# this module. Its process-wide knobs are kept in step with the ones below.
_C = None
if os.environ.get('DG_PYTHON_HOST', '0') in ('', '0'):
    try:
        from . import _C  # type: ignore[attr-defined,no-redef]
    except ImportError:
        _C = None

PACKED_FP4 = torch.int8           # csrc/utils/dtype.hpp:9
MK_ALIGNMENT = 256                # csrc/jit/jit.hpp:59-73

_state = threading.local()
_DEBUG = os.environ.get('DG_JIT_DEBUG', '0') not in ('', '0')
_global = {'dry_run': False, 'deterministic': False, 'arch': 100}
_workspaces: dict = {}
_ws_lock = threading.Lock()


def _host_assert(cond: bool, msg: str = 'Assertion failed') -> None:
    if not cond:
        raise RuntimeError(msg)


def _ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def _align(a: int, b: int) -> int:
    return _ceil_div(a, b) * b


# ------------------------------------------------------------------------------------------------
# Epilogue classes (csrc/jit_kernels/epilogue_class.hpp, csrc/apis/epilogue_class.hpp:10-21)
# ------------------------------------------------------------------------------------------------
class Epilogue:
    """Base class of the objects accepted by the `epilogue=` argument."""

    def check(self, c, d) -> None:
        _host_assert(d.dtype in (torch.bfloat16, torch.float32))

    def get_output_sf(self):
        return None


class Identity(Epilogue):
    pass


class Alpha(Epilogue):
    def __init__(self, alpha: float):
        self.alpha = float(alpha)


class _Bias(Epilogue):
    def __init__(self, bias: torch.Tensor):
        self.bias = bias


class BF16StochasticRounding(Epilogue):
    """FP32 accumulator -> BF16 by stochastic rounding with the reference's hash (operators.hpp:224-343)."""

    def check(self, c, d) -> None:
        _host_assert(c is None and d.dtype == torch.bfloat16, 'Stochastic rounding requires a direct BF16 output')


class FP8Quantization(Epilogue):
    """E4M3 output with one UE8M0 scale per row per 32 columns, written to `sfd` (int16 [M, batches * N / 64],
    MN-major, two scale bytes per element); csrc/jit_kernels/epilogue_class.hpp:80-108."""

    def __init__(self, sfd: torch.Tensor):
        self.sfd = sfd

    def get_output_sf(self):
        return self.sfd

    def check(self, c, d) -> None:
        _host_assert(c is None and d.dtype == torch.float8_e4m3fn, 'FP8 quantization requires a direct E4M3 output')
        _host_assert(d.dim() in (2, 3))
        m, n = d.size(-2), d.size(-1)
        batches = d.size(0) if d.dim() == 3 else 1
        _host_assert(n % 128 == 0, 'FP8 output requires N to be a multiple of 128')
        _host_assert(d.stride(-1) == 1 and (d.dim() == 2 or d.stride(0) == n),
                     'FP8 output must be contiguous in N and, when batched, hold the batches side by side in a row')
        sfd = self.sfd
        _host_assert(sfd.dtype == torch.int16 and sfd.dim() == 2 and sfd.device == d.device,
                     'sfd must be a 2-D int16 tensor on the output device')
        _host_assert(sfd.size(0) == m and sfd.size(1) == batches * n // 64, 'sfd must have shape [M, batches * N / 64]')
        _host_assert((sfd.stride(0) == 1 or m == 1) and sfd.stride(1) == m, 'sfd must be MN-major')


def _resolve_epilogue(epilogue, c, d, alpha=None, sfd=None) -> Epilogue:
    _host_assert((epilogue is not None) + (alpha is not None) + (sfd is not None) <= 1,
                 'The epilogue class, alpha and the FP8 output pair are exclusive')
    if alpha is not None:
        resolved = Alpha(alpha)
    elif sfd is not None:
        resolved = FP8Quantization(sfd)
    else:
        resolved = epilogue if epilogue is not None else Identity()
    _host_assert(isinstance(resolved, Epilogue), 'epilogue must be a deep_gemm.epilogue object')
    resolved.check(c, d)
    return resolved


# ------------------------------------------------------------------------------------------------
# Runtime knobs (csrc/apis/runtime.hpp:12-62)
# ------------------------------------------------------------------------------------------------
def get_num_sms() -> int:
    return L.lib().dg_get_num_sms()


def set_num_sms(n: int) -> None:
    L.check(L.lib().dg_set_num_sms(int(n)))


def set_npu_arch(arch: int) -> None:
    _global['arch'] = int(arch)
    if _C is not None:
        _C.set_npu_arch(int(arch))


def get_npu_arch() -> int:
    return _global['arch']


def set_mk_alignment_for_contiguous_layout(value: int) -> None:
    _host_assert(int(value) == MK_ALIGNMENT, f'mk alignment for the contiguous layout is fixed at {MK_ALIGNMENT}')


def get_mk_alignment_for_contiguous_layout() -> int:
    return MK_ALIGNMENT


def get_theoretical_mk_alignment_for_contiguous_layout() -> int:
    return MK_ALIGNMENT


def use_deterministic_algorithms(enabled: bool) -> None:
    _global['deterministic'] = bool(enabled)
    if _C is not None:
        _C.use_deterministic_algorithms(bool(enabled))


def get_deterministic_algorithms() -> bool:
    return _global['deterministic']


def set_dry_run(value: bool) -> None:
    _global['dry_run'] = bool(value)
    if _C is not None:
        _C.set_dry_run(bool(value))


def get_dry_run() -> bool:
    return _global['dry_run']


def init(version: str = '', library_root_path: str = '') -> None:
    """csrc/apis/runtime.hpp:41-44. The reference points its JIT at the installed headers here; this build has no
    JIT, so the call only checks that the compiled library is present and of the expected ABI (no device is touched)."""
    L.lib()


def npu_sleep(sleep_cycles: int, *, marker: int = 0) -> None:
    """csrc/apis/runtime.hpp:64-79: enqueue a kernel of one block per SM that spins for `sleep_cycles` SM clock
    cycles (at most 4e9). `marker` selects the kernel's name so that a profiler can find begin / end marks."""
    if get_dry_run():
        return
    device = torch.device('cuda', torch.cuda.current_device())
    L.check(L.lib().dg_sleep_launch(int(sleep_cycles), int(marker), get_num_sms(), _stream_ptr(device)))


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# ------------------------------------------------------------------------------------------------
# Layout helpers (csrc/utils/layout.hpp)
# ------------------------------------------------------------------------------------------------
def _major_check(t: torch.Tensor) -> None:
    if t.stride(-2) == 1 and t.stride(-1) == 1:
        raise RuntimeError(f'Ambiguous major axis, the tensor has both last two dimensions contiguous, '
                           f'strides={list(t.stride())}')
    _host_assert(t.stride(-2) == 1 or t.stride(-1) == 1)


def _major_ab(t: torch.Tensor) -> int:
    _major_check(t)
    return L.MAJOR_K if t.stride(-1) == 1 else L.MAJOR_MN


def _outer_stride(t: torch.Tensor, major: int) -> int:
    return t.stride(-2) if major == L.MAJOR_K else t.stride(-1)


def _shape_by_spec(out_dims: str, specs: list[tuple[str, torch.Tensor]]) -> tuple[int, ...]:
    """csrc/utils/layout.hpp:140-219: named-axis shape inference with conflict diagnostics; a packed-FP4
    tensor counts double along its contiguous axis."""
    majors = []
    for idx, (dims, t) in enumerate(specs):
        if t.dim() != len(dims):
            raise RuntimeError(f'Shape mismatch: tensor #{idx}, annotation="{dims}"')
        major = next((i for i in range(t.dim()) if t.stride(i) == 1), -1)
        if major < 0:
            raise RuntimeError(f'Tensor #{idx} annotation="{dims}" doesn\'t have major axis, strides={list(t.stride())}')
        majors.append(major)
    result = []
    for name in out_dims:
        found = None
        for idx, (dims, t) in enumerate(specs):
            for axis, ch in enumerate(dims):
                if ch != name:
                    continue
                value = t.size(axis) * (2 if (t.dtype == PACKED_FP4 and axis == majors[idx]) else 1)
                if found is None:
                    found = (value, idx, dims, axis)
                elif found[0] != value:
                    raise RuntimeError(
                        f"Conflicting shape dimension '{name}': tensor #{idx} annotation=\"{dims}\" axis={axis} gives {value}, "
                        f'but tensor #{found[1]} annotation="{found[2]}" axis={found[3]} gives {found[0]}')
        result.append(found[0] if found else 0)
    return tuple(result)


def _same_buffer(c: torch.Tensor, d: torch.Tensor) -> bool:
    """csrc/apis/gemm.hpp:105-106: meta and empty tensors have no address, so compare storage identity."""
    if c is d:
        return True
    if d.is_meta or d.numel() == 0:
        return (c.untyped_storage()._cdata == d.untyped_storage()._cdata and
                c.storage_offset() == d.storage_offset())
    return c.data_ptr() == d.data_ptr()


def _gemm_early_return(m, n, k, d, c, with_bias) -> bool:
    """csrc/utils/layout.hpp:54-86."""
    if m == 0 or n == 0:
        return True
    is_cd_same = c is not None and _same_buffer(c, d)
    if is_cd_same:
        _host_assert(c.shape == d.shape and c.stride() == d.stride())
    _host_assert(d.dtype in (torch.bfloat16, torch.float32, torch.float8_e4m3fn))
    if c is not None:
        _host_assert(c.dim() >= 2 and c.stride(-1) == 1)
        _host_assert(d.dtype == c.dtype)
    if k == 0:
        if not is_cd_same and not d.is_meta:
            d.copy_(c.expand_as(d)) if c is not None else d.zero_()
        return True
    if c is not None and not is_cd_same and not with_bias and not d.is_meta:
        d.copy_(c)
    return False


# ------------------------------------------------------------------------------------------------
# Scale-factor layout (csrc/apis/layout.hpp)
# ------------------------------------------------------------------------------------------------
def get_recipe(recipe, recipe_a, recipe_b) -> tuple[int, int, int, int]:
    """Returns (gran_m, gran_n, gran_k_a, gran_k_b). The reference requires both gran_k to be 32
    (csrc/apis/layout.hpp:55,125); here each may be 32 or 128 because a per-128 scale is expanded to the
    per-32 layout by the transform."""
    _host_assert(not (recipe is not None and (recipe_a is not None or recipe_b is not None)),
                 'recipe and recipe_a / recipe_b are mutually exclusive')
    if recipe is not None:
        gm, gn, gk = recipe
        return int(gm), int(gn), int(gk), int(gk)
    gm, gka = recipe_a if recipe_a is not None else (1, 32)
    gn, gkb = recipe_b if recipe_b is not None else (1, 32)
    return int(gm), int(gn), int(gka), int(gkb)


def _check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups) -> bool:
    """csrc/apis/layout.hpp:37-65. True when `sf` already is the required layout."""
    _host_assert(sf.dtype in (torch.float32, torch.int16), 'SF must be float32 or int16 (packed ue8m0x2)')
    _host_assert(sf.dim() == (1 if num_groups is not None else 0) + 2, 'SF has the wrong number of dimensions')
    _host_assert(sf.stride(-1) == 1 or sf.stride(-2) == 1 or sf.size(-1) == 1 or sf.size(-2) == 1,
                 'SF input must be contiguous in either the last or second-to-last dimension')
    if num_groups is not None:
        _host_assert(sf.size(-3) == num_groups)
    _host_assert(gran_k in (32, 128), 'gran_k must be 32 (or 128, expanded by the transform)')
    div_k = gran_k if sf.dtype == torch.float32 else gran_k * 2
    _host_assert(sf.size(-2) == _ceil_div(mn, gran_mn), f'SF rows: expected {_ceil_div(mn, gran_mn)}, got {sf.size(-2)}')
    _host_assert(sf.size(-1) == _ceil_div(k, div_k), f'SF columns: expected {_ceil_div(k, div_k)}, got {sf.size(-1)}')
    if sf.dtype == torch.int16 and gran_mn == 1 and gran_k == 32 and sf.stride(-2) == 1 and sf.stride(-1) == sf.size(-2):
        return num_groups is None or sf.stride(-3) == sf.size(-2) * sf.size(-1)
    return False


def _check_psum_layout(psum_layout, sf) -> int:
    _host_assert(psum_layout.device == sf.device, 'grouped_layout must be on the same device as the SF input')
    _host_assert(psum_layout.dtype == torch.int32 and psum_layout.dim() == 1 and psum_layout.is_contiguous(),
                 'grouped_layout must be a contiguous 1D int32 tensor')
    _host_assert(psum_layout.numel() > 0, 'grouped_layout must contain at least one group')
    return psum_layout.numel()


_SF_INVALID_MESSAGE = "Float32 SF must be non-negative and can't have non-zero mantissa"
STATUS_INVALID_SCALE_FACTOR = 201
_sf_flags: dict = {}


def _sf_invalid_flag(device: torch.device) -> torch.Tensor:
    """One int32 per device that the transform kernel sets when it meets an FP32 scale that is negative or not a
    power of two. The reference asserts on the device (deep_gemm/include/deep_gemm/transform_sf.hpp:13-21); a
    CUDA kernel that traps loses the context, so the flag is reported by `device_status()` at the caller's next
    synchronisation point, or at once when DG_JIT_DEBUG is set."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    with _ws_lock:
        flag = _sf_flags.get(key)
        if flag is None:
            flag = torch.zeros(1, dtype=torch.int32, device=device)
            _sf_flags[key] = flag
        return flag


def _launch_transform_sf(sf, mn, k, gran_mn, gran_k, psum_layout, tma_aligned: bool, k_psum_layout=None):
    """csrc/jit_kernels/transform_sf.hpp:15-105. With `tma_aligned` the column stride of the result is
    rounded up to 8 elements (what the GEMM's TMA descriptor needs); the public entry point never does that.
    `psum_layout` pads along MN (m-grouped operands), `k_psum_layout` along K (k-grouped operands)."""
    squeeze = sf.dim() == 2
    if squeeze:
        sf = sf.unsqueeze(0)
    _host_assert(sf.dim() == 3, f'Transform SF input must have 2 or 3 dimensions, but got {sf.dim() - int(squeeze)}')
    _host_assert(1 <= gran_mn <= 128 and (gran_mn & (gran_mn - 1)) == 0, 'gran_mn only support a power of two in [1, 128]')
    batches = sf.size(0)
    num_groups = 0
    if psum_layout is not None:
        _host_assert(batches == 1, 'Grouped transform SF requires one logical batch and grouped_layout')
        num_groups = _check_psum_layout(psum_layout, sf)
    num_k_groups = 0
    if k_psum_layout is not None:
        _host_assert(batches == 1 and psum_layout is None,
                     'Grouped transform SF requires one logical batch and grouped_layout')
        _host_assert(gran_k == 32, 'K-grouped transform SF requires gran_k = 32')
        num_k_groups = _check_psum_layout(k_psum_layout, sf)
    is_fp32 = sf.dtype == torch.float32
    k32 = _ceil_div(k, 32)
    dst_cols = sf.size(-1) if (not is_fp32 and gran_k == 32) else _ceil_div(k32, 2)
    col_stride = _align(mn, 8) if tma_aligned else mn
    storage = torch.empty((batches, dst_cols, col_stride), dtype=torch.int16, device=sf.device)
    out = storage[:, :, :mn].transpose(-2, -1)
    if out.numel() and not get_dry_run() and not sf.is_meta:
        flag = _sf_invalid_flag(sf.device) if is_fp32 else None
        rc = L.lib().dg_transform_sf_launch(
            sf.data_ptr(), int(is_fp32), sf.stride(-2), sf.stride(-1), sf.stride(0), sf.size(-2), sf.size(-1),
            storage.data_ptr(), col_stride, dst_cols * col_stride, mn, k32, gran_mn, gran_k // 32, batches,
            psum_layout.data_ptr() if psum_layout is not None else None, num_groups, MK_ALIGNMENT,
            flag.data_ptr() if flag is not None else None,
            k_psum_layout.data_ptr() if k_psum_layout is not None else None, num_k_groups,
            _stream_ptr(sf.device))
        L.check(rc)
        if flag is not None and _DEBUG and int(flag.item()) != 0:
            flag.zero_()
            raise RuntimeError(_SF_INVALID_MESSAGE)
    return out.squeeze(0) if squeeze else out


def transform_sf_into_required_layout(sf: torch.Tensor, mn: int, k: int, recipe,
                                      num_groups: Optional[int] = None, is_sfa: Optional[bool] = None,
                                      disable_ue8m0_cast: bool = False,
                                      psum_layout: Optional[torch.Tensor] = None) -> torch.Tensor:
    """csrc/apis/layout.hpp:68-92. Returns int16 [..., MN, ceil(K/64)], MN-major; returns `sf` itself when it
    already has that layout."""
    recipe = tuple(recipe)
    if len(recipe) == 3:
        _host_assert(is_sfa is not None, 'is_sfa must be set for a 3-element recipe')
        gran_mn, gran_k = (recipe[0] if is_sfa else recipe[1]), recipe[2]
    else:
        _host_assert(len(recipe) == 2, 'recipe must have 2 or 3 elements')
        gran_mn, gran_k = recipe
    return _transform_sf(sf, mn, k, int(gran_mn), int(gran_k), num_groups, disable_ue8m0_cast, psum_layout, False)


def transform_k_grouped_sf_into_required_layout(sf: torch.Tensor, mn: int, k: int, recipe, is_sfa: Optional[bool],
                                                psum_layout: torch.Tensor) -> torch.Tensor:
    """csrc/apis/layout.hpp:94-111. Scale factors of a k-grouped operand ([MN, K] with K holding the groups in
    psum layout): same result layout as above, with every K unit inside a group's padding set to 0 (a 32-block
    of an fp32 source, a whole packed column of an int16 source; tests/test_layout.py:95-97). An input that
    already has the required layout is returned as it is."""
    _host_assert(is_sfa is not None, 'is_sfa must be set')
    recipe = tuple(recipe)
    _host_assert(len(recipe) == 3, 'recipe must have 3 elements')
    gran_mn, gran_k = int(recipe[0] if is_sfa else recipe[1]), int(recipe[2])
    return _transform_sf(sf, mn, k, gran_mn, gran_k, None, False, None, False, k_psum_layout=psum_layout)


def _transform_sf(sf, mn, k, gran_mn, gran_k, num_groups, disable_ue8m0_cast, psum_layout, tma_aligned,
                  k_psum_layout=None):
    if _check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups):
        if not tma_aligned or mn % 8 == 0 or sf.is_meta:
            return sf
    elif sf.dtype == torch.float32:
        _host_assert(not disable_ue8m0_cast,
                     'Float32 SF must be converted into ue8m0, but disable_ue8m0_cast is set true')
    return _launch_transform_sf(sf, mn, gran_mn=gran_mn, gran_k=gran_k, k=k, psum_layout=psum_layout,
                                tma_aligned=tma_aligned, k_psum_layout=k_psum_layout)


# ------------------------------------------------------------------------------------------------
# GEMM (csrc/apis/gemm.hpp)
# ------------------------------------------------------------------------------------------------
_DTYPES = {torch.float8_e4m3fn: L.E4M3, PACKED_FP4: L.E2M1X2, torch.bfloat16: L.BF16, torch.float32: L.F32}
_BATCH_SPECS = {   # csrc/apis/einsum.hpp:187-215: expression -> permutations of (A, B, D / C) and compiled_dims
    'bhr,hdr->bhd': ((1, 0, 2), None, (1, 0, 2), 'nk'),
    'bhd,hdr->bhr': ((1, 0, 2), (0, 2, 1), (1, 0, 2), 'nk'),
    'bhd,bhr->hdr': ((1, 2, 0), (1, 2, 0), None, 'mn'),
}


def _ptr(t: torch.Tensor) -> int:
    # meta tensors (dry run) have no address; validation only needs something 16-byte aligned
    return 0x1000 if t.is_meta else t.data_ptr()


def _tma_ready_operand(t: torch.Tensor, major: int) -> torch.Tensor:
    """TMA needs a 16-byte aligned base and 16-byte multiples for every stride but the contiguous one. Operands
    that do not satisfy this (K or MN not a multiple of 16, odd views) are copied once into a padded buffer."""
    if t.is_meta:
        return t
    es = t.element_size()
    outer = _outer_stride(t, major)
    lead_ok = all(t.stride(i) * es % 16 == 0 for i in range(t.dim() - 2))
    if t.data_ptr() % 16 == 0 and outer * es % 16 == 0 and lead_ok:
        return t
    rows_axis = -2 if major == L.MAJOR_K else -1
    cols_axis = -1 if major == L.MAJOR_K else -2
    rows, cols = t.size(rows_axis), t.size(cols_axis) * es              # (columns in bytes)
    lead = t.shape[:-2]
    pitch = _align(cols, 16)
    buf = torch.empty((*lead, rows, pitch), dtype=torch.uint8, device=t.device)
    src = (t if major == L.MAJOR_K else t.transpose(-2, -1))
    # one launch per leading index keeps the source strides arbitrary
    flat_src = src.reshape(-1, rows, cols) if src.dim() > 2 and src.is_contiguous() else None
    stream = _stream_ptr(t.device)
    if src.dim() == 2:
        L.check(L.lib().dg_pad_rows_launch(src.data_ptr(), src.stride(0) * es, buf.data_ptr(), pitch, rows, cols, stream))
    else:
        _host_assert(src.dim() == 3, 'operands have at most one leading (group) dimension')
        for g in range(src.size(0)):
            L.check(L.lib().dg_pad_rows_launch(src[g].data_ptr(), src[g].stride(0) * es, buf[g].data_ptr(), pitch, rows, cols, stream))
    del flat_src
    view = buf[..., :cols].view(t.dtype)
    return view if major == L.MAJOR_K else view.transpose(-2, -1)


def _expand_fp4_operand(t: torch.Tensor, major: int) -> torch.Tensor:
    """Packed E2M1 operand (int8, two codes per byte along its contiguous axis) -> the same logical matrix as E4M3
    bytes, exactly, with the same major. For packed operands whose base, strides or extent break the rules of TMA's 4-bit
    unpacking where the kernel has no decoder (a packed A next to an MN-major or k-grouped operand, a k-grouped B)."""
    src = t if major == L.MAJOR_K else t.transpose(-2, -1)              # [..., rows, packed bytes], contiguous rows
    rows, cols = src.size(-2), src.size(-1)
    pitch = _align(2 * cols, 32)
    buf = torch.empty((*src.shape[:-2], rows, pitch), dtype=torch.uint8, device=t.device)
    if not t.is_meta:
        stream = _stream_ptr(t.device)
        _host_assert(src.dim() in (2, 3), 'operands have at most one leading (group) dimension')
        for s_g, b_g in ([(src, buf)] if src.dim() == 2 else [(src[g], buf[g]) for g in range(src.size(0))]):
            L.check(L.lib().dg_expand_fp4_launch(s_g.data_ptr(), s_g.stride(0), b_g.data_ptr(), pitch, rows, cols, stream))
    view = buf[..., :2 * cols].view(torch.float8_e4m3fn)
    return view if major == L.MAJOR_K else view.transpose(-2, -1)


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch for split-K, one per (device, stream); the library leaves it zeroed."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    with _ws_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            ws = torch.zeros(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
            _workspaces[key] = ws
        return ws


def _drop_workspaces(device_index: int) -> None:
    """Forget the cached split-K scratch of a device (its zero invariant can no longer be trusted)."""
    with _ws_lock:
        for key in [k for k in _workspaces if k[0] == device_index]:
            del _workspaces[key]


def _run_gemm(gemm_type, a, b, d, c, epilogue_obj, sfa_in, sfb_in, recipe, recipe_a, recipe_b,
              grouped_layout, compiled_dims, disable_ue8m0_cast, expected_m=None, config=None):
    """csrc/apis/gemm.hpp:60-197 followed by the dispatch of :22-33."""
    major_a, major_b = _major_ab(a), _major_ab(b)
    g = 0
    if gemm_type == L.GEMM_NORMAL:
        m, n, k = _shape_by_spec('mnk', [('mk', a), ('nk', b), ('mn', d)])
    elif gemm_type == L.GEMM_M_GROUPED_PSUM:
        g, m, n, k = _shape_by_spec('gmnk', [('mk', a), ('gnk', b), ('mn', d), ('g', grouped_layout)])
        _host_assert(major_a == L.MAJOR_K, 'A must be K-major for the m-grouped contiguous layout')
    elif gemm_type == L.GEMM_M_GROUPED_MASKED:
        g, m, n, k = _shape_by_spec('gmnk', [('gmk', a), ('gnk', b), ('gmn', d), ('g', grouped_layout)])
        _host_assert(major_a == L.MAJOR_K, 'A must be K-major for the m-grouped masked layout')
    elif gemm_type == L.GEMM_K_GROUPED_PSUM:
        g, m, n, k = _shape_by_spec('gmnk', [('mk', a), ('nk', b), ('gmn', d), ('g', grouped_layout)])
        _host_assert(major_a == L.MAJOR_MN, 'A must be MN-major for the k-grouped layout')
        _host_assert(major_b == L.MAJOR_MN, 'B must be MN-major for the k-grouped layout')
    elif gemm_type == L.GEMM_BATCHED:
        g, m, n, k = _shape_by_spec('bmnk', [('bmk', a), ('bnk', b), ('bmn', d)])
    else:
        raise RuntimeError('Unsupported gemm type')
    _host_assert(d.dim() >= 2 and d.stride(-1) == 1, 'D must be contiguous in its last dimension')
    if grouped_layout is not None:
        _host_assert(grouped_layout.is_contiguous(), 'grouped_layout must be contiguous')
        _host_assert(grouped_layout.dtype == torch.int32, 'grouped_layout must be int32')

    is_cd_same = c is not None and _same_buffer(c, d)
    with_bias = gemm_type == L.GEMM_NORMAL and c is not None and not is_cd_same
    if gemm_type == L.GEMM_NORMAL and c is not None:
        _host_assert(c.dim() == 2 and c.size(0) == (1 if with_bias else m) and c.size(1) == n,
                     "C must match D's pointer and shape for accumulation, or be a separate [1, N] bias")
        _host_assert(c.device == d.device, 'C and D must be on the same device')
    if with_bias:
        _host_assert(c.is_contiguous(), 'Bias must be contiguous')
        _host_assert(not isinstance(epilogue_obj, Alpha), 'alpha and bias cannot be used together')
    if _gemm_early_return(m, n, k, d, c, with_bias):
        return None
    if with_bias:
        epilogue_obj = _Bias(c)

    masked = gemm_type in (L.GEMM_M_GROUPED_MASKED, L.GEMM_BATCHED)    # A, SFA and D carry the group dimension
    bf16 = a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16       # no scale factors (csrc/apis/gemm.hpp:412-433)
    _host_assert(bf16 or (sfa_in is not None and sfb_in is not None), 'Unsupported operand dtypes')
    if bf16:
        sfa = sfb = None
    elif gemm_type == L.GEMM_K_GROUPED_PSUM:
        gran_m, gran_n, gran_k_a, gran_k_b = get_recipe(recipe, recipe_a, recipe_b)
        sfa = _transform_sf(sfa_in, m, k, gran_m, gran_k_a, None, False, None, True, k_psum_layout=grouped_layout)
        sfb = _transform_sf(sfb_in, n, k, gran_n, gran_k_b, None, False, None, True, k_psum_layout=grouped_layout)
    else:
        gran_m, gran_n, gran_k_a, gran_k_b = get_recipe(recipe, recipe_a, recipe_b)
        sfa = _transform_sf(sfa_in, m, k, gran_m, gran_k_a, g if masked else None, disable_ue8m0_cast,
                            grouped_layout if gemm_type == L.GEMM_M_GROUPED_PSUM else None, True)
        sfb = _transform_sf(sfb_in, n, k, gran_n, gran_k_b, g if gemm_type != L.GEMM_NORMAL else None,
                            disable_ue8m0_cast, None, True)

    _host_assert(a.dtype in _DTYPES and b.dtype in _DTYPES, 'Unsupported operand dtypes')
    a_use, b_use = _tma_ready_operand(a, major_a), _tma_ready_operand(b, major_b)

    desc = L.GemmDesc()
    desc.a, desc.b, desc.d = _ptr(a_use), _ptr(b_use), _ptr(d)
    desc.sfa, desc.sfb = (None, None) if bf16 else (_ptr(sfa), _ptr(sfb))
    desc.a_dtype, desc.b_dtype, desc.d_dtype = _DTYPES[a.dtype], _DTYPES[b.dtype], _DTYPES[d.dtype]
    desc.m, desc.n, desc.k = m, n, k
    desc.major_a, desc.major_b = major_a, major_b
    desc.outer_stride_a = _outer_stride(a_use, major_a)
    desc.outer_stride_b = _outer_stride(b_use, major_b)
    desc.outer_stride_d = d.stride(-2)
    desc.group_stride_a = a_use.stride(0) if masked else 0
    desc.group_stride_b = b_use.stride(0) if b_use.dim() == 3 else 0
    desc.group_stride_d = d.stride(0) if masked or gemm_type == L.GEMM_K_GROUPED_PSUM else 0
    if not bf16:
        desc.sfa_stride, desc.sfb_stride = sfa.stride(-1), sfb.stride(-1)
        desc.sfa_group_stride = sfa.stride(0) if sfa.dim() == 3 else 0
        desc.sfb_group_stride = sfb.stride(0) if sfb.dim() == 3 else 0
    desc.gemm_type = gemm_type
    if not bf16 and PACKED_FP4 in (a.dtype, b.dtype):
        # packed operands the kernels cannot read as they are become E4M3 first (exact)
        expand_a, expand_b = C.c_int(0), C.c_int(0)
        L.check(L.lib().dg_fp4_expansion_needed(C.byref(desc), C.byref(expand_a), C.byref(expand_b)))
        if expand_a.value:
            a_use = _expand_fp4_operand(a_use, major_a)
            desc.a, desc.a_dtype = _ptr(a_use), L.E4M3
            desc.outer_stride_a, desc.group_stride_a = _outer_stride(a_use, major_a), (a_use.stride(0) if masked else 0)
        if expand_b.value:
            b_use = _expand_fp4_operand(b_use, major_b)
            desc.b, desc.b_dtype = _ptr(b_use), L.E4M3
            desc.outer_stride_b, desc.group_stride_b = _outer_stride(b_use, major_b), (b_use.stride(0) if b_use.dim() == 3 else 0)
    desc.accumulate = int(c is not None and not with_bias)
    desc.grouped_layout = _ptr(grouped_layout) if grouped_layout is not None else None
    desc.num_groups = g
    # (for the k-grouped layout `expected_m` carries the expected K of one group, csrc/apis/gemm.hpp:35-43)
    desc.expected_m = int(expected_m) if expected_m else (m // g if gemm_type == L.GEMM_M_GROUPED_PSUM and g else m)
    if isinstance(epilogue_obj, Alpha):
        desc.epilogue, desc.alpha = L.EPILOGUE_ALPHA, epilogue_obj.alpha
    elif isinstance(epilogue_obj, _Bias):
        desc.epilogue, desc.bias = L.EPILOGUE_BIAS, _ptr(epilogue_obj.bias)
    elif isinstance(epilogue_obj, BF16StochasticRounding):
        desc.epilogue = L.EPILOGUE_STOCHASTIC_BF16
    elif isinstance(epilogue_obj, FP8Quantization):
        desc.epilogue = L.EPILOGUE_FP8_QUANT
        desc.sfd, desc.sfd_stride = _ptr(epilogue_obj.sfd), epilogue_obj.sfd.stride(1)
    else:
        desc.epilogue = L.EPILOGUE_IDENTITY
    desc.num_sms = 0
    desc.deterministic = int(_global['deterministic'])

    cfg = None
    if config is not None:
        cfg = L.GemmConfig()
        for key, value in config.items():
            if key == 'store_bufs':
                cfg.reserved[1] = int(value)
            elif key == 'k_stagger':
                cfg.reserved[2] = int(value)
            elif key == 'cluster_split':
                cfg.reserved[3] = int(value)
            elif key == 'raster_group':
                cfg.reserved[4] = int(value)
            elif key == 'epilogue_warps':
                cfg.reserved[5] = {4: 1, 8: 2}[int(value)]
            else:
                setattr(cfg, key, int(value))
    cfg_ptr = C.byref(cfg) if cfg is not None else None
    lib = L.lib()
    # The descriptor only holds addresses. Callers that keep it to launch again through the C ABI (the benchmarks do) must
    # not outlive the tensors behind it, some of which were made here (re-laid scales, repacked or expanded operands):
    # they ride along on the returned object.
    desc.keep_alive = (a_use, b_use, sfa, sfb, d, grouped_layout)
    if get_dry_run() or d.is_meta:
        L.check(lib.dg_gemm_dry_run(C.byref(desc), cfg_ptr))
        return desc
    ws_bytes = lib.dg_gemm_workspace_bytes(C.byref(desc), cfg_ptr)
    ws = _workspace(d.device, ws_bytes) if ws_bytes else None
    L.check(lib.dg_gemm_launch(C.byref(desc), cfg_ptr, ws.data_ptr() if ws is not None else None,
                               ws.numel() if ws is not None else 0, _stream_ptr(d.device)))
    # a_use / b_use / sfa / sfb may be temporaries: the caching allocator keeps them valid for work already
    # enqueued on this stream, exactly as the reference relies on (csrc/jit_kernels/gemm_config.hpp:77-78).
    return desc


def _transposed(pair, enable: bool, d0: int, d1: int):
    data, sf = pair
    return (data.transpose(d0, d1), sf.transpose(d0, d1)) if enable else (data, sf)


def _make_dense(trans_a: bool, trans_b: bool, default_dims: str):
    def fn(a, b, d, c=None, recipe=None, recipe_a=None, recipe_b=None, compiled_dims=default_dims,
           disable_ue8m0_cast=False, alpha=None, epilogue=None, *, config=None):
        a_t, sfa = _transposed(a, trans_a, 0, 1)
        b_t, sfb = _transposed(b, trans_b, 0, 1)
        _host_assert(d.dtype in (torch.bfloat16, torch.float32), 'D must be bf16 or fp32')
        _run_gemm(L.GEMM_NORMAL, a_t, b_t, d, c, _resolve_epilogue(epilogue, c, d, alpha), sfa, sfb,
                  recipe, recipe_a, recipe_b, None, compiled_dims, disable_ue8m0_cast, config=config)
    fn.__doc__ = ('D = A @ B^T (+ C) for block-scaled FP8 / FP4 operands; see csrc/apis/gemm.hpp:199-251. '
                  '`config` (keyword only, not in the reference) overrides the tiling heuristic.')
    return fn


fp8_fp4_gemm_nt = _make_dense(False, False, 'nk')
fp8_fp4_gemm_nn = _make_dense(False, True, 'nk')
fp8_fp4_gemm_tn = _make_dense(True, True, 'mn')
fp8_fp4_gemm_tt = _make_dense(True, False, 'mn')
fp8_gemm_nt, fp8_gemm_nn, fp8_gemm_tn, fp8_gemm_tt = fp8_fp4_gemm_nt, fp8_fp4_gemm_nn, fp8_fp4_gemm_tn, fp8_fp4_gemm_tt


def _make_m_grouped_contiguous(trans_b: bool):
    def fn(a, b, d, grouped_layout, recipe=None, recipe_a=None, recipe_b=None, compiled_dims='nk',
           disable_ue8m0_cast=False, use_psum_layout=True, ensure_zero_padding=True,
           expected_m_for_psum_layout=None, epilogue=None, *, config=None):
        a_t, sfa = a
        b_t, sfb = _transposed(b, trans_b, 1, 2)
        _host_assert(a_t.dtype in (torch.float8_e4m3fn, PACKED_FP4) and b_t.dtype in (torch.float8_e4m3fn, PACKED_FP4),
                     'Unsupported operand dtypes')
        _host_assert(d.dtype in (torch.bfloat16, torch.float32), 'D must be bf16 or fp32')
        _host_assert(use_psum_layout is True, 'use_psum_layout must be True')
        _run_gemm(L.GEMM_M_GROUPED_PSUM, a_t, b_t, d, None, _resolve_epilogue(epilogue, None, d), sfa, sfb,
                  recipe, recipe_a, recipe_b, grouped_layout, compiled_dims, disable_ue8m0_cast,
                  expected_m=expected_m_for_psum_layout, config=config)
    fn.__doc__ = 'Per-group D[rows_g] = A[rows_g] @ B[g]^T over the psum layout; see csrc/apis/gemm.hpp:258-321.'
    return fn


m_grouped_fp8_fp4_gemm_nt_contiguous = _make_m_grouped_contiguous(False)
m_grouped_fp8_fp4_gemm_nn_contiguous = _make_m_grouped_contiguous(True)
m_grouped_fp8_gemm_nt_contiguous = m_grouped_fp8_fp4_gemm_nt_contiguous
m_grouped_fp8_gemm_nn_contiguous = m_grouped_fp8_fp4_gemm_nn_contiguous


def m_grouped_fp8_fp4_gemm_nt_masked(a, b, d, masked_m, expected_m, recipe=None, recipe_a=None, recipe_b=None,
                                     compiled_dims='nk', disable_ue8m0_cast=False, epilogue=None, *, config=None):
    """D[g, :masked_m[g]] = A[g, :masked_m[g]] @ B[g]^T. The reference only names this entry point
    (csrc/apis/gemm.hpp:606,630); the signature follows its contiguous sibling. A [G, max_m, K], B [G, N, K],
    D [G, max_m, N], masked_m int32 [G] read on the device; rows at or beyond masked_m[g] are unspecified."""
    a_t, sfa = a
    b_t, sfb = b
    _host_assert(d.dtype in (torch.bfloat16, torch.float32), 'D must be bf16 or fp32')
    _run_gemm(L.GEMM_M_GROUPED_MASKED, a_t, b_t, d, None, _resolve_epilogue(epilogue, None, d), sfa, sfb,
              recipe, recipe_a, recipe_b, masked_m, compiled_dims, disable_ue8m0_cast,
              expected_m=expected_m, config=config)


m_grouped_fp8_gemm_nt_masked = m_grouped_fp8_fp4_gemm_nt_masked


def k_grouped_fp8_gemm_tn_contiguous(a, b, d, ks_cpu, grouped_layout, c=None, recipe=(1, 1, 32), compiled_dims='mn',
                                     use_psum_layout=True, epilogue=None, *, config=None):
    """csrc/apis/gemm.hpp:325-384. Weight-gradient GEMM of an MoE layer: a = (A [K, M], sfA [ceil(K/32), M]),
    b = (B [K, N], sfB), K holding G groups in psum layout (`grouped_layout[g]` = end of group g, each group
    starting at the previous end rounded up to the 256 alignment, operand data zero in the padding);
    D[g] = A[group g]^T @ B[group g] (+ C[g] when `c` is D itself), D[g] = 0 (or kept) for an empty group."""
    (a_data, sfa), (b_data, sfb) = _transposed(a, True, 0, 1), _transposed(b, True, 0, 1)
    _host_assert(a_data.dtype in (torch.float8_e4m3fn, PACKED_FP4) and b_data.dtype in (torch.float8_e4m3fn, PACKED_FP4),
                 'Unsupported operand dtypes')
    _host_assert(d.dtype in (torch.bfloat16, torch.float32))
    _host_assert(use_psum_layout is True)
    k, g = a_data.size(-1), grouped_layout.numel()
    expected_k = max(1, sum(ks_cpu) // len(ks_cpu)) if ks_cpu else (k // g if g else k)
    _run_gemm(L.GEMM_K_GROUPED_PSUM, a_data, b_data, d, c, _resolve_epilogue(epilogue, c, d), sfa, sfb,
              tuple(recipe), None, None, grouped_layout, compiled_dims, False, expected_m=expected_k, config=config)


def k_grouped_fp8_gemm_nt_contiguous(a, b, d, ks_cpu, grouped_layout, c=None, recipe=(1, 1, 32), compiled_dims='mn',
                                     use_psum_layout=True, epilogue=None, *, config=None):
    """csrc/apis/gemm.hpp:386-410. Deprecated: takes A [M, K] and B [N, K] and forwards their transposes."""
    warnings.warn('Calling k_grouped_fp8_gemm_nt_contiguous is deprecated, please transpose a, b into [k, m] and [k, n] '
                  'shape and call `k_grouped_fp8_gemm_tn_contiguous` instead', DeprecationWarning, stacklevel=2)
    k_grouped_fp8_gemm_tn_contiguous(_transposed(a, True, 0, 1), _transposed(b, True, 0, 1), d, ks_cpu, grouped_layout,
                                     c, recipe, compiled_dims, use_psum_layout, epilogue, config=config)


# ------------------------------------------------------------------------------------------------
# BF16 GEMM family (csrc/apis/gemm.hpp:412-560): same kernels with kind::f16 MMAs and no scale factors
# ------------------------------------------------------------------------------------------------
def _make_bf16_dense(trans_a: bool, trans_b: bool, default_dims: str):
    def fn(a, b, d, c=None, compiled_dims=default_dims, alpha=None, epilogue=None, *, config=None):
        a_t = a.transpose(0, 1) if trans_a else a
        b_t = b.transpose(0, 1) if trans_b else b
        _host_assert(a_t.dtype == torch.bfloat16 and b_t.dtype == torch.bfloat16, 'A and B must be bfloat16')
        _host_assert(d.dtype in (torch.bfloat16, torch.float32), 'D must be bf16 or fp32')
        _run_gemm(L.GEMM_NORMAL, a_t, b_t, d, c, _resolve_epilogue(epilogue, c, d, alpha), None, None,
                  None, None, None, None, compiled_dims, False, config=config)
    fn.__doc__ = 'D = A @ B^T (+ C) for BF16 operands; see csrc/apis/gemm.hpp:412-440.'
    return fn


bf16_gemm_nt = _make_bf16_dense(False, False, 'nk')
bf16_gemm_nn = _make_bf16_dense(False, True, 'nk')
bf16_gemm_tn = _make_bf16_dense(True, True, 'mn')
bf16_gemm_tt = _make_bf16_dense(True, False, 'mn')


def _make_m_grouped_bf16_contiguous(trans_b: bool):
    def fn(a, b, d, grouped_layout, compiled_dims='nk', use_psum_layout=True, ensure_zero_padding=True,
           expected_m_for_psum_layout=None, epilogue=None, *, config=None):
        b_t = b.transpose(1, 2) if trans_b else b
        _host_assert(a.dtype == torch.bfloat16 and b_t.dtype == torch.bfloat16, 'A and B must be bfloat16')
        _host_assert(d.dtype in (torch.bfloat16, torch.float32), 'D must be bf16 or fp32')
        _host_assert(use_psum_layout is True, 'use_psum_layout must be True')
        _run_gemm(L.GEMM_M_GROUPED_PSUM, a, b_t, d, None, _resolve_epilogue(epilogue, None, d), None, None,
                  None, None, None, grouped_layout, compiled_dims, True, expected_m=expected_m_for_psum_layout, config=config)
    fn.__doc__ = 'Per-group D[rows_g] = A[rows_g] @ B[g]^T for BF16 operands; see csrc/apis/gemm.hpp:442-475.'
    return fn


m_grouped_bf16_gemm_nt_contiguous = _make_m_grouped_bf16_contiguous(False)
m_grouped_bf16_gemm_nn_contiguous = _make_m_grouped_bf16_contiguous(True)


def k_grouped_bf16_gemm_tn_contiguous(a, b, d, ks_cpu, grouped_layout, c=None, compiled_dims='mn', use_psum_layout=True,
                                      epilogue=None, *, config=None):
    """csrc/apis/gemm.hpp:477-514. A [K, M], B [K, N] BF16 with K in psum layout; D[g] = A[group g]^T @ B[group g] (+ C[g])."""
    a_t, b_t = a.transpose(0, 1), b.transpose(0, 1)
    _host_assert(a_t.dtype == torch.bfloat16 and b_t.dtype == torch.bfloat16, 'A and B must be bfloat16')
    _host_assert(d.dtype in (torch.bfloat16, torch.float32))
    _host_assert(use_psum_layout is True)
    k, g = a_t.size(-1), grouped_layout.numel()
    expected_k = max(1, sum(ks_cpu) // len(ks_cpu)) if ks_cpu else (k // g if g else k)
    _run_gemm(L.GEMM_K_GROUPED_PSUM, a_t, b_t, d, c, _resolve_epilogue(epilogue, c, d), None, None,
              None, None, None, grouped_layout, compiled_dims, False, expected_m=expected_k, config=config)


def fp8_bmm(a, b, d, c=None, recipe=(1, 1, 32), compiled_dims='nk', epilogue=None, *, config=None):
    """Batched D[i] = A[i] @ B[i]^T (+ C[i]); csrc/apis/einsum.hpp:37-71. A [B,M,K], B [B,N,K] (E4M3, either major, any
    batch stride), D [B,M,N] bf16 / fp32, or a (D, sfd) pair for E4M3 output with UE8M0 scales per 1x32."""
    a_t, sfa = a
    b_t, sfb = b
    d_t, sfd = d if isinstance(d, (tuple, list)) else (d, None)
    _host_assert(a_t.dtype == torch.float8_e4m3fn and b_t.dtype == torch.float8_e4m3fn, 'fp8_bmm operands must be E4M3')
    _host_assert(d_t.dim() == 3 and d_t.stride(-1) == 1, 'D must be [B, M, N] and contiguous in N')
    if a_t.size(0) == 0:
        return
    resolved = _resolve_epilogue(epilogue, c, d_t, None, sfd)
    if isinstance(resolved, FP8Quantization) and 0 in (a_t.size(-2), b_t.size(-2), a_t.size(-1)):
        if not d_t.is_meta:
            d_t.zero_()
            resolved.sfd.zero_()
        return
    _run_gemm(L.GEMM_BATCHED, a_t, b_t, d_t, c, resolved, sfa, sfb, recipe, None, None, None, compiled_dims, False,
              config=config)


def fp8_einsum(expr, a, b, d, c=None, recipe=(1, 1, 32), epilogue=None, *, config=None):
    """FP8 einsum over the reference's three contraction strings (csrc/apis/einsum.hpp:161-216): operands and their
    scale factors are permuted (views only) into a batched GEMM."""
    _host_assert(expr in _BATCH_SPECS, 'Unsupported einsum expression')
    pa, pb, pd, dims = _BATCH_SPECS[expr]

    def perm(t, p):
        return t if p is None or t is None else t.permute(p)
    is_pair = isinstance(d, (tuple, list))
    _host_assert(not is_pair or expr == 'bhr,hdr->bhd', 'only the forward expression accepts a (D, SFD) pair')
    d_arg = (perm(d[0], pd), d[1]) if is_pair else perm(d, pd)
    fp8_bmm((perm(a[0], pa), perm(a[1], pa)), (perm(b[0], pb), perm(b[1], pb)), d_arg, perm(c, pd), recipe, dims,
            epilogue, config=config)


def bf16_bmm(a, b, d, c=None, compiled_dims='nk', epilogue=None, *, config=None):
    """Batched D[i] = A[i] @ B[i]^T (+ C[i]) for BF16 operands; csrc/apis/einsum.hpp:73-100. A [B,M,K], B [B,N,K] (either
    major, any batch stride), D [B,M,N] bf16 / fp32."""
    _host_assert(a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, 'A and B must be bfloat16')
    _host_assert(d.dtype in (torch.bfloat16, torch.float32), 'D must be bf16 or fp32')
    _host_assert(d.dim() == 3 and d.stride(-1) == 1, 'D must be [B, M, N] and contiguous in N')
    if a.size(0) == 0:
        return
    _run_gemm(L.GEMM_BATCHED, a, b, d, c, _resolve_epilogue(epilogue, c, d), None, None, None, None, None, None,
              compiled_dims, False, config=config)


def einsum(expr, a, b, d, c=None, use_cublaslt=False, epilogue=None, *, config=None):
    """BF16 einsum over the reference's three contraction strings (csrc/apis/einsum.hpp:102-145): the operands are
    permuted (views only) into a batched BF16 GEMM."""
    _host_assert(not use_cublaslt, 'einsum: use_cublaslt is not implemented (csrc/apis/einsum.hpp:128-130)')
    _host_assert(expr in _BATCH_SPECS, 'Unsupported einsum expression')
    pa, pb, pd, dims = _BATCH_SPECS[expr]

    def perm(t, p):
        return t if p is None or t is None else t.permute(p)
    bf16_bmm(perm(a, pa), perm(b, pb), perm(d, pd), perm(c, pd), dims, epilogue, config=config)


def device_status() -> int:
    """0, or the code of the first problem a kernel recorded since the last call: 101..107 = a bounded wait inside a
    GEMM kernel gave up (its output is incomplete), 201 = a scale-factor transform met an FP32 scale that is negative
    or not a power of two (the reference's device assert, transform_sf.hpp:13-21). Synchronises the device; the
    record is cleared. After a wait that gave up the split-K scratch may hold partial sums, so it is dropped and
    the next split-K launch starts from a fresh zeroed buffer."""
    out = C.c_int32(0)
    L.check(L.lib().dg_device_status(C.byref(out)))
    code = out.value
    device = torch.cuda.current_device()
    if code != 0:
        _drop_workspaces(device)
    flag = _sf_flags.get(device)
    if flag is not None and int(flag.item()) != 0:
        flag.zero_()
        code = code or STATUS_INVALID_SCALE_FACTOR
    if _C is not None:
        # (the compiled host layer keeps a flag and a scratch cache of its own)
        if out.value != 0:
            _C._drop_workspaces(device)
        c_code = _C.device_status()
        code = code or c_code
    return code
