"""Host-side behaviour that needs no GPU: the C ABI loads and exports what include/dg_b200.h declares,
argument validation, shape / major inference, the tiling heuristic and the dry-run path on meta tensors."""

import ctypes
import os
import re

import pytest
import torch

import deep_gemm
from deep_gemm import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _meta_pair(rows, k, gran=(1, 32), dtype=torch.float8_e4m3fn, mn_major=False):
    data = torch.empty((k, rows) if mn_major else (rows, k), dtype=dtype, device='meta')
    if mn_major:
        data = data.transpose(0, 1)
    sf = torch.empty((rows + gran[0] - 1) // gran[0], (k + gran[1] - 1) // gran[1], dtype=torch.float32, device='meta')
    return data, sf


@pytest.fixture(autouse=True)
def dry_run():
    deep_gemm.set_dry_run(True)
    yield
    deep_gemm.set_dry_run(False)


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, 'include', 'dg_b200.h')).read()
    declared = set(re.findall(r'\b(dg_[a-z0-9_]+)\s*\(', header))
    assert declared, 'no declarations found'
    handle = ctypes.CDLL(L.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(handle, name), f'{name} is declared but not exported'
    assert declared == set(L.EXPORTED_SYMBOLS)
    assert L.lib().dg_abi_version() == L.ABI_VERSION == 3


def test_struct_sizes_match_the_header():
    # 5 pointers, 8 x 4-byte, 10 x 8-byte, 2 x 4, pointer, 2 x 4, 2 x 4, pointer, 4 (+4 padding), pointer, 8, 2 x 4
    assert ctypes.sizeof(L.GemmDesc) == 224
    assert ctypes.sizeof(L.GemmConfig) == 64


def test_public_names_of_the_hot_path_exist():
    for name in ('fp8_gemm_nt', 'fp8_gemm_nn', 'fp8_gemm_tn', 'fp8_gemm_tt',
                 'fp8_fp4_gemm_nt', 'fp8_fp4_gemm_nn', 'fp8_fp4_gemm_tn', 'fp8_fp4_gemm_tt',
                 'm_grouped_fp8_gemm_nt_contiguous', 'm_grouped_fp8_gemm_nn_contiguous',
                 'm_grouped_fp8_fp4_gemm_nt_contiguous', 'm_grouped_fp8_fp4_gemm_nn_contiguous',
                 'm_grouped_fp8_gemm_nt_masked', 'm_grouped_fp8_fp4_gemm_nt_masked',
                 'k_grouped_fp8_gemm_tn_contiguous', 'k_grouped_fp8_gemm_nt_contiguous', 'k_grouped_bf16_gemm_tn_contiguous',
                 'bf16_gemm_nt', 'bf16_gemm_nn', 'bf16_gemm_tn', 'bf16_gemm_tt', 'm_grouped_bf16_gemm_nt_contiguous',
                 'm_grouped_bf16_gemm_nn_contiguous', 'fp8_bmm', 'fp8_einsum', 'bf16_bmm', 'einsum',
                 'transform_k_grouped_sf_into_required_layout', 'get_recipe', 'npu_sleep',
                 'transform_sf_into_required_layout', 'get_num_sms', 'set_num_sms',
                 'get_mk_alignment_for_contiguous_layout', 'use_deterministic_algorithms', 'set_dry_run'):
        assert callable(getattr(deep_gemm, name)), name
    assert deep_gemm.fp8_gemm_nt is deep_gemm.fp8_fp4_gemm_nt
    assert deep_gemm.get_mk_alignment_for_contiguous_layout() == 256
    deep_gemm.epilogue.Identity(), deep_gemm.epilogue.Alpha(0.5)


def test_num_sms_knob_round_trips():
    deep_gemm.set_num_sms(132)
    assert deep_gemm.get_num_sms() == 132
    deep_gemm.set_num_sms(0)
    assert deep_gemm.get_num_sms() >= 1


def test_dry_run_on_meta_tensors_all_spellings():
    m, n, k = 256, 384, 512
    d = torch.empty(m, n, dtype=torch.bfloat16, device='meta')
    for name, ta, tb in (('nt', False, False), ('nn', False, True), ('tn', True, True), ('tt', True, False)):
        a, sfa = _meta_pair(m, k, mn_major=ta)
        b, sfb = _meta_pair(n, k, mn_major=tb)
        a_arg = (a.transpose(0, 1), sfa.transpose(0, 1)) if ta else (a, sfa)
        b_arg = (b.transpose(0, 1), sfb.transpose(0, 1)) if tb else (b, sfb)
        getattr(deep_gemm, f'fp8_gemm_{name}')(a_arg, b_arg, d)


def test_alpha_and_bias_are_exclusive():
    a, b = _meta_pair(128, 256), _meta_pair(64, 256)
    d = torch.empty(128, 64, dtype=torch.bfloat16, device='meta')
    bias = torch.empty(1, 64, dtype=torch.bfloat16, device='meta')
    with pytest.raises(RuntimeError, match='alpha and bias cannot be used together'):
        deep_gemm.fp8_gemm_nt(a, b, d, c=bias, alpha=0.5)
    deep_gemm.fp8_gemm_nt(a, b, d, c=bias)
    deep_gemm.fp8_gemm_nt(a, b, d, alpha=0.5)
    with pytest.raises(RuntimeError, match='exclusive'):
        deep_gemm.fp8_gemm_nt(a, b, d, alpha=0.5, epilogue=deep_gemm.epilogue.Identity())


def test_shape_conflicts_and_bad_c_are_reported():
    a, b = _meta_pair(128, 256), _meta_pair(64, 128)
    d = torch.empty(128, 64, dtype=torch.bfloat16, device='meta')
    with pytest.raises(RuntimeError, match="Conflicting shape dimension 'k'"):
        deep_gemm.fp8_gemm_nt(a, b, d)
    b = _meta_pair(64, 256)
    with pytest.raises(RuntimeError, match="C must match D's pointer and shape"):
        deep_gemm.fp8_gemm_nt(a, b, d, c=torch.empty(2, 64, dtype=torch.bfloat16, device='meta'))
    with pytest.raises(RuntimeError, match='bf16 or fp32'):
        deep_gemm.fp8_gemm_nt(a, b, torch.empty(128, 64, dtype=torch.float16, device='meta'))


def test_recipe_rules():
    assert deep_gemm.get_recipe(None, None, None) == (1, 1, 32, 32)
    assert deep_gemm.get_recipe((1, 128, 128), None, None) == (1, 128, 128, 128)
    assert deep_gemm.get_recipe(None, (1, 128), (1, 32)) == (1, 1, 128, 32)
    with pytest.raises(RuntimeError, match='mutually exclusive'):
        deep_gemm.get_recipe((1, 1, 32), (1, 32), None)


def test_sf_fast_path_returns_the_same_tensor():
    mn, k = 64, 256
    sf = torch.empty(k // 64, mn, dtype=torch.int16, device='meta').transpose(0, 1)
    assert deep_gemm.transform_sf_into_required_layout(sf, mn, k, (1, 1, 32), is_sfa=True) is sf
    sf32 = torch.empty(mn, k // 32, dtype=torch.float32, device='meta')
    out = deep_gemm.transform_sf_into_required_layout(sf32, mn, k, (1, 1, 32), is_sfa=True)
    assert out.dtype == torch.int16 and tuple(out.shape) == (mn, k // 64)
    assert out.stride(-2) == 1 and out.stride(-1) == mn
    with pytest.raises(RuntimeError, match='disable_ue8m0_cast'):
        deep_gemm.transform_sf_into_required_layout(sf32, mn, k, (1, 1, 32), is_sfa=True, disable_ue8m0_cast=True)
    with pytest.raises(RuntimeError, match='is_sfa'):
        deep_gemm.transform_sf_into_required_layout(sf32, mn, k, (1, 1, 32))


def _desc(m, n, k, d_dtype=L.BF16, **kw):
    d = L.GemmDesc()
    d.a = d.b = d.d = d.sfa = d.sfb = 0x1000
    d.a_dtype, d.b_dtype, d.d_dtype = L.E4M3, L.E4M3, d_dtype
    d.m, d.n, d.k = m, n, k
    d.outer_stride_a = d.outer_stride_b = k
    d.outer_stride_d = n
    d.sfa_stride, d.sfb_stride = (m + 7) // 8 * 8, (n + 7) // 8 * 8
    for key, value in kw.items():
        setattr(d, key, value)
    return d


def test_heuristic_respects_hardware_limits():
    lib = L.lib()
    for m in (1, 64, 128, 4096):
        for n, k in ((2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)):
            desc, cfg = _desc(m, n, k), L.GemmConfig()
            assert lib.dg_select_config(ctypes.byref(desc), ctypes.byref(cfg)) == 0, L.last_error()
            c = cfg.as_dict()
            assert c['block_m'] == 128 * c['cta_group'] and c['block_k'] == 128
            # up to 256 columns in steps of 32, or a wide tile of two halves (a CTA pair with many rows only)
            assert (32 <= c['block_n'] <= 256 and c['block_n'] % 32 == 0) or \
                   (c['block_n'] in (320, 384, 448) and c['cta_group'] == 2 and m > 128 and c['accum_stages'] == 1)
            assert c['smem_bytes'] <= 227 * 1024 and 1 <= c['num_stages'] <= 12
            assert c['tmem_cols'] in (32, 64, 128, 256, 512)
            slabs = (c['block_n'] + 127) // 128 if c['block_n'] <= 256 else 2 * ((c['block_n'] // 2 + 127) // 128)
            assert c['accum_stages'] * c['block_n'] + 4 + 4 * slabs <= c['tmem_cols']
            assert c['split_k'] >= 1 and (c['split_k'] == 1 or m <= 1024)
            ws = lib.dg_gemm_workspace_bytes(ctypes.byref(desc), ctypes.byref(cfg))
            if c['split_k'] > 1 and c['cluster_split']:
                # the splits of a tile form a cluster (at most 8 CTAs) and need no workspace; the grid is not persistent
                assert c['split_k'] <= 8 and c['cta_group'] == 1 and c['num_ctas'] % c['split_k'] == 0 and ws == 0
                assert c['num_stages'] >= 3
            else:
                assert 1 <= c['num_ctas'] <= 148
                assert (ws >= m * n * 4) if c['split_k'] > 1 else ws == 0


def test_c_abi_validation_messages():
    lib = L.lib()
    cfg = L.GemmConfig()
    bad = _desc(128, 128, 128, a_dtype=L.E2M1X2, b_dtype=L.E4M3)
    assert lib.dg_select_config(ctypes.byref(bad), ctypes.byref(cfg)) == L.DG_ERR_INVALID
    assert 'Unsupported operand dtypes' in L.last_error()
    bad = _desc(128, 128, 128, epilogue=L.EPILOGUE_BIAS)
    assert lib.dg_gemm_dry_run(ctypes.byref(bad), None) == L.DG_ERR_INVALID
    bad = _desc(128, 128, 100)
    bad.outer_stride_a = 100
    assert lib.dg_gemm_dry_run(ctypes.byref(bad), None) == L.DG_ERR_UNSUPPORTED
    assert '16 bytes' in L.last_error()
    grouped = _desc(1000, 128, 128, gemm_type=L.GEMM_M_GROUPED_PSUM, num_groups=2, grouped_layout=0x1000)
    assert lib.dg_gemm_dry_run(ctypes.byref(grouped), None) == L.DG_ERR_INVALID
    assert '256' in L.last_error()
    forced = L.GemmConfig()
    forced.block_n, forced.cta_group, forced.split_k = 100, 1, 1
    assert lib.dg_gemm_dry_run(ctypes.byref(_desc(128, 256, 256)), ctypes.byref(forced)) == L.DG_ERR_INVALID
    assert 'block_n' in L.last_error()


def test_wide_tile_with_split_k_is_rejected():
    """A tile wider than 256 columns is walked by tile index alone; with K splits the walk would mix the two up."""
    lib = L.lib()
    forced = L.GemmConfig()
    forced.block_n, forced.cta_group, forced.split_k = 448, 2, 2
    assert lib.dg_gemm_dry_run(ctypes.byref(_desc(4096, 4096, 4096)), ctypes.byref(forced)) == L.DG_ERR_INVALID
    assert 'cannot be combined with split_k' in L.last_error()
    forced.split_k = 1
    assert lib.dg_gemm_dry_run(ctypes.byref(_desc(4096, 4096, 4096)), ctypes.byref(forced)) == 0, L.last_error()


def test_deterministic_flag_keeps_away_from_arrival_order_reductions():
    """use_deterministic_algorithms (csrc/apis/runtime.hpp:56-62): split-K through the FP32 workspace adds partial
    sums in arrival order, so the heuristic must not pick it and an explicit request for it is an error; the
    cluster reduction (rank order) stays available."""
    lib = L.lib()
    for m, n, k, major_b in ((128, 512, 16384, L.MAJOR_MN), (64, 2112, 7168, L.MAJOR_K), (128, 256, 32768, L.MAJOR_MN)):
        desc = _desc(m, n, k, major_b=major_b, deterministic=1)
        if major_b == L.MAJOR_MN:
            desc.outer_stride_b = n
        cfg = L.GemmConfig()
        assert lib.dg_select_config(ctypes.byref(desc), ctypes.byref(cfg)) == 0, L.last_error()
        c = cfg.as_dict()
        assert c['split_k'] == 1 or c['cluster_split'] == 1
        assert lib.dg_gemm_workspace_bytes(ctypes.byref(desc), ctypes.byref(cfg)) == 0
    forced = L.GemmConfig()
    forced.block_n, forced.cta_group, forced.split_k = 128, 1, 4
    desc = _desc(128, 512, 4096, deterministic=1)
    assert lib.dg_gemm_dry_run(ctypes.byref(desc), ctypes.byref(forced)) == L.DG_ERR_INVALID
    assert 'deterministic' in L.last_error()
    forced.reserved[3] = 1
    assert lib.dg_gemm_dry_run(ctypes.byref(desc), ctypes.byref(forced)) == 0, L.last_error()
    # the Python knob reaches the descriptor
    deep_gemm.use_deterministic_algorithms(True)
    try:
        a, b = _meta_pair(128, 4096), _meta_pair(512, 4096)
        d = torch.empty(128, 512, dtype=torch.bfloat16, device='meta')
        with pytest.raises(RuntimeError, match='deterministic'):
            deep_gemm.fp8_gemm_nt(a, b, d, config={'block_n': 128, 'cta_group': 1, 'split_k': 4})
        deep_gemm.fp8_gemm_nt(a, b, d)
    finally:
        deep_gemm.use_deterministic_algorithms(False)
    assert deep_gemm.get_deterministic_algorithms() is False


def test_status_report_drops_the_split_k_scratch():
    """After a kernel reported a wait that gave up, the cached split-K scratch of that device may hold partial sums:
    the host layer must forget it so that the next split-K launch gets a fresh zeroed buffer."""
    from deep_gemm import _api
    _api._workspaces[(0, 123)] = object()
    _api._workspaces[(0, 456)] = object()
    _api._workspaces[(1, 123)] = object()
    try:
        _api._drop_workspaces(0)
        assert list(_api._workspaces) == [(1, 123)]
    finally:
        _api._workspaces.clear()


def test_npu_sleep_and_init_exist_and_dry_run_is_a_no_op():
    deep_gemm.init('', '')
    deep_gemm.npu_sleep(0)                      # dry run (autouse fixture): nothing is launched
    deep_gemm.npu_sleep(1000, marker=1)
    lib = L.lib()
    assert lib.dg_sleep_launch(-1, 0, 148, None) == L.DG_ERR_INVALID
    assert lib.dg_sleep_launch(5 * 10 ** 9, 0, 148, None) == L.DG_ERR_INVALID
    assert 'sleep_cycles' in L.last_error()


def test_compiled_host_layer_is_in_use_and_agrees_with_the_python_one():
    """When the `_C` extension is built the public entry points are its functions; the Python host layer stays
    importable and must accept and reject the same calls with the same messages (both end in the same C ABI)."""
    from deep_gemm import _api
    if _api._C is None:
        pytest.skip('the _C extension has not been built')
    assert deep_gemm.BACKEND == '_C'
    assert deep_gemm.fp8_gemm_nt is _api._C.fp8_fp4_gemm_nt
    assert deep_gemm.epilogue.Alpha is _api._C.epilogue.Alpha
    a, b = _meta_pair(128, 256), _meta_pair(64, 256)
    d = torch.empty(128, 64, dtype=torch.bfloat16, device='meta')
    bias = torch.empty(1, 64, dtype=torch.bfloat16, device='meta')
    cases = [
        (dict(c=bias, alpha=0.5), 'alpha and bias cannot be used together'),
        (dict(c=torch.empty(2, 64, dtype=torch.bfloat16, device='meta')), "C must match D's pointer and shape"),
        (dict(recipe=(1, 1, 32), recipe_a=(1, 32)), 'mutually exclusive'),
        (dict(config={'block_n': 100}), 'block_n'),
        (dict(), None), (dict(c=bias), None), (dict(alpha=2.0), None), (dict(config={'block_n': 64, 'cta_group': 1}), None),
    ]
    for kwargs, message in cases:
        for fn in (_api._C.fp8_gemm_nt, _api.fp8_gemm_nt):
            if message is None:
                fn(a, b, d, **kwargs)
            else:
                with pytest.raises(RuntimeError, match=message):
                    fn(a, b, d, **kwargs)
    with pytest.raises(RuntimeError, match="Conflicting shape dimension 'k'"):
        _api._C.fp8_gemm_nt(a, _meta_pair(64, 128), d)
    # the knobs set through the package reach both layers
    deep_gemm.set_dry_run(False)
    assert _api._C.get_dry_run() is False and _api.get_dry_run() is False
    deep_gemm.set_dry_run(True)
    assert _api._C.get_dry_run() is True and _api.get_dry_run() is True


def test_packed_fp4_operand_kinds_and_majors_on_meta_tensors():
    """FP4 x FP4 with MN-major operands and the k-grouped layout with FP8 x FP4 / FP4 x FP4 operands are accepted by both
    host layers (csrc/apis/gemm.hpp:325-384 names the three operand kinds); a packed A next to an E4M3 B is not."""
    from deep_gemm import _api
    layers = [_api] + ([_api._C] if _api._C is not None else [])
    m, n, k = 256, 384, 1024

    def packed(rows, kk, mn_major):         # logical [rows, kk] view of packed storage
        t = torch.empty((kk, rows // 2) if mn_major else (rows, kk // 2), dtype=torch.int8, device='meta')
        return t.transpose(0, 1) if mn_major else t

    def scales(rows, kk, mn_major):
        t = torch.empty((kk // 32, rows) if mn_major else (rows, kk // 32), dtype=torch.float32, device='meta')
        return t.transpose(0, 1) if mn_major else t

    d = torch.empty(m, n, dtype=torch.bfloat16, device='meta')
    for layer in layers:
        for trans in ('nt', 'nn', 'tn', 'tt'):
            a = (packed(m, k, trans[0] == 't'), scales(m, k, trans[0] == 't'))
            b = (packed(n, k, trans[1] == 'n'), scales(n, k, trans[1] == 'n'))
            a_arg = tuple(x.transpose(0, 1) for x in a) if trans[0] == 't' else a
            b_arg = tuple(x.transpose(0, 1) for x in b) if trans[1] == 'n' else b
            getattr(layer, f'fp8_fp4_gemm_{trans}')(a_arg, b_arg, d, recipe_a=(1, 32), recipe_b=(1, 32))
        layout = torch.empty(2, dtype=torch.int32, device='meta')
        dk = torch.empty(2, m, n, dtype=torch.float32, device='meta')
        sfa, sfb = torch.empty(k // 32, m, device='meta'), torch.empty(k // 32, n, device='meta')
        a8 = torch.empty(k, m, dtype=torch.float8_e4m3fn, device='meta')
        b8 = torch.empty(k, n, dtype=torch.float8_e4m3fn, device='meta')
        a4 = torch.empty(k, m // 2, dtype=torch.int8, device='meta')
        b4 = torch.empty(k, n // 2, dtype=torch.int8, device='meta')
        layer.k_grouped_fp8_gemm_tn_contiguous((a8, sfa), (b4, sfb), dk, [512, 512], layout, recipe=(1, 1, 32))
        layer.k_grouped_fp8_gemm_tn_contiguous((a4, sfa), (b4, sfb), dk, None, layout, recipe=(1, 1, 32))
        with pytest.raises(RuntimeError, match='Unsupported operand dtypes'):
            layer.k_grouped_fp8_gemm_tn_contiguous((a4, sfa), (b8, sfb), dk, None, layout, recipe=(1, 1, 32))


def test_fp4_expansion_rule_of_the_c_abi():
    """dg_fp4_expansion_needed: a packed A outside the K-major x K-major kernel, or a k-grouped packed B, must have a
    32-byte aligned base, 32-byte strides and a contiguous extent that is a multiple of 128 elements."""
    lib = L.lib()
    d = L.GemmDesc()
    d.a = d.b = d.d = d.sfa = d.sfb = 0x1000
    d.a_dtype, d.b_dtype, d.d_dtype = L.E2M1X2, L.E2M1X2, L.BF16
    d.m, d.n, d.k = 256, 384, 1024
    d.major_a, d.major_b = L.MAJOR_MN, L.MAJOR_MN
    d.outer_stride_a, d.outer_stride_b, d.outer_stride_d = 128, 192, 384        # bytes of packed storage per K row
    ea, eb = ctypes.c_int(-1), ctypes.c_int(-1)
    assert lib.dg_fp4_expansion_needed(ctypes.byref(d), ctypes.byref(ea), ctypes.byref(eb)) == 0
    assert (ea.value, eb.value) == (0, 0)
    d.m, d.outer_stride_a = 130, 65                                           # neither a 128-element extent nor a 32-byte stride
    lib.dg_fp4_expansion_needed(ctypes.byref(d), ctypes.byref(ea), ctypes.byref(eb))
    assert (ea.value, eb.value) == (1, 0)                                      # (B falls back to the in-kernel decoder)
    d.m, d.outer_stride_a, d.n, d.outer_stride_b = 256, 128, 200, 100
    d.gemm_type, d.num_groups, d.grouped_layout = L.GEMM_K_GROUPED_PSUM, 2, 0x1000
    lib.dg_fp4_expansion_needed(ctypes.byref(d), ctypes.byref(ea), ctypes.byref(eb))
    assert (ea.value, eb.value) == (1, 1)                                      # (an expanded B is E4M3: the packed A follows it)
    d.a_dtype = L.E4M3
    lib.dg_fp4_expansion_needed(ctypes.byref(d), ctypes.byref(ea), ctypes.byref(eb))
    assert (ea.value, eb.value) == (0, 1)
    d.a_dtype = L.E2M1X2
    d.major_a = d.major_b = L.MAJOR_K                                          # the kind::mxf4 kernel reads packed operands itself
    d.gemm_type, d.n, d.outer_stride_a, d.outer_stride_b = L.GEMM_NORMAL, 200, 515, 515
    lib.dg_fp4_expansion_needed(ctypes.byref(d), ctypes.byref(ea), ctypes.byref(eb))
    assert (ea.value, eb.value) == (0, 0)


def test_the_shipped_package_never_refers_to_the_oracle():
    """The oracle is test infrastructure: no module of the package (its benchmark helpers included) imports it; the
    benchmark hands the checkers in from outside."""
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'deepgemm-ascend_b200')
    offenders = []
    for folder, _, files in os.walk(root):
        for name in files:
            if name.endswith(('.py', '.cu', '.cuh', '.cpp', '.hpp', '.h')):
                text = open(os.path.join(folder, name), encoding='utf-8').read()
                if re.search(r'^\s*(import|from)\s+oracle\b', text, re.M) or 'oracle/' in text:
                    offenders.append(os.path.join(folder, name))
    assert offenders == []


def _run_bench(*argv):
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, os.path.join(root, 'bench.py'), *argv], capture_output=True, text=True, timeout=600)
    return proc, (json.loads(proc.stdout.strip().splitlines()[-1]) if proc.stdout.strip() else None)


def test_reference_arm_of_the_benchmark_follows_the_multi_gpu_workload():
    """`bench.py --impl reference --gpus 2` times the oracle on a sample of the grouped problem the two-GPU arm shards
    and prints that arm's `config` object, the contract's keys and no GPU launches."""
    from deep_gemm.testing import moe_bench
    proc, line = _run_bench('--impl', 'reference', '--gpus', '2', '--steps', '1', '--warmup', '0')
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert line['impl'] == 'reference' and line['n_gpus'] == 2 and line['gpu_launches'] == 0
    assert line['config'] == moe_bench.grouped_config(2, 32, False)
    assert line['metric'] == 'fp8_block_scaled_gemm_tflops' and line['unit'] == 'TFLOP/s' and line['higher_is_better'] is True
    assert line['value'] > 0 and line['cpu_baseline']['kind'] == 'port' and line['cpu_baseline']['value'] == line['value']
    assert line['e2e'] == {'value': line['value'], 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}


@pytest.mark.skipif(torch.cuda.is_available(), reason='checks the behaviour of a box without a GPU')
def test_benchmark_refuses_to_run_without_a_gpu():
    proc, line = _run_bench('--steps', '1')
    assert proc.returncode != 0 and line is None
    assert 'no CPU fallback' in proc.stderr


def test_cluster_split_never_exceeds_the_resident_clusters():
    """A K split inside a thread-block cluster only pays when all clusters run as one wave: for a range of few-hundred-row
    problems the heuristic's cluster tilings stay within `dg_resident_clusters` (a cluster must fit into one GPC)."""
    lib = L.lib()
    caps = [lib.dg_resident_clusters(s) for s in range(0, 9)]
    assert caps[1] == 148 and caps[2] <= 74 and caps[4] <= 148 // 4 and caps[8] <= 148 // 8 and all(c > 0 for c in caps[1:])
    for m in (1, 64, 128, 256, 384, 512, 768, 1024):
        for n, k in ((2112, 7168), (576, 7168), (4096, 7168), (7168, 2048), (7168, 16384), (1024, 7168)):
            d = L.GemmDesc()
            d.a = d.b = d.d = d.sfa = d.sfb = 0x1000
            d.a_dtype, d.b_dtype, d.d_dtype = L.E4M3, L.E4M3, L.BF16
            d.m, d.n, d.k = m, n, k
            d.outer_stride_a = d.outer_stride_b = k
            d.outer_stride_d = n
            d.sfa_stride, d.sfb_stride = (m + 7) // 8 * 8, (n + 7) // 8 * 8
            cfg = L.GemmConfig()
            assert lib.dg_select_config(ctypes.byref(d), ctypes.byref(cfg)) == 0, L.last_error()
            c = cfg.as_dict()
            if c['cluster_split']:
                clusters = -(-m // 128) * -(-n // c['block_n'])
                assert clusters <= caps[c['split_k']], (m, n, k, c)
