"""Generate the golden fixtures in this directory from the reference's own test code.

Run once, in a container that has the reference checkout (it cannot travel to a
GPU box):  ``python tests/golden/make_golden.py /path/to/reference``

The reference's ``tests/generators.py`` and the ``reference()`` layout model in
``tests/test_layout.py`` are pure torch; the only NPU dependency is the device
string and one seeding call. This script loads their source text, rewrites
``'npu'`` to ``'cpu'`` in memory (nothing is copied into this repository), calls
them, and stores inputs and expected outputs as small ``.pt`` files. The parity
tests and the oracle tests then compare against these files.
"""

from __future__ import annotations

import ast
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_generators(ref_root: str) -> types.ModuleType:
    src = open(os.path.join(ref_root, 'tests', 'generators.py')).read()
    src = src.replace("'npu'", "'cpu'").replace('torch.npu.manual_seed(seed)', 'pass')
    mod = types.ModuleType('ref_generators')
    sys.modules['ref_generators'] = mod      # dataclasses look the module up by name
    mod.__dict__['__name__'] = 'ref_generators'
    exec(compile(src, 'ref_generators', 'exec'), mod.__dict__)
    return mod


def load_reference_layout_model(ref_root: str):
    """Only the pure function ``reference(sf, mn, gran_mn)`` of tests/test_layout.py."""
    tree = ast.parse(open(os.path.join(ref_root, 'tests', 'test_layout.py')).read())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == 'reference']
    ns = {'torch': torch}
    exec(compile(ast.Module(body=fn, type_ignores=[]), 'ref_layout', 'exec'), ns)
    return ns['reference']


def load_reference_stochastic_model(ref_root: str):
    """tests/utils.py::assert_stochastic_bf16_matches_fp32 with its final assert turned into `return expected`."""
    import numpy as np
    text = open(os.path.join(ref_root, 'tests', 'utils.py')).read()
    tree = ast.parse(text)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == 'assert_stochastic_bf16_matches_fp32')
    assert isinstance(fn.body[-1], ast.Assert)
    fn.body[-1] = ast.Return(value=ast.Name(id='expected', ctx=ast.Load()))
    ast.fix_missing_locations(fn)
    ns = {'torch': torch, 'np': np}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), 'ref_utils', 'exec'), ns)
    model = ns['assert_stochastic_bf16_matches_fp32']

    def run(x: torch.Tensor) -> torch.Tensor:
        return model(torch.empty(x.shape, dtype=torch.bfloat16), lambda buf: buf.copy_(x), 'golden')
    return run


def raw(t: torch.Tensor) -> torch.Tensor:
    """Store fp8 as bytes so that the files load on any torch build."""
    return t.contiguous().view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t.contiguous()


def main(ref_root: str) -> None:
    g = load_reference_generators(ref_root)
    layout_reference = load_reference_layout_model(ref_root)
    Major, GemmType, Desc = g.Major, g.GemmType, g.GemmTestDesc
    fp8, fp4 = torch.float8_e4m3fn, torch.float4_e2m1fn_x2
    out = {}

    # ---- dense cases through GemmTestDesc.generate() ------------------------------------
    dense = [
        ('dense_fp8_nt_bf16', fp8, fp8, torch.bfloat16, (48, 72, 160), Major.K, Major.K, {}),
        ('dense_fp8_nt_acc_f32', fp8, fp8, torch.float32, (33, 40, 96), Major.K, Major.K, dict(accumulate=True)),
        ('dense_fp8_nn_bias', fp8, fp8, torch.bfloat16, (40, 64, 128), Major.K, Major.MN, dict(with_bias=True)),
        ('dense_fp8_tn_alpha', fp8, fp8, torch.bfloat16, (64, 48, 64), Major.MN, Major.MN, dict(alpha=-0.375)),
        ('dense_fp8_unaligned_k', fp8, fp8, torch.float32, (16, 24, 234), Major.K, Major.K, dict(accumulate=True)),
        ('dense_fp8_recipe_32_32', fp8, fp8, torch.float32, (70, 90, 128), Major.K, Major.K,
         dict(accumulate=True, recipe=(32, 32, 32))),
        ('dense_fp8fp4_nn', fp8, fp4, torch.bfloat16, (32, 64, 128), Major.K, Major.MN, {}),
        ('dense_fp8fp4_nt', fp8, fp4, torch.bfloat16, (32, 48, 192), Major.K, Major.K, {}),
        ('dense_fp4fp4_nt', fp4, fp4, torch.bfloat16, (32, 48, 192), Major.K, Major.K, {}),
        ('dense_fp4fp4_nt_acc_f32', fp4, fp4, torch.float32, (40, 72, 448), Major.K, Major.K, dict(accumulate=True)),
    ]
    for name, adt, bdt, cdt, shape, ma, mb, kw in dense:
        d = Desc(GemmType.Normal, adt, bdt, cdt, shape, ma, mb, **kw)
        (m, n, k), a, b, c, d_ref, _ = d.generate()
        out[name] = dict(m=m, n=n, k=k, a=raw(a[0]), sfa=a[1], b=raw(b[0]), sfb=b[1],
                         a_major=ma.name, b_major=mb.name, c=c, d=d_ref,
                         recipe=d.recipe, alpha=d.alpha, accumulate=d.accumulate, with_bias=d.with_bias,
                         a_is_fp4=adt == fp4, b_is_fp4=bdt == fp4)

    # ---- BF16 family: operands are plain tensors, no scale factors --------------------------
    bf16 = torch.bfloat16
    for name, cdt, shape, ma, mb, kw in (
            ('bf16_dense_nt', bf16, (48, 72, 160), Major.K, Major.K, {}),
            ('bf16_dense_tn_acc_f32', torch.float32, (64, 48, 96), Major.MN, Major.MN, dict(accumulate=True)),
            ('bf16_dense_nn_bias', bf16, (40, 64, 128), Major.K, Major.MN, dict(with_bias=True))):
        d = Desc(GemmType.Normal, bf16, bf16, cdt, shape, ma, mb, **kw)
        (m, n, k), a, b, c, d_ref, _ = d.generate()
        out[name] = dict(m=m, n=n, k=k, a=a.contiguous(), b=b.contiguous(), a_major=ma.name, b_major=mb.name, c=c, d=d_ref,
                         accumulate=d.accumulate, with_bias=d.with_bias)
    d = Desc(GemmType.MGroupedContiguousWithPsumLayout, bf16, bf16, bf16, (200, 64, 96), Major.K, Major.K, num_groups=3)
    (m, n, k), a, b, c, d_ref, (g_layout, _) = d.generate()
    out['bf16_mgrouped_nt'] = dict(m=m, n=n, k=k, a=a.contiguous(), b=b.contiguous(), d=d_ref, psum=g_layout.tolist())
    d = Desc(GemmType.KGroupedContiguousWithPsumLayout, bf16, bf16, torch.float32, (40, 48, 256), Major.MN, Major.MN,
             accumulate=True, num_groups=3, ks_cpu=[300, 0, 170])
    (m, n, k), a, b, c, d_ref, (g_layout, _) = d.generate()
    out['bf16_kgrouped_acc_f32'] = dict(m=m, n=n, k=k, a=a.contiguous(), b=b.contiguous(), c=c, d=d_ref, psum=g_layout.tolist())

    # ---- m-grouped psum case -------------------------------------------------------------
    for name, mb in (('mgrouped_fp8_nt', Major.K), ('mgrouped_fp8_nn', Major.MN)):
        d = Desc(GemmType.MGroupedContiguousWithPsumLayout, fp8, fp8, torch.bfloat16, (200, 64, 96),
                 Major.K, mb, num_groups=3)
        (m, n, k), a, b, c, d_ref, (g_layout, _) = d.generate()
        out[name] = dict(m=m, n=n, k=k, a=raw(a[0]), sfa=a[1], b=raw(b[0]), sfb=b[1],
                         b_major=mb.name, d=d_ref, psum=g_layout.tolist(), recipe=d.recipe)

    # ---- k-grouped psum cases (operands [K, M] / [K, N], scale padding poisoned by the generator) ----
    for name, ks, acc, cdt in (('kgrouped_fp8_bf16', [300, 0, 170], False, torch.bfloat16),
                               ('kgrouped_fp8_acc_f32', [96, 512, 33], True, torch.float32)):
        d = Desc(GemmType.KGroupedContiguousWithPsumLayout, fp8, fp8, cdt, (40, 48, 256), Major.MN, Major.MN,
                 accumulate=acc, num_groups=3, ks_cpu=ks)
        (m, n, k), a, b, c, d_ref, (g_layout, _) = d.generate()
        out[name] = dict(m=m, n=n, k=k, a=raw(a[0]), sfa=a[1], b=raw(b[0]), sfb=b[1], c=c, d=d_ref,
                         psum=g_layout.tolist(), ks=ks, recipe=d.recipe)

    # ---- psum layout and N(0,1) quantiser ------------------------------------------------
    g.reset_seed()
    total, psum_list, _ = g.generate_psum_layout(300, 5, 256, device='cpu')
    out['psum_layout'] = dict(total=total, psum=psum_list,
                              valid=[(s.start, s.stop) for s in g.iter_psum_slice(psum_list, 256)],
                              pad=[(s.start, s.stop) for s in g.iter_psum_sep(psum_list, 256)])
    g.reset_seed()
    x = torch.randn(70, 300)
    (q, sf), rep = g.quantize_with_major(x, [1, 128], fp8, major_dim=1)
    out['quant_fp8_1x128'] = dict(x=x, q=raw(q), sf=sf, repr=rep)
    (q, sf), rep = g.quantize_with_major(x, [128, 128], fp8, major_dim=1)
    out['quant_fp8_128x128'] = dict(x=x, q=raw(q), sf=sf, repr=rep)
    x4 = torch.randn(64, 96)
    (q, sf), rep = g.quantize_with_major(x4, [1, 32], fp4, major_dim=1)
    out['quant_fp4_1x32'] = dict(x=x4, q=q.contiguous(), sf=sf, repr=rep)

    # ---- scale-factor layout model --------------------------------------------------------
    torch.manual_seed(1)
    sf_cases = {}
    for dtype in (torch.float32, torch.int16):
        for mn, k, gran, batches in ((40, 128, 1, 1), (41, 7168 // 8, 1, 1), (130, 224, 32, 1),
                                     (257, 96, 128, 1), (64, 160, 1, 2), (96, 352, 32, 3)):
            div = 32 if dtype == torch.float32 else 64
            shape = ((mn + gran - 1) // gran, (k + div - 1) // div)
            if batches > 1:
                shape = (batches, *shape)
            if dtype == torch.float32:
                sf = (torch.randint(1, 255, shape, dtype=torch.int32) * (1 << 23)).view(torch.float32)
            else:
                sf = torch.randint(-32768, 32768, shape, dtype=torch.int16)
            exp = layout_reference(sf, mn, gran)
            sf_cases[f'{str(dtype)[6:]}_mn{mn}_k{k}_g{gran}_b{batches}'] = dict(
                sf=sf, mn=mn, k=k, gran=gran, expected=exp.contiguous(),
                expected_stride=tuple(exp.stride()))
    out['sf_layout'] = sf_cases

    # ---- scale-factor layout of k-grouped operands (tests/test_layout.py:77-104 with its own helpers) ----
    kg_cases = {}
    for dtype in (torch.float32, torch.int16):
        for mn, sizes, gran, mn_major in ((72, (240, 0, 512, 100), 1, False), (130, (256, 33), 32, True),
                                          (257, (16, 496, 1), 128, False)):
            div = 32 if dtype == torch.float32 else 64
            k, psum = g.generate_psum_layout_with_sizes(sizes, 256)
            shape = ((mn + gran - 1) // gran, (k + div - 1) // div)
            if dtype == torch.float32:
                sf = (torch.randint(1, 255, shape, dtype=torch.int32) * (1 << 23)).view(torch.float32)
            else:
                sf = torch.randint(-32768, 32768, shape, dtype=torch.int16)
            expected = sf.clone()
            for span in g.iter_psum_sep(psum, 256, div):
                expected[..., span] = 0
                sf[..., span] = 0 if dtype == torch.int16 else -1
            exp = layout_reference(expected, mn, gran)
            kg_cases[f'{str(dtype)[6:]}_mn{mn}_k{k}_g{gran}_{"mn" if mn_major else "k"}major'] = dict(
                sf=sf, mn=mn, k=k, gran=gran, psum=list(psum), mn_major=mn_major, expected=exp.contiguous())
    out['sf_layout_k_grouped'] = kg_cases

    # ---- stochastic BF16 rounding model ----------------------------------------------------
    stochastic = load_reference_stochastic_model(ref_root)
    torch.manual_seed(2)
    x = torch.randn(9, 37) * 5
    x[0, 0], x[1, 1], x[2, 2] = float('nan'), float('inf'), 0.0
    out['stochastic_bf16'] = dict(x=x, expected=stochastic(x).view(torch.int16))

    torch.save(out, os.path.join(HERE, 'reference_vectors.pt'))
    size = os.path.getsize(os.path.join(HERE, 'reference_vectors.pt'))
    print(f'wrote reference_vectors.pt, {size / 1024:.1f} KiB, {len(out)} groups')


if __name__ == '__main__':
    if len(sys.argv) != 2:
        raise SystemExit('usage: python tests/golden/make_golden.py <path of the DeepGEMM-Ascend checkout>')
    main(sys.argv[1])
