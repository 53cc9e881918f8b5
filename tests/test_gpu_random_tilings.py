"""Seeded random walk over dense problems, operand kinds, majors, epilogue variants and forced tilings.

Every draw is a problem of random extents (a quarter of them tiny, a quarter powers of two) with a random `config=`
override (block_n, cta_group, K splits through the workspace or a cluster, pipeline depth, epilogue warps, raster
group, staging boxes). Combinations the library refuses are skipped (it must refuse them with a message, not with a
CUDA error); everything it accepts must match the CPU oracle within the tolerance of tests/helpers.py and leave the
device status at zero. This is how the plain-store kernel with several tiles per CTA and the cluster split that
shrinks to fewer splits were found.
"""

import random

import pytest
import torch

import deep_gemm
import test_gpu_bf16 as bf16_cases
import test_gpu_fp4_majors as fp4_cases
import test_gpu_gemm as fp8_cases

pytestmark = pytest.mark.gpu


def _extent(rng, hi):
    r = rng.random()
    if r < 0.25:
        return rng.randint(1, 64)
    if r < 0.75:
        return rng.randint(1, hi)
    return rng.choice([128, 256, 384, 512, 1024, 2048, 4096])


@pytest.mark.parametrize('seed', [3, 13, 41, 42])
def test_random_problems_with_forced_tilings(seed):
    rng = random.Random(seed)
    ran = 0
    for i in range(150):
        m, n, k = _extent(rng, 1200), _extent(rng, 3000), _extent(rng, 4096)
        cfg = {'block_n': rng.choice([32, 64, 96, 128, 160, 192, 224, 256, 320, 384, 448]), 'cta_group': rng.choice([1, 2])}
        if rng.random() < 0.3:
            cfg['split_k'] = rng.choice([2, 3, 4, 5, 8])
        if 'split_k' in cfg and rng.random() < 0.6:
            cfg['cluster_split'] = 1
        if rng.random() < 0.3:
            cfg['num_stages'] = rng.choice([2, 3, 4, 5, 6])
        if rng.random() < 0.15:
            cfg['epilogue_warps'] = 8
        if rng.random() < 0.2:
            cfg['raster_group'] = rng.choice([1, 2, 4, 16, 64])
        if rng.random() < 0.15:
            cfg['store_bufs'] = rng.choice([1, 2, 3, 4])
        kind = rng.choice(['fp8', 'fp8', 'fp8', 'bf16', 'fp4', 'mixed'])
        trans = rng.choice(['nt', 'nt', 'nn', 'tn', 'tt'])
        variant = rng.choice(['plain', 'acc32', 'bias', 'alpha', 'f32', 'acc16'])
        kw = {'plain': {}, 'acc32': dict(out=torch.float32, acc=True), 'bias': dict(bias=True), 'alpha': dict(alpha=-0.75),
              'f32': dict(out=torch.float32), 'acc16': dict(acc=True)}[variant]
        try:
            if kind == 'fp8':
                fp8_cases._dense(m, n, k, trans=trans, config=cfg, seed=i, **kw)
            elif kind == 'bf16':
                bf16_cases._dense(m, n, k, trans, config=cfg, seed=i, **kw)
            else:
                kinds = ('fp4', 'fp4') if kind == 'fp4' else ('fp8', 'fp4')
                if kinds[0] == 'fp4' and trans[0] == 't' and m % 2:
                    m += 1
                if trans[1] == 'n' and n % 2:
                    n += 1
                k += k % 2
                fp4_cases._dense(kinds, m, n, k, trans, config=cfg, seed=i, **{key: v for key, v in kw.items() if key in ('out', 'acc')})
            ran += 1
        except RuntimeError as exc:
            assert 'CUDA' not in str(exc) and 'cuda' not in str(exc), f'{kind} {trans} {m}x{n}x{k} {cfg} {variant}: {exc}'
    assert ran >= 30 and deep_gemm.device_status() == 0
