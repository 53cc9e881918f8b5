"""Importing the package (and loading libdg_b200.so and the `_C` extension) must not create a CUDA context: a process that
imports deep_gemm and then forks workers, as tests/test_lazy_init.py does, still gets a working device in every child."""

import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = textwrap.dedent('''
    import sys
    sys.path.insert(0, %r)
    import torch
    import torch.multiprocessing as mp
    import deep_gemm
    from deep_gemm import _lib
    _lib.lib()                                   # the C ABI library is loaded in the parent as well
    assert deep_gemm._C is None or deep_gemm._C.__file__
    assert not torch.cuda.is_initialized(), 'importing deep_gemm initialised CUDA'


    def main(local_rank):
        torch.cuda.set_device(0)
        a = torch.zeros(128, 128, dtype=torch.uint8, device='cuda').view(torch.float8_e4m3fn)
        sf = torch.ones(128, 4, device='cuda')
        d = torch.full((128, 128), float('nan'), dtype=torch.bfloat16, device='cuda')
        deep_gemm.fp8_gemm_nt((a, sf), (a, sf), d)
        torch.cuda.synchronize()
        assert deep_gemm.device_status() == 0 and float(d.abs().max()) == 0.0


    mp.start_processes(main, nprocs=2, start_method='fork')
    print('PASS')
''') % os.path.join(ROOT, 'deepgemm-ascend_b200')


def test_import_then_fork_then_use_the_device():
    proc = subprocess.run([sys.executable, '-c', SCRIPT], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and 'PASS' in proc.stdout, proc.stderr[-3000:]
