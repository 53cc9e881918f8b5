"""Build libdg_b200.so in-tree with nvcc for sm_100a.

Usage: ``python deepgemm-ascend_b200/build.py [--force] [--verbose]``. The library lands next to the Python
package (``deep_gemm/libdg_b200.so``) so that it is found without installation.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OUT = os.path.join(HERE, 'deep_gemm', 'libdg_b200.so')
SOURCES = ['api.cu', 'mx_gemm.cu', 'transform_sf.cu', 'quant_ops.cu', 'sleep.cu']
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=hidden', '--expt-relaxed-constexpr']


def find_nvcc() -> str:
    nvcc = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(nvcc):
        raise RuntimeError('nvcc not found: libdg_b200.so cannot be built')
    return nvcc


def is_stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, '..', 'include', 'dg_b200.h'))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return OUT
    nvcc = find_nvcc()
    objs = []
    build_dir = os.path.join(HERE, 'build')
    os.makedirs(build_dir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace('.cu', '.o'))
        cmd = [nvcc, *NVCC_FLAGS, *os.environ.get('DG_EXTRA_NVCC_FLAGS', '').split(), '-c', os.path.join(CSRC, src), '-o', obj]
        if verbose:
            cmd += ['-Xptxas', '-v']
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}')
    link = [nvcc, '-shared', '-o', OUT, *objs, '-gencode', 'arch=compute_100a,code=sm_100a']
    subprocess.run(link, check=True)
    return OUT


EXT_OUT = os.path.join(HERE, 'deep_gemm', '_C.so')


def ext_is_stale() -> bool:
    if not os.path.exists(EXT_OUT):
        return True
    built = os.path.getmtime(EXT_OUT)
    deps = [os.path.join(CSRC, 'python_api.cpp'), os.path.join(HERE, '..', 'include', 'dg_b200.h')]
    deps += [os.path.join(CSRC, 'apis', f) for f in os.listdir(os.path.join(CSRC, 'apis'))]
    return any(os.path.getmtime(d) > built for d in deps) or os.path.getmtime(OUT) > built


def build_extension(force: bool = False, verbose: bool = False) -> str:
    """The `_C` torch extension (pybind11 + torch headers, g++): the reference's csrc/python_api.cpp surface over the
    C ABI. Needs libdg_b200.so next to it (linked with an $ORIGIN run path)."""
    if not force and not ext_is_stale():
        return EXT_OUT
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    cxx = shutil.which('g++') or 'g++'
    torch_lib = os.path.join(os.path.dirname(torch.__file__), 'lib')
    cmd = [cxx, '-O2', '-std=c++17', '-shared', '-fPIC', '-fvisibility=hidden', '-Wno-attributes',
           '-DTORCH_EXTENSION_NAME=_C', '-DTORCH_API_INCLUDE_EXTENSION_H',
           '-D_GLIBCXX_USE_CXX11_ABI=%d' % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           os.path.join(CSRC, 'python_api.cpp'), '-o', EXT_OUT,
           *['-I' + p for p in cpp_extension.include_paths()], '-I' + sysconfig.get_paths()['include'],
           '-I/usr/local/cuda/include',
           '-L' + torch_lib, '-ltorch_python', '-ltorch', '-ltorch_cpu', '-lc10', '-lc10_cuda',
           '-L' + os.path.dirname(OUT), '-l:libdg_b200.so', '-Wl,-rpath,$ORIGIN', '-Wl,-rpath,' + torch_lib]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError('g++ failed on python_api.cpp')
    return EXT_OUT


if __name__ == '__main__':
    path = build(force='--force' in sys.argv, verbose='--verbose' in sys.argv)
    print(path)
    print(build_extension(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
