"""Builds libnsa_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m native_sparse_attention_pytorch_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'libnsa_b200.so')
SOURCES = ['nsa_abi.cu', 'nsa_simt_attend.cu', 'nsa_select.cu', 'nsa_combine.cu', 'nsa_rotary.cu', 'nsa_windows.cu', 'nsa_rmsnorm.cu', 'nsa_decode.cu', 'nsa_sm100_sel.cu']


def _newest_source_mtime():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, 'include', 'nsa_b200.h')]
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
    """Compile every kernel file for sm_100a and link the shared library."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source_mtime():
        return LIB
    nvcc = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
    objdir = os.path.join(HERE, 'build')
    os.makedirs(objdir, exist_ok=True)
    flags = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
             '-Xcompiler', '-fPIC', '-I', os.path.join(ROOT, 'include'), '-I', CSRC]
    if verbose:
        flags += ['-Xptxas', '-v']
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace('.cu', '.o'))
        cmd = [nvcc, *flags, '-c', os.path.join(CSRC, src), '-o', obj]
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(f'--- {src} ---\n{out}\n')
        if p.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}')
        objs.append(obj)
    link = [nvcc, '-shared', '-o', LIB, *objs, '-cudart', 'static', '-gencode', 'arch=compute_100a,code=sm_100a']
    subprocess.run(link, check=True)
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
