"""
Build libios_runtime.so in-tree with nvcc for sm_100a.

    python build.py [--force]

Every translation unit under csrc/ is compiled to build/*.o (in parallel) and linked into
ios/libios_runtime.so, where ios/contrib/ios_runtime.py looks for it.  The CUDA runtime is linked
statically, so the library loads on a machine without a GPU (the driver is only opened by the first
call that needs a device).
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OBJ = os.path.join(HERE, 'build')
TARGET = os.path.join(HERE, 'ios', 'libios_runtime.so')
SOURCES = ['graph.cc', 'dp_search.cc', 'bandwidth_ops.cu', 'conv_direct.cu', 'conv_tc.cu', 'conv_tc_patch.cu', 'plan.cu', 'runtime.cu', 'no_alloc.cu']
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
         '-Xcompiler', '-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function', '-x', 'cu']


def _newer(path, deps):
    if not os.path.exists(path):
        return False
    stamp = os.path.getmtime(path)
    return all(os.path.getmtime(d) <= stamp for d in deps)


def build(force=False, verbose=True):
    os.makedirs(OBJ, exist_ok=True)
    sources = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith('.h')]
    headers.append(os.path.join(HERE, '..', 'include', 'ios_runtime.h'))
    jobs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + '.o')
        path = os.path.join(CSRC, src)
        if force or not _newer(obj, [path] + headers):
            jobs.append((path, obj))
    objs = [os.path.join(OBJ, os.path.splitext(s)[0] + '.o') for s in sources]

    def compile_one(job):
        path, obj = job
        cmd = [NVCC] + FLAGS + ['-c', path, '-o', obj]
        done = subprocess.run(cmd, capture_output=True, text=True)
        return path, done

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs)))) as pool:
        for path, done in pool.map(compile_one, jobs):
            if verbose and (done.stdout.strip() or done.stderr.strip()):
                print(done.stdout + done.stderr)
            if done.returncode != 0:
                raise RuntimeError(f'nvcc failed on {path}:\n{done.stdout}\n{done.stderr}')
    if jobs or force or not os.path.exists(TARGET):
        cmd = [NVCC, '-shared', '-o', TARGET] + objs + ['-cudart', 'static', '-lpthread', '-ldl', '-lrt']
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f'link failed:\n{done.stdout}\n{done.stderr}')
    return TARGET


if __name__ == '__main__':
    print(build(force='--force' in sys.argv))
