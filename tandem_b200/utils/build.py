"""Ahead-of-time, in-tree builds of the two native libraries.

  _host<ext>.so       C++17 host runtime (shared memory, channels, progress
                      thread, CPU collectives), a pybind11 module.
  libtb200_cuda.so    every sm_100a kernel plus the symmetric-memory helpers,
                      exported as plain C symbols and called through ctypes.

Both land beside the package so a source checkout with its built libraries can
be copied to a GPU machine as is.  The reference instead JIT-builds into
~/.cache/torch_extensions on first use and passes no -arch flag
(tandem/engine.py:22-37); here the only target is sm_100a.
"""

import os
import shutil
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG, "csrc")
CUDA = os.path.join(PKG, "cuda")
HOST_SOURCES = ["shm.cpp", "channel.cpp", "engine.cpp", "bind.cpp"]
HOST_LIB = os.path.join(PKG, "_host" + sysconfig.get_config_var("EXT_SUFFIX"))
CUDA_LIB = os.path.join(PKG, "libtb200_cuda.so")
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)
    return r


def _sources(folder, exts):
    return sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(exts))


def build_host(force=False, verbose=False):
    import pybind11

    srcs = [os.path.join(CSRC, s) for s in HOST_SOURCES]
    deps = _sources(CSRC, (".cpp", ".h"))
    if not force and not _newer(HOST_LIB, deps):
        return HOST_LIB
    tmp = HOST_LIB + f".{os.getpid()}.tmp"
    cmd = ["g++", "-O3", "-std=c++17", "-Wall", "-Wextra", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-I{sysconfig.get_paths()['include']}", f"-I{pybind11.get_include()}", *srcs, "-o", tmp, "-lrt", "-lpthread"]
    _run(cmd, verbose)
    os.replace(tmp, HOST_LIB)
    return HOST_LIB


def nvcc_path():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def build_cuda(force=False, verbose=False):
    """Compiles every .cu under cuda/ into one shared library for sm_100a."""
    srcs = [s for s in _sources(CUDA, (".cu",))]
    deps = _sources(CUDA, (".cu", ".cuh", ".h"))
    if not srcs:
        return None
    if not force and not _newer(CUDA_LIB, deps):
        return CUDA_LIB
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    flags = [*NVCC_ARCH, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v", f"-I{CUDA}"]
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [s] + [d for d in deps if not d.endswith(".cu")]):
            cmd = [nvcc, *flags, "-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    for cmd, p in procs:
        out, _ = p.communicate()
        log.append(out)
        if p.returncode != 0:
            raise RuntimeError(f"build failed: {' '.join(cmd)}\n{out}")
    with open(os.path.join(objdir, "ptxas.log"), "a" if not force else "w") as f:
        f.write("\n".join(log))
    tmp = CUDA_LIB + f".{os.getpid()}.tmp"
    _run([nvcc, *NVCC_ARCH, "-shared", "-o", tmp, *objs], verbose)
    os.replace(tmp, CUDA_LIB)
    return CUDA_LIB


def build_all(force=False, verbose=False):
    return build_host(force, verbose), build_cuda(force, verbose)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
