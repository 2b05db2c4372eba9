"""In-tree build of the native parts: the C++ host runtime (`_core`, pybind11) and the sm_100a
CUDA kernel library (`libxllm_kernels.so`, plain `extern "C"` entry points called through ctypes).

    python -m xllm_wxh_b200.build_ext [--force] [--core-only|--cuda-only]

The kernels are compiled for exactly one target: `-gencode arch=compute_100a,code=sm_100a`.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CORE_DIR = os.path.join(HERE, "csrc", "core")
CUDA_DIR = os.path.join(HERE, "csrc", "cuda")
BUILD_DIR = os.path.join(HERE, "csrc", "build")
CORE_SO = os.path.join(HERE, "_core" + sysconfig.get_config_var("EXT_SUFFIX"))
KERNELS_SO = os.path.join(HERE, "libxllm_kernels.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _newer(src_files, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_files)


def _run(cmd, log=None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + p.stdout)
    if p.returncode != 0:
        sys.stderr.write(p.stdout)
        raise RuntimeError("build failed: " + " ".join(cmd))
    return p.stdout


def build_core(force=False):
    import pybind11
    srcs = [os.path.join(CORE_DIR, f) for f in os.listdir(CORE_DIR) if f.endswith((".cpp", ".h"))]
    if not force and not _newer(srcs, CORE_SO):
        return CORE_SO
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           os.path.join(CORE_DIR, "bindings.cpp"), "-o", CORE_SO, "-lrt", "-lpthread"]
    _run(cmd)
    return CORE_SO


def build_core_sanitized(force=False):
    """The same extension with AddressSanitizer and UndefinedBehaviorSanitizer (host-side race / memory checking of the
    scheduler, block manager, batch builder, tokenizer ...).  Load it with XLLM_CORE_SO=<path> and libasan preloaded."""
    import pybind11
    out_dir = os.path.join(BUILD_DIR, "asan")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "_core" + sysconfig.get_config_var("EXT_SUFFIX"))
    srcs = [os.path.join(CORE_DIR, f) for f in os.listdir(CORE_DIR) if f.endswith((".cpp", ".h"))]
    if not force and not _newer(srcs, out):
        return out
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall", "-fno-omit-frame-pointer",
           "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           os.path.join(CORE_DIR, "bindings.cpp"), "-o", out, "-lrt", "-lpthread"]
    _run(cmd)
    return out


def sanitizer_runtime():
    """Value for LD_PRELOAD: libasan (the interpreter itself is not instrumented) followed by libstdc++, which must be
    loaded by the time libasan resolves the real `__cxa_throw`, or the first C++ exception aborts the process."""
    out = []
    for lib in ("libasan.so", "libstdc++.so.6"):
        p = subprocess.run(["g++", "-print-file-name=" + lib], stdout=subprocess.PIPE, text=True).stdout.strip()
        if not p or os.path.sep not in p:
            return ""
        out.append(os.path.realpath(p))
    return " ".join(out)


CAPI_DIR = os.path.join(HERE, "csrc", "capi")
CAPI_SO = os.path.join(HERE, "libxllm.so")


def build_capi(force=False):
    """`libxllm.so`: the C interface (csrc/capi/xllm_c_api.h) over the Python API, through the CPython C API."""
    srcs = [os.path.join(CAPI_DIR, f) for f in os.listdir(CAPI_DIR)]
    if not force and not _newer(srcs, CAPI_SO):
        return CAPI_SO
    inc = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall", "-I", inc, "-I", CAPI_DIR,
           os.path.join(CAPI_DIR, "xllm_c_api.cpp"), "-o", CAPI_SO]
    # link libpython when a shared one exists, so that a plain C program can load the library; inside a Python process
    # the interpreter's own symbols are used either way
    if any(os.path.exists(os.path.join(d, f"libpython{ver}.so")) for d in (libdir, "/usr/lib/x86_64-linux-gnu")):
        cmd += [f"-L{libdir}", f"-lpython{ver}"]
    _run(cmd + ["-lpthread"])
    return CAPI_SO


def cuda_sources():
    return sorted(os.path.join(CUDA_DIR, f) for f in os.listdir(CUDA_DIR) if f.endswith(".cu"))


def build_cuda(force=False):
    os.makedirs(BUILD_DIR, exist_ok=True)
    srcs = cuda_sources()
    hdrs = [os.path.join(CUDA_DIR, f) for f in os.listdir(CUDA_DIR) if f.endswith((".cuh", ".h"))]
    objs, jobs = [], []
    for s in srcs:
        o = os.path.join(BUILD_DIR, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer([s] + hdrs, o):
            jobs.append((s, o))
    def compile_one(job):
        s, o = job
        _run([NVCC, *NVCC_FLAGS, "-I", CUDA_DIR, "-c", s, "-o", o], log=o + ".log")
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    if jobs or not os.path.exists(KERNELS_SO):
        _run([NVCC, "-shared", "-o", KERNELS_SO, *objs, "-lcuda", "-L/usr/local/cuda/lib64/stubs", "-lcudart"])
    return KERNELS_SO


def build_all(force=False, core=True, cuda=True):
    out = []
    if core:
        out.append(build_core(force))
        try:
            out.append(build_capi(force))
        except Exception as e:            # the C interface is optional: Python headers may be missing on a serving box
            sys.stderr.write(f"libxllm.so not built: {e}\n")
    if cuda:
        out.append(build_cuda(force))
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_all(force, core="--cuda-only" not in sys.argv, cuda="--core-only" not in sys.argv))
