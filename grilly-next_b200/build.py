"""Build the CUDA C-ABI library (nvcc, sm_100a only) and the grilly_core pybind11 module (g++).

    python grilly-next_b200/build.py [--force] [--verbose]

Outputs, in-tree: grilly-next_b200/lib/libgrilly_cuda.so and
grilly-next_b200/python/grilly_core*.so.  No JIT cache is used.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
PYDIR = os.path.join(HERE, "python")
CPPDIR = os.path.join(HERE, "cpp")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# the environment's CC/CXX may point at a compiler tree without OpenMP or libstdc++ headers
HOST_CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
CUDA_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-ccbin", HOST_CXX, "-I", os.path.join(ROOT, "include"), "-I", CSRC]

CU_SOURCES = ["device.cu", "flash.cu", "prefill_fp32.cu", "prefill_sm100.cu", "decode_splitkv.cu", "decode_mma.cu", "p2p_merge.cu", "kv_evict.cu",
              "kv_cache.cu", "rope_mask.cu", "nccl_group.cu", "linear_sm100.cu", "attention_unfused.cu"]
HEADERS = ["common.cuh", "tmem_ops.cuh", "sm100_ptx.cuh", os.path.join(ROOT, "include", "grilly_cuda.h")]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_cuda(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    procs = []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            cmd = [NVCC] + CUDA_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd)))
    for src, p in procs:
        if p.wait() != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    lib = os.path.join(LIBDIR, "libgrilly_cuda.so")
    if force or procs or _newer(lib, objs):
        _run([NVCC, "-shared", "-ccbin", HOST_CXX, "-o", lib] + objs + ["-lcudart", "-ldl"], verbose)
    return lib


def build_pybind(force=False, verbose=False):
    import pybind11
    srcs = [os.path.join(CPPDIR, "python", "bindings.cpp")] + sorted(
        os.path.join(CPPDIR, "src", f) for f in os.listdir(os.path.join(CPPDIR, "src")) if f.endswith(".cpp"))
    hdrs = []
    for d, _, fs in os.walk(os.path.join(CPPDIR, "include")):
        hdrs += [os.path.join(d, f) for f in fs]
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(PYDIR, "grilly_core" + ext)
    lib = os.path.join(LIBDIR, "libgrilly_cuda.so")
    if not (force or _newer(out, srcs + hdrs + [lib, os.path.join(ROOT, "include", "grilly_cuda.h")])):
        return out
    cmd = [HOST_CXX, "-O3", "-mavx2", "-pthread", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           "-I", os.path.join(CPPDIR, "include"), "-I", os.path.join(ROOT, "include")] + srcs + [
           "-L", LIBDIR, "-lgrilly_cuda", "-Wl,-rpath,$ORIGIN/../lib", "-o", out]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False):
    lib = build_cuda(force, verbose)
    mod = build_pybind(force, verbose) if os.path.isdir(os.path.join(CPPDIR, "python")) else None
    return lib, mod


if __name__ == "__main__":
    print(build_all("--force" in sys.argv, "--verbose" in sys.argv))
