"""Builds libspiky_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m spiky_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects go to spiky_b200/lib/obj, the library to
spiky_b200/lib/libspiky_b200.so; `-Xptxas -v` output (registers, spills, shared memory per kernel)
is kept in spiky_b200/lib/ptxas.log.
"""
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libspiky_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xptxas", "-v", "--compiler-options", "-fPIC", "-Xcompiler", "-Wall"]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA toolkit is required to build spiky_b200")


def _host_compiler():
    # the distribution g++ links libstdc++ dynamically; some images ship a static-libstdc++ g++ first on PATH
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def _cutlass_includes():
    """Include directories of the CUTLASS / CuTe header tree shipped inside the flashinfer package (headers only;
    used by fp32_gemm_sm100.cu).  Empty when no tree is found: that file then builds its stubs."""
    import importlib.util
    for pkg, sub in (("flashinfer", ("data", "cutlass")), ("tilelang", ("3rdparty", "cutlass"))):
        try:
            spec = importlib.util.find_spec(pkg)
        except (ImportError, ValueError):
            spec = None
        if spec is None or not spec.submodule_search_locations:
            continue
        root = os.path.join(list(spec.submodule_search_locations)[0], *sub)
        inc, util = os.path.join(root, "include"), os.path.join(root, "tools", "util", "include")
        if os.path.exists(os.path.join(inc, "cutlass", "gemm", "collective", "builders", "sm100_9xBF16_umma_builder.inl")):
            return [inc] + ([util] if os.path.isdir(util) else [])
    return []


def _extra_flags(src):
    if os.path.basename(src) != "fp32_gemm_sm100.cu":
        return []
    inc = _cutlass_includes()
    if not inc:
        return ["-DLUTB_NO_CUTLASS"]
    flags = ["--expt-relaxed-constexpr"]
    for d in inc:
        flags += ["-I", d]
    return flags


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    if not sources:
        raise RuntimeError("no CUDA sources found under " + CSRC)
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest(sources + headers):
        return LIB
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    hdr_time = _newest(headers) if headers else 0.0

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
            return obj, ""
        cmd = [nvcc] + ARCH + FLAGS + _extra_flags(src) + _host_compiler() + ["-c", src, "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, p.stdout, p.stderr))
        return obj, "== %s\n%s%s" % (os.path.basename(src), p.stdout, p.stderr)

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(compile_one, sources))
    objs = [r[0] for r in results]
    log = "".join(r[1] for r in results)
    if log:
        with open(os.path.join(LIBDIR, "ptxas.log"), "a" if not force else "w") as f:
            f.write(log)
        if verbose:
            print(log)
    cmd = [nvcc] + ARCH + _host_compiler() + ["-shared", "-o", LIB] + objs
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (p.stdout, p.stderr))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
