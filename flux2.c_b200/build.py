"""Builds the CUDA library of this package in-tree with nvcc for sm_100a.

The output, ``libflux_cuda.so``, sits next to this file. It is the only artefact the host side
loads; there is no JIT cache and no fallback when it is missing.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libflux_cuda.so")
LIB_CHECKED = os.path.join(HERE, "libflux_cuda_debug.so")  # the same sources with -DFLUX_CUDA_DEBUG

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC,-O3,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cc", ".c")))


def needs_build(lib=LIB):
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, checked=False):
    """Compile every source under csrc/ into libflux_cuda.so (one nvcc -c per file, then a link). checked=True builds
    libflux_cuda_debug.so instead: the same sources with -DFLUX_CUDA_DEBUG (index and alignment checks in the
    kernels that record a violation in the context's error word instead of accessing memory)."""
    lib = LIB_CHECKED if checked else LIB
    extra = ["-DFLUX_CUDA_DEBUG"] if checked else []
    if not force and not needs_build(lib):
        return lib
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build", "checked" if checked else "plain")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-I", INCLUDE, "-I", CSRC, "-c", src, "-o", obj]
        if src.endswith(".c"):
            cmd = ["gcc", "-O2", "-fPIC", "-Wall"] + extra + ["-I", INCLUDE, "-I", CSRC, "-c", src, "-o", obj]
        if verbose and not src.endswith(".c"):
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write("nvcc failed on %s:\n%s\n" % (src, out))
        elif verbose or out.strip():
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("CUDA build failed")
    link = [nvcc, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart", "-ldl",
                                                  "-lpthread"]
    subprocess.check_call(link)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv))
