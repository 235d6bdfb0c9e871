"""The C-ABI library loads without a GPU and exports every symbol include/flux_cuda.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "flux_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(flux_cuda_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(fx):
    L = fx.lib()
    names = declared_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, "declared in flux_cuda.h but not exported: %s" % missing


def test_no_cpu_fallback_without_gpu(fx):
    import torch
    if torch.cuda.is_available():
        return
    h = ctypes.c_void_p()
    rc = fx.lib().flux_cuda_ctx_create(0, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert b"no CUDA device" in fx.lib().flux_cuda_last_error()


def test_product_does_not_touch_the_oracle():
    """Nothing in the package, the headers or the C sources may import, link or read oracle/."""
    bad = []
    for base in ("flux2.c_b200", "include"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, base)):
            if "build" in dirpath.split(os.sep):
                continue
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".c", ".cc", ".h")):
                    src = open(os.path.join(dirpath, f), errors="ignore").read()
                    if re.search(r"\boracle[/.]|from oracle|import oracle|_ref/", src):
                        bad.append(os.path.join(dirpath, f))
    assert not bad, bad


def test_seam_defines_every_symbol_of_the_objects_it_replaces():
    """flux_cuda_seam.c stands in for the reference's flux_transformer.o and flux_sample.o: every function or global
    those objects export must be defined by the seam, or the reference's other objects would not link."""
    import subprocess
    ref = os.path.join(ROOT, "oracle", "_ref")
    seam = os.path.join(ref, "obj_seam", "flux_cuda_seam.o")
    theirs = [os.path.join(ref, "obj_blas", f) for f in ("flux_transformer.o", "flux_sample.o")]
    if not (os.path.exists(seam) and all(os.path.exists(t) for t in theirs)):
        import pytest
        pytest.skip("oracle/_ref objects not built (make -C oracle cli)")

    def exported(path):
        out = subprocess.run(["nm", "--defined-only", "-g", path], capture_output=True, text=True, check=True).stdout
        return {line.split()[-1] for line in out.splitlines() if line.strip()}

    missing = set().union(*[exported(t) for t in theirs]) - exported(seam)
    assert not missing, sorted(missing)
    # the same for the text encoder's file and its seam
    qseam, qtheirs = os.path.join(ref, "obj_seam", "flux_cuda_qwen3_seam.o"), os.path.join(ref, "obj_blas", "flux_qwen3.o")
    if os.path.exists(qseam) and os.path.exists(qtheirs):
        missing = exported(qtheirs) - exported(qseam)
        assert not missing, sorted(missing)
