"""The checked build of the library (libflux_cuda_debug.so, compiled with -DFLUX_CUDA_DEBUG): kernels verify the tile,
row and alignment arithmetic of every access they are about to make and record a violation in the error word instead
of touching memory. The tiny-model tests must pass under it unchanged - no check may fire on a correct run."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "flux2.c_b200", "libflux_cuda_debug.so")


def test_tiny_model_suite_passes_on_the_checked_build(fx):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    if not os.path.exists(CHECKED):
        pytest.skip("libflux_cuda_debug.so is not built (python flux2.c_b200/build.py --checked)")
    assert fx.lib().flux_cuda_build_checked() == 0  # this process runs the normal build
    env = dict(os.environ, FLUX_CUDA_LIBRARY=CHECKED)
    probe = subprocess.run([sys.executable, "-c",
                            "import sys; sys.path.insert(0, %r); from conftest import load_package; "
                            "print(load_package().lib().flux_cuda_build_checked())" % os.path.join(ROOT, "tests")],
                           capture_output=True, text=True, env=env, timeout=300)
    assert probe.stdout.strip().endswith("1"), probe.stdout + probe.stderr
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_model_gpu.py"),
                        os.path.join(ROOT, "tests", "test_kernels_gpu.py"), os.path.join(ROOT, "tests", "test_gemm_gpu.py"),
                        "-q", "-m", "gpu", "-k", "tiny or attention_matches or adaln or gemm", "-x", "-p",
                        "no:cacheprovider"], capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
