"""Host-side C code of the library (schedules, seeded noise) and the numpy oracle's restatement of the same
functions, both against values produced by the reference implementation (tests/golden/reference_host.npz)."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_host.npz")


@pytest.fixture(scope="module")
def gold():
    if not os.path.exists(GOLDEN):
        pytest.skip("reference_host.npz missing")
    return np.load(GOLDEN)


SCHED = [(4, 256), (4, 1024), (4, 4096), (50, 1024), (2, 16), (4, 4301), (8, 12544)]


@pytest.mark.parametrize("steps,n", SCHED)
def test_official_schedule_library_and_oracle(fx, gold, steps, n):
    from oracle import flux_oracle as fo
    want = gold["official_%d_%d" % (steps, n)]
    assert want[0] == 1.0 and want[-1] == 0.0
    # the reference is built with -ffast-math, so the last bits of expf may differ
    assert np.allclose(fx.official_schedule(steps, n), want, rtol=0, atol=1e-6)
    assert np.allclose(fo.official_schedule(steps, n), want, rtol=0, atol=1e-6)


def test_known_schedule_values(fx):
    """Known answers of the reference's schedule for the benchmark configurations."""
    assert np.allclose(fx.official_schedule(4, 256), [1.0, 0.955391, 0.877134, 0.704112, 0.0], atol=2e-6)
    assert np.allclose(fx.official_schedule(4, 1024), [1.0, 0.958085, 0.883982, 0.717497, 0.0], atol=2e-6)
    assert np.allclose(fx.official_schedule(2, 16), [1.0, 0.876574, 0.0], atol=2e-6)


def test_linear_and_power_schedules(fx, gold):
    from oracle import flux_oracle as fo
    assert np.allclose(fx.linear_schedule(7), gold["linear_7"], atol=1e-7)
    assert np.allclose(fx.power_schedule(5, 2.0), gold["power_5_2"], atol=1e-6)
    assert np.allclose(fo.linear_schedule(7), gold["linear_7"], atol=1e-7)
    assert np.allclose(fo.power_schedule(5, 2.0), gold["power_5_2"], atol=1e-6)


@pytest.mark.parametrize("h,w,seed", [(4, 4, 42), (16, 16, 42), (32, 32, 42), (6, 4, 7), (64, 48, 123456789),
                                      (112, 112, 1)])
def test_init_noise_library(fx, gold, h, w, seed):
    n = fx.init_noise(128, h, w, seed)
    key = "noise_%d_%d_%d_" % (h, w, seed)
    assert np.allclose(n.reshape(-1)[:64], gold[key + "head"], atol=2e-6)
    assert np.allclose(n.reshape(-1)[-64:], gold[key + "tail"], atol=2e-6)
    assert abs(n.astype(np.float64).sum() - float(gold[key + "sum"])) < 1e-2
    assert abs(np.abs(n.astype(np.float64)).sum() - float(gold[key + "abs"])) < 1e-2


def test_init_noise_oracle_restatement(gold):
    """The oracle's pure-Python xoshiro256** / Box-Muller stream and subsampling map, on the elements the fixture holds."""
    from oracle import flux_oracle as fo
    src = fo.noise_source_index(128, 4, 4).reshape(-1)
    need = int(src[:64].max()) + 1
    stream = fo.randn(42, need)
    assert np.allclose(stream[src[:64]], gold["noise_4_4_42_head"], atol=2e-6)


def test_noise_is_size_independent(fx):
    """A smaller latent is a nearest-neighbour subsample of the same 112x112 master field."""
    big = fx.init_noise(128, 112, 112, 5)
    small = fx.init_noise(128, 16, 8, 5)
    sy = (np.arange(16) * 112) // 16
    sx = (np.arange(8) * 112) // 8
    assert np.array_equal(small, big[:, sy][:, :, sx])


def test_patchify_oracle_matches_reference():
    """2x2 space-to-depth between VAE latents and DiT latents (flux_patchify / flux_unpatchify): bit-exact."""
    from oracle import flux_oracle as fo
    path = os.path.join(os.path.dirname(GOLDEN), "reference_patchify.npz")
    if not os.path.exists(path):
        pytest.skip("reference_patchify.npz missing")
    g = np.load(path)
    assert np.array_equal(fo.patchify(g["in"]), g["patchified"])
    assert np.array_equal(fo.unpatchify(g["patchified"]), g["in"])
