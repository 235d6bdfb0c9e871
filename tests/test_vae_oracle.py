"""Pins the CPU restatement of the VAE decoder (oracle/vae_oracle.py) to the reference build (oracle/_ref): the two
must produce the same image from the same seeded weights and latent. Runs on the CPU."""
import os

import numpy as np
import pytest


def psnr(a, b):
    mse = float(((a.astype(np.float64) - b.astype(np.float64)) ** 2).mean())
    return 99.0 if mse == 0 else 10.0 * np.log10(255.0 ** 2 / mse)


@pytest.mark.parametrize("h,w", [(4, 4), (5, 3)])
def test_vae_oracle_matches_reference(fx, tmp_path, h, w):
    import flux2_c_b200.synth as synth
    from oracle import ref_binding as rb
    from oracle.vae_oracle import VaeOracle
    kind = rb.best_kind()
    if kind is None:
        pytest.skip("the reference build (oracle/_ref) is not present")
    W = synth.make_vae_weights(seed=5, rich=True)
    path = str(tmp_path / "vae.safetensors")
    synth.write_safetensors(path, W, dtype="F32")
    lib = rb.RefLib(kind)
    vae = lib.load_vae(path)
    lat = synth.make_latent(77, 128, h, w)
    want = lib.vae_decode(vae, lat)
    got, f = VaeOracle(W).decode(lat)
    assert got.shape == want.shape == (16 * h, 16 * w, 3)
    # not a flat image: the weights make the output use a good part of the range
    assert want.std() > 10
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1 and (d > 0).mean() < 0.02  # f32 summation order only: an occasional off-by-one after truncation
    assert psnr(got, want) > 55


@pytest.mark.parametrize("H,W", [(64, 64), (48, 80)])
def test_vae_oracle_encode_matches_reference(fx, tmp_path, H, W):
    import flux2_c_b200.synth as synth
    from oracle import ref_binding as rb
    from oracle.vae_oracle import VaeOracle
    kind = rb.best_kind()
    if kind is None:
        pytest.skip("the reference build (oracle/_ref) is not present")
    Wt = synth.make_vae_weights(seed=5, rich=True)
    path = str(tmp_path / "vae.safetensors")
    synth.write_safetensors(path, Wt, dtype="F32")
    lib = rb.RefLib(kind)
    vae = lib.load_vae(path)
    img = np.random.default_rng(H).uniform(-1.0, 1.0, (3, H, W)).astype(np.float32)
    want = lib.vae_encode(vae, img)
    got = VaeOracle(Wt).encode(img)
    assert got.shape == want.shape == (128, H // 16, W // 16)
    assert float(np.abs(want).mean()) > 0.05
    rel = float(np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64)))
    assert rel < 2e-4
