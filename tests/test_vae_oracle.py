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
