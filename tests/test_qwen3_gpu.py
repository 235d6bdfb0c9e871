"""The Qwen3 text encoder on the GPU against the numpy oracle (tiny shape, several lengths and masks) and against
outputs of the reference implementation itself at the Qwen3-4B shape (tests/golden/reference_qwen3.npz).

Tolerance: relative L2 over the whole [seq, 3 * hidden] output <= 2e-2 (the encoder's output is the DiT's text
context; the step tolerances of the denoising path are stated on the velocity, which this feeds)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 2e-2


def rel(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / np.linalg.norm(b))


@pytest.fixture(scope="module")
def tiny_enc(fx, ctx):
    import flux2_c_b200.synth as synth
    from oracle import flux_oracle as fo
    d = synth.QwenDims.tiny()
    W = synth.make_qwen_weights(d, seed=1, std=0.05)
    enc = fx.TextEncoder.from_tensors(ctx, d, W, max_seq=512)
    yield synth, d, enc, fo.QwenOracle(W, d)
    enc.close()


@pytest.mark.parametrize("seq,valid", [(48, 30), (128, 128), (200, 77), (512, 300), (1, 1), (300, 299)])
def test_tiny_encoder_matches_oracle(tiny_enc, seq, valid):
    synth, d, enc, oracle = tiny_enc
    ids = np.random.default_rng(seq).integers(0, d.vocab, seq)
    mask = np.array([1] * valid + [0] * (seq - valid))
    got = enc.forward(ids, mask)
    want = oracle.forward(ids, mask)
    assert got.shape == want.shape == (seq, 3 * d.hidden)
    # rows of padded positions attend like the reference does (causal + key mask); all rows are compared
    assert rel(got, want) < TOL


def test_tiny_encoder_mask_and_order_matter(tiny_enc):
    """Guards against blind spots: the padding mask, the causal mask and token order must change the output."""
    synth, d, enc, oracle = tiny_enc
    ids = np.random.default_rng(5).integers(0, d.vocab, 96)
    full = enc.forward(ids, None)
    masked = enc.forward(ids, np.array([1] * 40 + [0] * 56))
    assert rel(masked[60:], full[60:]) > 5 * TOL          # later rows lose 40..59 as keys
    assert rel(masked[:40], full[:40]) < 1e-3              # causal: rows before the padding see the same keys
    swapped = ids.copy()
    swapped[[70, 80]] = swapped[[80, 70]]
    out_sw = enc.forward(swapped, None)
    assert rel(out_sw[:70], full[:70]) < 1e-3              # causal: earlier rows unaffected by later tokens
    assert rel(out_sw[85:], full[85:]) > 1e-3              # later rows see the swap (positions differ through RoPE)
    assert rel(oracle.forward(swapped, None), out_sw) < TOL


def test_out_of_vocabulary_ids_are_zero_rows(tiny_enc):
    synth, d, enc, oracle = tiny_enc
    ids = np.array([3, -1, d.vocab + 7, 5] * 8)
    assert rel(enc.forward(ids, None), oracle.forward(ids, None)) < TOL


def test_encoder_rejects_bad_calls(tiny_enc, fx, ctx):
    synth, d, enc, oracle = tiny_enc
    with pytest.raises(fx.FluxCudaError):
        enc.forward(np.zeros(513, dtype=np.int32))  # longer than max_seq
    W = synth.make_qwen_weights(d, seed=1, std=0.05)
    del W["model.layers.0.mlp.up_proj.weight"]
    with pytest.raises(fx.FluxCudaError):
        fx.TextEncoder.from_tensors(ctx, d, W)


def test_batch_of_prompts_equals_single_prompts(tiny_enc):
    """Three prompts with different padding in one pass: every prompt's rows equal its own single-prompt pass (up to
    the summation order of the split-K projections, which depends on the row count)."""
    synth, d, enc, oracle = tiny_enc
    seq = 96
    rng = np.random.default_rng(17)
    ids = rng.integers(0, d.vocab, (3, seq))
    mask = np.array([[1] * 96, [1] * 40 + [0] * 56, [1] * 77 + [0] * 19])
    got = enc.forward_batch(ids, mask)
    assert got.shape == (3, seq, 3 * d.hidden)
    for b in range(3):
        assert rel(got[b], enc.forward(ids[b], mask[b])) < 1e-4
        assert rel(got[b], oracle.forward(ids[b], mask[b])) < TOL
    with pytest.raises(Exception):
        enc.forward_batch(rng.integers(0, d.vocab, (6, seq)), None)  # 576 tokens: more than the capacity of 512


def test_embeddings_stay_on_the_device(tiny_enc, fx, ctx):
    """forward_device hands the sampler a device buffer: the latent equals the one obtained through host embeddings."""
    import torch
    synth, d, enc, oracle = tiny_enc
    dd = synth.Dims(hidden=256, heads=2, head_dim=128, mlp=768, n_double=1, n_single=2, text_dim=3 * d.hidden)
    model = fx.Model.from_tensors(ctx, dd, synth.make_transformer_weights(dd, seed=3, sharp=True, std=0.08))
    try:
        h, w, seq = 6, 4, 40
        ids = np.random.default_rng(9).integers(0, d.vocab, seq)
        z0 = fx.init_noise(dd.latent_ch, h, w, 5)
        sch = fx.official_schedule(3, h * w)
        want = model.sample(z0, h, w, enc.forward(ids, None), sch)
        sampler = fx.Sampler(model, h, w, seq, batch=1, max_steps=3)
        zp = torch.from_numpy(z0.copy()).pin_memory()
        got = torch.zeros(z0.size, dtype=torch.float32).pin_memory()
        for _ in range(2):  # twice: the encoder's buffer is reused by the next forward
            sampler.upload(zp.data_ptr(), enc.forward_device(ids, None))
            sampler.run(sch)
            sampler.download(got.data_ptr())
            assert rel(got.numpy().reshape(z0.shape), want) < 1e-6
        sampler.close()
    finally:
        model.close()


def test_qwen3_4b_matches_reference(fx, ctx):
    """Qwen3-4B shape, seeded weights, 64 tokens of which 40 are valid: output of the reference's qwen3_forward
    (stored for every 4th column)."""
    path = os.path.join(GOLDEN, "reference_qwen3.npz")
    if not os.path.exists(path):
        pytest.skip("reference_qwen3.npz missing")
    import flux2_c_b200.synth as synth
    g = np.load(path)
    d = synth.QwenDims.qwen3_4b()
    W = synth.make_qwen_weights(d, seed=0, threads=os.cpu_count())
    chk = float(np.abs(synth.bf16_bits_to_f32(W["model.layers.0.self_attn.q_norm.weight"]).astype(np.float64)).sum() +
                np.abs(synth.bf16_bits_to_f32(W["model.layers.26.mlp.down_proj.weight"][:64]).astype(np.float64)).sum())
    assert abs(chk - float(g["weights_checksum"])) < 1e-6 * chk
    enc = fx.TextEncoder.from_tensors(ctx, d, W, max_seq=2048)
    del W
    try:
        got = enc.forward(g["ids"], g["mask"])
        assert rel(got[:, ::4], g["out_sub"]) < TOL
        # the benchmark's length: 512 tokens, all valid, against the reference's output for the same ids
        p512 = os.path.join(GOLDEN, "reference_qwen3_512.npz")
        if os.path.exists(p512):
            g512 = np.load(p512)
            out512 = enc.forward(g512["ids"], None)
            assert out512.shape == (512, 7680) and np.isfinite(out512).all()
            assert rel(out512[:, ::4], g512["out_sub"]) < TOL
            assert abs(np.sqrt((out512.astype(np.float64) ** 2).mean()) / float(g512["out_rms"]) - 1.0) < 1e-2
            # four prompts per pass (the throughput mode of the prompt-to-image leg): same rows for every copy
            ids4 = np.stack([g512["ids"], g512["ids"][::-1], g512["ids"], g512["ids"][::-1]])
            out4 = enc.forward_batch(ids4, None)
            assert rel(out4[0][:, ::4], g512["out_sub"]) < TOL and rel(out4[2], out4[0]) < 1e-6
        else:
            ids512 = np.random.default_rng(0).integers(0, d.vocab, 512)
            out512 = enc.forward(ids512, None)
            assert out512.shape == (512, 7680) and np.isfinite(out512).all()
    finally:
        enc.close()
