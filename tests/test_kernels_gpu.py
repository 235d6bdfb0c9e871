"""Attention (K2), AdaLN (K3) and QK-norm+RoPE (K5) kernels against plain torch f32 references, through the C ABI."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch,seq,heads,sharp", [
    (1, 128, 1, 1.0), (1, 256, 2, 1.0), (1, 48, 2, 1.0), (1, 300, 3, 3.0), (1, 1536, 24, 1.0), (2, 200, 2, 2.0),
    (1, 768, 24, 0.02),
])
def test_attention_matches_torch(fx, ctx, batch, seq, heads, sharp, dtype):
    hid = heads * 128
    g = torch.Generator(device="cuda").manual_seed(seq + heads)
    qkv = (torch.randn(batch * seq, 3 * hid, device="cuda", generator=g) * sharp).to(dtype)
    out_ld = hid + 256  # output lands inside a wider [attention | mlp] buffer
    out = torch.zeros(batch * seq, out_ld, device="cuda", dtype=dtype)
    torch.cuda.synchronize()
    ctx.attention(qkv.data_ptr(), batch, seq, 3 * hid, 0, hid, 2 * hid, heads, out.data_ptr(), out_ld, 0,
                  f16=dtype == torch.float16)
    ctx.sync()
    q, k, v = [t.float().reshape(batch, seq, heads, 128).transpose(1, 2) for t in qkv.split(hid, dim=1)]
    s = (q @ k.transpose(-1, -2)) / math.sqrt(128.0)
    ref = (torch.softmax(s, dim=-1) @ v).transpose(1, 2).reshape(batch * seq, hid)
    assert torch.isfinite(out.float()).all()
    assert (out[:, hid:] == 0).all()
    assert _rel(out[:, :hid].float(), ref) < (2e-3 if dtype == torch.float16 else 1e-2)  # 16-bit P and output


def _attention_ref(qkv, batch, seq, heads):
    hid = heads * 128
    q, k, v = [t.float().reshape(batch, seq, heads, 128).transpose(1, 2) for t in qkv.split(hid, dim=1)]
    s = (q @ k.transpose(-1, -2)) / math.sqrt(128.0)
    return (torch.softmax(s, dim=-1) @ v).transpose(1, 2).reshape(batch * seq, hid)


@pytest.mark.parametrize("batch,seq,heads", [(1, 300, 3), (1, 1536, 24), (2, 200, 2)])
def test_attention_eight_warp_variant_matches_torch(fx, batch, seq, heads, monkeypatch):
    """FLUX_CUDA_ATTN=3 selects the variant with eight softmax warps per query tile (attention3.cu), kept for
    comparison with the default kernel (attention2.cu)."""
    monkeypatch.setenv("FLUX_CUDA_ATTN", "3")
    c3 = fx.Context(0)
    try:
        hid = heads * 128
        g = torch.Generator(device="cuda").manual_seed(seq + heads)
        qkv = torch.randn(batch * seq, 3 * hid, device="cuda", generator=g).half()
        out = torch.zeros(batch * seq, hid, device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        c3.attention(qkv.data_ptr(), batch, seq, 3 * hid, 0, hid, 2 * hid, heads, out.data_ptr(), hid, 0, f16=True)
        c3.sync()
        assert _rel(out.float(), _attention_ref(qkv, batch, seq, heads)) < 2e-3
    finally:
        c3.close()


@pytest.mark.parametrize("spec", ["1", "0"])
@pytest.mark.parametrize("profile", ["growing", "plateau", "spikes"])
def test_attention_when_the_row_maximum_moves(fx, profile, spec, monkeypatch):
    """Key tiles whose scores climb from tile to tile: the reference maximum has to be raised and the accumulator
    rescaled again and again ("growing"), the scores of the later tiles sit a few bits above the first tile's without
    reaching the rescaling threshold ("plateau"), single keys far above everything else appear late ("spikes").
    With FLUX_CUDA_ATTN_SPEC=1 (the default) the kernel takes the exponentials against the current reference first and
    falls back to the exact path when its overflow check fails; =0 is the exact path on every tile."""
    monkeypatch.setenv("FLUX_CUDA_ATTN_SPEC", spec)
    c = fx.Context(0)
    try:
        batch, seq, heads = 1, 1024, 2
        hid = heads * 128
        g = torch.Generator(device="cuda").manual_seed(7)
        q = torch.randn(seq, hid, device="cuda", generator=g)
        k = torch.randn(seq, hid, device="cuda", generator=g)
        v = torch.randn(seq, hid, device="cuda", generator=g)
        tile = torch.arange(seq, device="cuda") // 128
        if profile == "growing":
            k = k * (1.0 + 1.5 * tile)[:, None]            # the score spread grows ~2 bits per tile
        elif profile == "plateau":
            k = k * torch.where(tile == 0, 0.2, 2.5)[:, None]  # later tiles a few bits above the first, not 8
        else:
            k[700] *= 12.0
            k[1000] *= 25.0
        qkv = torch.cat([q, k, v], dim=1).half()
        out = torch.zeros(seq, hid, device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        c.attention(qkv.data_ptr(), batch, seq, 3 * hid, 0, hid, 2 * hid, heads, out.data_ptr(), hid, 0, f16=True)
        c.sync()
        assert torch.isfinite(out.float()).all()
        assert _rel(out.float(), _attention_ref(qkv, batch, seq, heads)) < 3e-3
    finally:
        c.close()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden", [(1, 256), (37, 256), (1536, 3072), (1000, 1024)])
def test_adaln_matches_torch(fx, ctx, rows, hidden, dtype):
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = torch.randn(rows, hidden, device="cuda", generator=g) * 3 + 0.5
    shift = torch.randn(hidden, device="cuda", generator=g)
    scale = torch.randn(hidden, device="cuda", generator=g)
    out = torch.zeros(rows, hidden, device="cuda", dtype=dtype)
    torch.cuda.synchronize()
    ctx.adaln(x.data_ptr(), out.data_ptr(), rows, hidden, shift.data_ptr(), scale.data_ptr(),
              f16=dtype == torch.float16)
    ctx.sync()
    ref = torch.nn.functional.layer_norm(x, (hidden,), eps=1e-6) * (1 + scale) + shift
    assert _rel(out.float(), ref) < (5e-4 if dtype == torch.float16 else 4e-3)


def test_adaln_rejects_unsupported_hidden(fx, ctx):
    x = torch.zeros(4, 384, device="cuda")
    o = torch.zeros(4, 384, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(fx.FluxCudaError):
        ctx.adaln(x.data_ptr(), o.data_ptr(), 4, 384, x.data_ptr(), x.data_ptr())


@pytest.mark.parametrize("batch,seq,heads", [(1, 48, 2), (2, 100, 3), (1, 1536, 24)])
def test_qk_norm_rope_matches_torch(fx, ctx, batch, seq, heads):
    hid = heads * 128
    g = torch.Generator(device="cuda").manual_seed(seq)
    qkv = torch.randn(batch * seq, 3 * hid, device="cuda", generator=g).to(torch.bfloat16)
    wq = torch.randn(128, device="cuda", generator=g)
    wk = torch.randn(128, device="cuda", generator=g)
    ang = torch.rand(seq, 64, device="cuda", generator=g) * 6.28
    cos = torch.cos(ang).repeat_interleave(2, dim=1).contiguous()
    sin = torch.sin(ang).repeat_interleave(2, dim=1).contiguous()
    work = qkv.clone()
    torch.cuda.synchronize()
    ctx.qk_norm_rope(work.data_ptr(), 3 * hid, 0, hid, seq, batch, heads, wq.data_ptr(), wk.data_ptr(), cos.data_ptr(),
                     sin.data_ptr())
    ctx.sync()

    def ref_one(x, w):
        x = x.float().reshape(batch, seq, heads, 128)
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w
        x0, x1 = x[..., 0::2], x[..., 1::2]
        c, s = cos[None, :, None, 0::2], sin[None, :, None, 0::2]
        return torch.stack([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1).reshape(batch * seq, hid)

    assert _rel(work[:, :hid].float(), ref_one(qkv[:, :hid], wq)) < 4e-3
    assert _rel(work[:, hid:2 * hid].float(), ref_one(qkv[:, hid:2 * hid], wk)) < 4e-3
    assert torch.equal(work[:, 2 * hid:], qkv[:, 2 * hid:])  # V untouched


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,heads,K,seq", [(100, 2, 256, 50), (1536, 24, 3072, 1536), (300, 4, 128, 300)])
def test_fused_qkv_projection_norm_rope(fx, ctx, M, heads, K, seq, dtype):
    """GEMM epilogue variant: projection + per-head RMSNorm + rotation on Q, K; V untouched."""
    hid = heads * 128
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, K, device="cuda", generator=g).to(dtype)
    w = (torch.randn(3 * hid, K, device="cuda", generator=g) * 0.05).to(dtype)  # both operands in one format
    wq = torch.randn(128, device="cuda", generator=g)
    wk = torch.randn(128, device="cuda", generator=g)
    ang = torch.rand(seq, 64, device="cuda", generator=g) * 6.28
    cos = torch.cos(ang).repeat_interleave(2, dim=1).contiguous()
    sin = torch.sin(ang).repeat_interleave(2, dim=1).contiguous()
    out = torch.zeros(M, 3 * hid, device="cuda", dtype=dtype)
    torch.cuda.synchronize()
    ctx.gemm_qkv_norm_rope(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, hid, K, wq.data_ptr(), wk.data_ptr(),
                           cos.data_ptr(), sin.data_ptr(), seq, f16=dtype == torch.float16)
    ctx.sync()
    y = x.float() @ w.float().t()
    pos = torch.arange(M, device="cuda") % seq

    def ref_one(t, wv):
        t = t.reshape(M, heads, 128)
        t = t * torch.rsqrt((t * t).mean(-1, keepdim=True) + 1e-6) * wv
        t0, t1 = t[..., 0::2], t[..., 1::2]
        c, s = cos[pos][:, None, 0::2], sin[pos][:, None, 0::2]
        return torch.stack([t0 * c - t1 * s, t1 * c + t0 * s], dim=-1).reshape(M, hid)

    tol = 5e-4 if dtype == torch.float16 else 4e-3
    assert _rel(out[:, :hid].float(), ref_one(y[:, :hid], wq)) < tol
    assert _rel(out[:, hid:2 * hid].float(), ref_one(y[:, hid:2 * hid], wk)) < tol
    assert _rel(out[:, 2 * hid:].float(), y[:, 2 * hid:]) < tol


@pytest.mark.parametrize("B,C,H,W,p", [(2, 32, 12, 8, 2), (1, 32, 64, 64, 2), (1, 3, 9, 6, 3)])
def test_patchify_round_trip_bit_exact(fx, ctx, B, C, H, W, p):
    import numpy as np
    import os
    from oracle import flux_oracle as fo
    x = torch.randn(B, C, H, W, device="cuda")
    packed = torch.zeros(B, C * p * p, H // p, W // p, device="cuda")
    back = torch.zeros_like(x)
    torch.cuda.synchronize()
    ctx.patchify(packed.data_ptr(), x.data_ptr(), B, C, H, W, p)
    ctx.unpatchify(back.data_ptr(), packed.data_ptr(), B, C, H // p, W // p, p)
    ctx.sync()
    assert np.array_equal(packed.cpu().numpy(), fo.patchify(x.cpu().numpy(), p))
    assert torch.equal(back, x)
    gold = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_patchify.npz")
    if (B, C, H, W, p) == (2, 32, 12, 8, 2) and os.path.exists(gold):
        g = np.load(gold)
        xin = torch.from_numpy(g["in"]).cuda()
        torch.cuda.synchronize()
        ctx.patchify(packed.data_ptr(), xin.data_ptr(), B, C, H, W, p)
        ctx.sync()
        assert np.array_equal(packed.cpu().numpy(), g["patchified"])
