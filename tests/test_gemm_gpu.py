"""tcgen05 GEMM (K1) against torch matmul in f32 on the same bf16 inputs, through the C ABI."""
import pytest
import torch

pytestmark = pytest.mark.gpu

# (M, N, K): the shapes one DiT step issues at 512x512 plus ragged / tiny M cases.
SHAPES = [
    (128, 256, 64),
    (128, 256, 256),
    (256, 512, 3072),
    (1536, 9216, 3072),
    (1536, 3072, 12288),
    (1024, 3072, 9216),
    (512, 3072, 7680),
    (48, 3072, 3072),      # M not a multiple of the 128-row tile
    (200, 768, 128),       # K = 128 (x_embedder), ragged M
    (1000, 128, 3072),     # N = 128 (proj_out), ragged M
]


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


def _inputs(M, N, K, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    return x, w


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_store_bf16(fx, ctx, M, N, K):
    x, w = _inputs(M, N, K)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, fx.EPI_STORE_BF16)
    ctx.sync()
    ref = x.float() @ w.float().t()
    assert torch.isfinite(out.float()).all()
    assert _rel(out.float(), ref) < 4e-3  # bf16 output rounding only


@pytest.mark.parametrize("M,N,K", [(1536, 3072, 3072), (48, 256, 128), (1000, 128, 3072)])
def test_gemm_store_f32_exact_accumulation(fx, ctx, M, N, K):
    x, w = _inputs(M, N, K, seed=1)
    out = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, fx.EPI_STORE_F32, tile_n=128 if N == 128 else 0)
    ctx.sync()
    ref = x.double() @ w.double().t()
    assert _rel(out, ref) < 1e-5  # f32 accumulation of exact bf16 products


@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_tile_widths_agree(fx, ctx, tile_n):
    M, N, K = 300, 1024, 512
    x, w = _inputs(M, N, K, seed=2)
    out = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, fx.EPI_STORE_F32, tile_n=tile_n)
    ctx.sync()
    assert _rel(out, x.double() @ w.double().t()) < 1e-5


def test_gemm_gated_residual(fx, ctx):
    M, N, K = 1536, 3072, 9216
    x, w = _inputs(M, N, K, seed=3)
    g = torch.Generator(device="cuda").manual_seed(7)
    h0 = torch.randn(M, N, device="cuda", generator=g)
    gate = torch.randn(N, device="cuda", generator=g)
    h = h0.clone()
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), h.data_ptr(), M, N, K, fx.EPI_GATED_RES_F32, gate_ptr=gate.data_ptr())
    ctx.sync()
    ref = h0.double() + gate.double() * (x.double() @ w.double().t())
    assert _rel(h, ref) < 3e-5


def test_gemm_swiglu(fx, ctx):
    M, Nh, K = 1024, 9216, 3072  # Nh output columns, 2*Nh weight rows
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    wg = (torch.randn(Nh, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(Nh, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    # library layout: per 256 weight rows, 128 gate rows then the 128 matching up rows
    w = torch.stack([wg.view(Nh // 128, 128, K), wu.view(Nh // 128, 128, K)], dim=1).reshape(2 * Nh, K).contiguous()
    out = torch.zeros(M, Nh, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, 2 * Nh, K, fx.EPI_SWIGLU_BF16)
    ctx.sync()
    ref = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    assert _rel(out.float(), ref) < 4e-3


def test_gemm_store_transposed(fx, ctx):
    M, N, K = 1000, 128, 3072
    x, w = _inputs(M, N, K, seed=6)
    out = torch.zeros(N, M, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, fx.EPI_STORE_F32_T, ld_out=M, tile_n=128)
    ctx.sync()
    assert _rel(out, (x.double() @ w.double().t()).t()) < 1e-5


def test_gemm_rejects_bad_shape(fx, ctx):
    x, w = _inputs(128, 256, 64)
    out = torch.zeros(128, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(fx.FluxCudaError):
        ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), 128, 256, 48, fx.EPI_STORE_BF16)  # K % 64 != 0


# ---- paired kernel (two CTAs per 256 x 256 tile, tcgen05 cta_group::2): tile_n = 512 selects it
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 512, 256), (1536, 9216, 3072), (1536, 3072, 12288),
                                   (48, 3072, 3072), (300, 768, 128), (129, 256, 192)])
def test_gemm_pair_store_f32(fx, ctx, M, N, K):
    x, w = _inputs(M, N, K, seed=11)
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, fx.EPI_STORE_F32, tile_n=512)
    ctx.sync()
    assert torch.isfinite(out).all()
    assert _rel(out, x.double() @ w.double().t()) < 3e-5


def test_gemm_pair_agrees_with_single_cta_kernel(fx, ctx):
    M, N, K = 1000, 2048, 1024
    x, w = _inputs(M, N, K, seed=12)
    a = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), a.data_ptr(), M, N, K, fx.EPI_STORE_BF16, tile_n=256)
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), b.data_ptr(), M, N, K, fx.EPI_STORE_BF16, tile_n=512)
    ctx.sync()
    assert torch.equal(a, b)  # same k order, same accumulation: bit-identical


def test_gemm_pair_swiglu_and_gated(fx, ctx):
    M, Nh, K = 1024, 1024, 512
    g = torch.Generator(device="cuda").manual_seed(13)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    wg = (torch.randn(Nh, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(Nh, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    w = torch.stack([wg.view(Nh // 128, 128, K), wu.view(Nh // 128, 128, K)], dim=1).reshape(2 * Nh, K).contiguous()
    out = torch.zeros(M, Nh, device="cuda", dtype=torch.bfloat16)
    h0 = torch.randn(M, Nh, device="cuda", generator=g)
    gate = torch.randn(Nh, device="cuda", generator=g)
    h = h0.clone()
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, 2 * Nh, K, fx.EPI_SWIGLU_BF16, tile_n=512)
    ctx.gemm_bf16(x.data_ptr(), wg.data_ptr(), h.data_ptr(), M, Nh, K, fx.EPI_GATED_RES_F32, gate_ptr=gate.data_ptr(),
                  tile_n=512)
    ctx.sync()
    ref = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    assert _rel(out.float(), ref) < 4e-3
    assert _rel(h, h0.double() + gate.double() * (x.double() @ wg.double().t())) < 3e-5


# ---- f16 operands (what the engine runs by default): same kernels, other operand format.
# tcgen05 kind::f16 wants both operands in ONE format: an f16 x bf16 descriptor is an illegal instruction.
@pytest.mark.parametrize("tile_n", [256, 512, 128])
@pytest.mark.parametrize("M,N,K", [(1536, 3072, 3072), (200, 768, 128)])
def test_gemm_f16_operands(fx, ctx, M, N, K, tile_n):
    g = torch.Generator(device="cuda").manual_seed(21)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.float16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.float16)
    out32 = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    out16 = torch.zeros(M, N, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out32.data_ptr(), M, N, K, fx.EPI_STORE_F32 | fx.EPI_X_F16, tile_n=tile_n)
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out16.data_ptr(), M, N, K,
                  fx.EPI_STORE_BF16 | fx.EPI_X_F16 | fx.EPI_OUT_F16, tile_n=tile_n)
    ctx.sync()
    ref = x.double() @ w.double().t()
    assert _rel(out32, ref) < 3e-5
    assert _rel(out16.float(), ref) < 5e-4  # f16 output rounding


def test_gemm_f16_output_saturates_instead_of_overflowing(fx, ctx):
    M, N, K = 128, 256, 64
    x = torch.full((M, K), 200.0, device="cuda", dtype=torch.float16)
    w = torch.full((N, K), 8.0, device="cuda", dtype=torch.float16)
    out = torch.zeros(M, N, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, fx.EPI_STORE_BF16 | fx.EPI_X_F16 | fx.EPI_OUT_F16)
    ctx.sync()
    assert torch.isfinite(out).all() and (out == 65504).all()  # 200 * 8 * 64 = 102400 > f16 max
