"""The error and range reports of the library, provoked without harming the device: a bounded wait that is meant to
run out (a one-warp kernel waiting on a barrier nobody arrives on, with a millisecond limit) and f16 stores that are
meant to clamp. Neither traps, faults or hangs anything; both must leave the context usable."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _gemm_ok(fx, ctx):
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.randn(256, 128, device="cuda", generator=g)).half()
    w = (torch.randn(256, 128, device="cuda", generator=g) * 0.1).half()
    out = torch.zeros(256, 256, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), 256, 256, 128,
                  fx.EPI_STORE_F32 | fx.EPI_X_F16 | fx.EPI_OUT_F16)
    ctx.sync()
    want = x.float() @ w.float().t()
    assert ((out - want).norm() / want.norm()).item() < 1e-5


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(fx, ctx):
    ctx.sync()
    waited = torch.zeros(1, device="cuda", dtype=torch.int64)
    torch.cuda.synchronize()
    limit = 2_000_000  # about a millisecond of SM clock
    ctx.selftest_wait_timeout(limit, waited.data_ptr())
    with pytest.raises(fx.FluxCudaError, match="bounded wait .code 7."):
        ctx.sync()
    # the wait really ran to its limit, and not far beyond it
    assert limit <= int(waited.item()) < 20 * limit
    ctx.sync()  # the error word was cleared by the report
    _gemm_ok(fx, ctx)
    with pytest.raises(fx.FluxCudaError):
        ctx.selftest_wait_timeout(0)
    with pytest.raises(fx.FluxCudaError):
        ctx.selftest_wait_timeout(3_000_000_000)


def test_saturating_f16_stores_are_counted(fx, ctx):
    ctx.sync()
    ctx.saturated_stores(reset=True)
    _gemm_ok(fx, ctx)
    assert ctx.saturated_stores() == 0
    # 128 products of 60 * 60 per output element = 460800: far outside the f16 range, so every store clamps
    x = torch.full((256, 128), 60.0, device="cuda").half()
    w = torch.full((256, 128), 60.0, device="cuda").half()
    out = torch.zeros(256, 256, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    ctx.gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), 256, 256, 128,
                  fx.EPI_STORE_BF16 | fx.EPI_X_F16 | fx.EPI_OUT_F16)
    ctx.sync()
    assert torch.all(out == 65504.0)  # clamped, not infinite
    n = ctx.saturated_stores(reset=True)
    assert n >= 256  # at least one count per output row (one thread per row and tile)
    assert ctx.saturated_stores() == 0
    # the same product stored as bf16 is in range: nothing to count
    xb, wb = x.bfloat16(), w.bfloat16()
    outb = torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ctx.gemm_bf16(xb.data_ptr(), wb.data_ptr(), outb.data_ptr(), 256, 256, 128, fx.EPI_STORE_BF16)
    ctx.sync()
    assert ctx.saturated_stores() == 0 and torch.all(outb.float() == 460800.0)
