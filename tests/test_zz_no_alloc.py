"""flux_cuda_group_norm_noalloc (scratch inside the library image, no allocation) against flux_cuda_group_norm, through
the C ABI, on two calls in a row. Collected last on purpose: it must hold both on a fresh context and after every other
test has used the device."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("in16", [False, True])
@pytest.mark.parametrize("n,pixels,C,swish", [(1, 4096, 512, True), (2, 1000, 256, False), (4, 333, 128, True),
                                              (1, 65536, 128, True)])
def test_noalloc_group_norm_equals_the_allocating_entry_point(fx, ctx, n, pixels, C, swish, in16):
    g = torch.Generator(device="cuda").manual_seed(n * 7 + C)
    x = torch.randn(n, pixels, C, device="cuda", generator=g) * 1.5 - 0.3
    if in16:
        x = x.half()
    gamma = 1 + 0.3 * torch.randn(C, device="cuda", generator=g)
    beta = 0.2 * torch.randn(C, device="cuda", generator=g)
    want = torch.zeros(n, pixels, C, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    ctx.group_norm(x.data_ptr(), in16, want.data_ptr(), n, pixels, C, gamma.data_ptr(), beta.data_ptr(), 1e-4, swish)
    ctx.sync()
    ref = torch.nn.functional.group_norm(x.float().permute(0, 2, 1), 32, gamma, beta, eps=1e-4).permute(0, 2, 1)
    if swish:
        ref = torch.nn.functional.silu(ref)
    for call in range(2):
        got = torch.full((n, pixels, C), float("nan"), device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        ctx.group_norm_noalloc(x.data_ptr(), in16, got.data_ptr(), n, pixels, C, gamma.data_ptr(), beta.data_ptr(), 1e-4,
                               swish)
        ctx.sync()
        if call == 1:
            # the array's module was loaded by the first call at the latest: this one takes nothing from the device
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after == free_before, "the second call changed the free device memory"
        assert torch.equal(got, want), "call %d differs from flux_cuda_group_norm" % call
        err = (got.float().double() - ref.double()).norm() / ref.double().norm()
        assert err.item() < 6e-4


def test_noalloc_group_norm_rejects_what_does_not_fit(fx, ctx):
    x = torch.zeros(5, 8, 128, device="cuda")
    o = torch.zeros(5, 8, 128, device="cuda", dtype=torch.float16)
    w = torch.ones(128, device="cuda")
    with pytest.raises(fx.FluxCudaError, match="at most 4"):
        ctx.group_norm_noalloc(x.data_ptr(), False, o.data_ptr(), 5, 8, 128, w.data_ptr(), w.data_ptr(), 1e-4, False)
    with pytest.raises(fx.FluxCudaError):
        ctx.group_norm_noalloc(x.data_ptr(), False, o.data_ptr(), 1, 8, 96, w.data_ptr(), w.data_ptr(), 1e-4, False)
    # a pointer that is not 16-byte aligned is refused on the host, before anything is launched
    for entry in (ctx.group_norm_noalloc, ctx.group_norm):
        with pytest.raises(fx.FluxCudaError, match="16-byte aligned"):
            entry(x.data_ptr() + 4, False, o.data_ptr(), 1, 8, 128, w.data_ptr(), w.data_ptr(), 1e-4, False)
    ctx.sync()
