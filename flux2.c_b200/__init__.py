"""Host-side Python binding of the B200 denoising engine (ctypes over the C ABI in include/flux_cuda.h).

The directory name contains a dot, so it is not importable with a plain ``import``; load it with
``importlib`` (see ``load_package`` in ``__graft_entry__.py``) under the module name ``flux2_c_b200``.

Everything here calls into ``libflux_cuda.so``; when that library is missing or no B200 is
visible the calls raise — there is no CPU implementation behind this module.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflux_cuda.so")

EPI_STORE_BF16, EPI_STORE_F32, EPI_GATED_RES_F32, EPI_SWIGLU_BF16, EPI_STORE_F32_T = range(5)

_lib = None


class FluxCudaError(RuntimeError):
    pass


def lib():
    """Returns the loaded C library (ctypes.CDLL), loading it on first use."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FluxCudaError(
                "%s is missing: build it with `python flux2.c_b200/build.py` (needs nvcc)" % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(L):
    c_void_p, c_int, c_ll, c_char_p = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_char_p
    L.flux_cuda_last_error.restype = c_char_p
    L.flux_cuda_last_error.argtypes = []
    L.flux_cuda_ctx_create.restype = c_int
    L.flux_cuda_ctx_create.argtypes = [c_int, ctypes.POINTER(c_void_p)]
    L.flux_cuda_ctx_destroy.restype = None
    L.flux_cuda_ctx_destroy.argtypes = [c_void_p]
    L.flux_cuda_ctx_sync.restype = c_int
    L.flux_cuda_ctx_sync.argtypes = [c_void_p]
    L.flux_cuda_ctx_stream.restype = c_void_p
    L.flux_cuda_ctx_stream.argtypes = [c_void_p]
    L.flux_cuda_gemm_bf16.restype = c_int
    L.flux_cuda_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll,
                                      c_void_p, c_int]


def check(rc):
    if rc != 0:
        raise FluxCudaError("flux_cuda error %d: %s" % (rc, lib().flux_cuda_last_error().decode()))


class Context:
    """One per GPU. Mirrors flux_cuda_ctx_create / _destroy / _sync."""

    def __init__(self, device=0):
        self.handle = ctypes.c_void_p()
        check(lib().flux_cuda_ctx_create(device, ctypes.byref(self.handle)))
        self.device = device

    def sync(self):
        check(lib().flux_cuda_ctx_sync(self.handle))

    @property
    def stream(self):
        return lib().flux_cuda_ctx_stream(self.handle)

    def close(self):
        if self.handle:
            lib().flux_cuda_ctx_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- kernel-level entry points (device pointers as ints) ----
    def gemm_bf16(self, x_ptr, w_ptr, out_ptr, M, N, K, epilogue=EPI_STORE_BF16, ld_out=None, gate_ptr=None,
                  tile_n=0):
        if ld_out is None:
            ld_out = N // 2 if epilogue == EPI_SWIGLU_BF16 else N
        check(lib().flux_cuda_gemm_bf16(self.handle, x_ptr, w_ptr, out_ptr, M, N, K, epilogue, ld_out, gate_ptr,
                                        tile_n))
