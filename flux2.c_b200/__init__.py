"""Host-side Python binding of the B200 denoising engine (ctypes over the C ABI in include/flux_cuda.h).

The directory name contains a dot, so it is not importable with a plain ``import``; load it with
``importlib`` (see ``load_package`` in ``__graft_entry__.py``) under the module name ``flux2_c_b200``.

Everything here calls into ``libflux_cuda.so``; when that library is missing or no B200 is
visible the calls raise — there is no CPU implementation behind this module.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FLUX_CUDA_LIBRARY selects another build of the same library, e.g. the checked one (libflux_cuda_debug.so)
LIB_PATH = os.environ.get("FLUX_CUDA_LIBRARY") or os.path.join(_HERE, "libflux_cuda.so")

EPI_STORE_BF16, EPI_STORE_F32, EPI_GATED_RES_F32, EPI_SWIGLU_BF16, EPI_STORE_F32_T = range(5)
EPI_X_F16, EPI_OUT_F16 = 0x100, 0x200  # or-ed into the epilogue: f16 activations in / out

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
    L.flux_cuda_build_checked.restype = c_int
    L.flux_cuda_build_checked.argtypes = []
    L.flux_cuda_ctx_create.restype = c_int
    L.flux_cuda_ctx_create.argtypes = [c_int, ctypes.POINTER(c_void_p)]
    L.flux_cuda_ctx_destroy.restype = None
    L.flux_cuda_ctx_destroy.argtypes = [c_void_p]
    L.flux_cuda_ctx_sync.restype = c_int
    L.flux_cuda_ctx_sync.argtypes = [c_void_p]
    L.flux_cuda_ctx_stream.restype = c_void_p
    L.flux_cuda_ctx_stream.argtypes = [c_void_p]
    L.flux_cuda_ctx_set_half_format.restype = c_int
    L.flux_cuda_ctx_set_half_format.argtypes = [c_void_p, c_int]
    L.flux_cuda_ctx_set_gemm_pair.restype = c_int
    L.flux_cuda_ctx_set_gemm_pair.argtypes = [c_void_p, c_int]
    L.flux_cuda_gemm_bf16.restype = c_int
    L.flux_cuda_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll,
                                      c_void_p, c_int]


    fp = ctypes.POINTER(ctypes.c_float)
    L.flux_cuda_gemm_qkv_norm_rope.restype = c_int
    L.flux_cuda_gemm_qkv_norm_rope.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_int, c_int]
    L.flux_cuda_attention.restype = c_int
    L.flux_cuda_attention.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_int, c_int, c_int, c_int, c_void_p,
                                      c_ll, c_int, c_int]
    L.flux_cuda_adaln.restype = c_int
    L.flux_cuda_adaln.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int]
    L.flux_cuda_qk_norm_rope.restype = c_int
    L.flux_cuda_qk_norm_rope.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                         c_void_p, c_void_p, c_void_p]
    L.flux_cuda_qwen3_create.restype = c_int
    L.flux_cuda_qwen3_create.argtypes = [c_void_p, ctypes.POINTER(CQwenDims), c_int, ctypes.POINTER(c_void_p)]
    L.flux_cuda_qwen3_load_dir.restype = c_int
    L.flux_cuda_qwen3_load_dir.argtypes = [c_void_p, c_char_p, c_int, ctypes.POINTER(c_void_p)]
    L.flux_cuda_qwen3_set_tensor.restype = c_int
    L.flux_cuda_qwen3_set_tensor.argtypes = [c_void_p, c_char_p, c_void_p, c_int, ctypes.POINTER(c_ll), c_int]
    L.flux_cuda_qwen3_finalize.restype = c_int
    L.flux_cuda_qwen3_finalize.argtypes = [c_void_p]
    L.flux_cuda_qwen3_free.restype = None
    L.flux_cuda_qwen3_free.argtypes = [c_void_p]
    L.flux_cuda_qwen3_forward.restype = c_int
    L.flux_cuda_qwen3_forward.argtypes = [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_int, fp]
    L.flux_cuda_vae_load_safetensors.restype = c_int
    L.flux_cuda_vae_load_safetensors.argtypes = [c_void_p, ctypes.c_char_p, ctypes.POINTER(c_void_p)]
    L.flux_cuda_vae_create.restype = c_int
    L.flux_cuda_vae_create.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
    L.flux_cuda_vae_set_tensor.restype = c_int
    L.flux_cuda_vae_set_tensor.argtypes = [c_void_p, ctypes.c_char_p, c_void_p, c_int, ctypes.POINTER(ctypes.c_longlong),
                                           c_int]
    L.flux_cuda_vae_finalize.restype = c_int
    L.flux_cuda_vae_finalize.argtypes = [c_void_p]
    L.flux_cuda_vae_free.restype = None
    L.flux_cuda_vae_free.argtypes = [c_void_p]
    L.flux_cuda_vae_decode.restype = c_int
    L.flux_cuda_vae_decode.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p]
    L.flux_cuda_vae_decode_device.restype = c_int
    L.flux_cuda_vae_decode_device.argtypes = [c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(c_void_p)]
    L.flux_cuda_vae_encode.restype = c_int
    L.flux_cuda_vae_encode.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p]
    L.flux_cuda_vae_has_encoder.restype = c_int
    L.flux_cuda_vae_has_encoder.argtypes = [c_void_p]
    L.flux_cuda_vae_last_launches.restype = ctypes.c_longlong
    L.flux_cuda_vae_last_launches.argtypes = [c_void_p]
    L.flux_cuda_sampler_latent_device.restype = c_int
    L.flux_cuda_sampler_latent_device.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
    L.flux_cuda_conv3x3.restype = c_int
    L.flux_cuda_conv3x3.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                    c_void_p, ctypes.c_longlong, c_int]
    L.flux_cuda_conv3x3_stride2.restype = c_int
    L.flux_cuda_conv3x3_stride2.argtypes = L.flux_cuda_conv3x3.argtypes
    L.flux_cuda_gemm_bias.restype = c_int
    L.flux_cuda_gemm_bias.argtypes = [c_void_p, c_void_p, ctypes.c_longlong, c_void_p, ctypes.c_longlong, c_int, c_int,
                                      c_int, c_int, c_void_p, c_int, c_void_p, ctypes.c_longlong, c_int]
    L.flux_cuda_group_norm.restype = c_int
    L.flux_cuda_group_norm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, ctypes.c_longlong, c_int, c_void_p,
                                       c_void_p, ctypes.c_float, c_int, c_int]
    L.flux_cuda_group_norm_noalloc.restype = c_int
    L.flux_cuda_group_norm_noalloc.argtypes = L.flux_cuda_group_norm.argtypes
    L.flux_cuda_qwen3_forward_batch.restype = c_int
    L.flux_cuda_qwen3_forward_batch.argtypes = [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_int, c_int, fp]
    L.flux_cuda_qwen3_forward_batch_device.restype = c_int
    L.flux_cuda_qwen3_forward_batch_device.argtypes = [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_int, c_int,
                                                       ctypes.POINTER(c_void_p)]
    L.flux_cuda_qwen3_forward_device.restype = c_int
    L.flux_cuda_qwen3_forward_device.argtypes = [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), c_int,
                                                 ctypes.POINTER(c_void_p)]
    L.flux_cuda_patchify.restype = c_int
    L.flux_cuda_patchify.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]
    L.flux_cuda_unpatchify.restype = c_int
    L.flux_cuda_unpatchify.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]
    L.flux_cuda_dims_klein4b.restype = None
    L.flux_cuda_dims_klein4b.argtypes = [ctypes.POINTER(CDims)]
    L.flux_cuda_model_load_safetensors.restype = c_int
    L.flux_cuda_model_load_safetensors.argtypes = [c_void_p, c_char_p, ctypes.POINTER(c_void_p)]
    L.flux_cuda_model_create.restype = c_int
    L.flux_cuda_model_create.argtypes = [c_void_p, ctypes.POINTER(CDims), ctypes.POINTER(c_void_p)]
    L.flux_cuda_model_set_tensor.restype = c_int
    L.flux_cuda_model_set_tensor.argtypes = [c_void_p, c_char_p, c_void_p, c_int, ctypes.POINTER(c_ll), c_int]
    L.flux_cuda_model_finalize.restype = c_int
    L.flux_cuda_model_finalize.argtypes = [c_void_p]
    L.flux_cuda_model_free.restype = None
    L.flux_cuda_model_free.argtypes = [c_void_p]
    L.flux_cuda_model_dims.restype = c_int
    L.flux_cuda_model_dims.argtypes = [c_void_p, ctypes.POINTER(CDims)]
    L.flux_cuda_forward.restype = c_int
    L.flux_cuda_forward.argtypes = [c_void_p, fp, c_int, c_int, ctypes.POINTER(CRef), c_int, fp, c_int,
                                    ctypes.c_float, fp]
    L.flux_cuda_sample.restype = c_int
    L.flux_cuda_sample.argtypes = [c_void_p, ctypes.POINTER(CSampleParams), fp, fp, fp]
    L.flux_cuda_sampler_create.restype = c_int
    L.flux_cuda_sampler_create.argtypes = [c_void_p, c_int, c_int, c_int, ctypes.POINTER(CRefShape), c_int, c_int,
                                           c_int, ctypes.POINTER(c_void_p)]
    L.flux_cuda_sampler_free.restype = None
    L.flux_cuda_sampler_free.argtypes = [c_void_p]
    L.flux_cuda_sampler_upload.restype = c_int
    L.flux_cuda_sampler_upload.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p)]
    L.flux_cuda_sampler_run.restype = c_int
    L.flux_cuda_sampler_run.argtypes = [c_void_p, fp, c_int, ctypes.c_float, c_int, c_int]
    L.flux_cuda_sampler_run_steps.restype = c_int
    L.flux_cuda_sampler_run_steps.argtypes = [c_void_p, fp, c_int, c_int, c_int, ctypes.c_float, c_int]
    L.flux_cuda_sampler_predict.restype = c_int
    L.flux_cuda_sampler_predict.argtypes = [c_void_p, fp, c_int, c_int]
    L.flux_cuda_sampler_velocity.restype = c_int
    L.flux_cuda_sampler_velocity.argtypes = [c_void_p, c_void_p, ctypes.c_float]
    L.flux_cuda_sampler_apply_velocity.restype = c_int
    L.flux_cuda_sampler_apply_velocity.argtypes = [c_void_p, c_void_p, c_int]
    L.flux_cuda_sampler_download.restype = c_int
    L.flux_cuda_sampler_download.argtypes = [c_void_p, c_void_p, c_void_p]
    L.flux_cuda_sampler_stage_inputs.restype = c_int
    L.flux_cuda_sampler_stage_inputs.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p)]
    L.flux_cuda_sampler_download_async.restype = c_int
    L.flux_cuda_sampler_download_async.argtypes = [c_void_p, c_void_p]
    L.flux_cuda_sampler_last_run.restype = c_int
    L.flux_cuda_sampler_last_run.argtypes = [c_void_p, fp, ctypes.POINTER(c_ll)]
    L.flux_cuda_sampler_set_profiling.restype = c_int
    L.flux_cuda_sampler_set_profiling.argtypes = [c_void_p, c_int]
    L.flux_cuda_sampler_profile.restype = c_int
    L.flux_cuda_sampler_profile.argtypes = [c_void_p, fp, ctypes.POINTER(c_ll)]
    L.flux_cuda_sampler_profile_groups.restype = c_int
    L.flux_cuda_sampler_profile_groups.argtypes = [c_void_p, fp]
    L.flux_cuda_sampler_profile_launches.restype = c_int
    L.flux_cuda_sampler_profile_launches.argtypes = [c_void_p, fp, ctypes.POINTER(c_int), c_int, ctypes.POINTER(c_int)]
    L.flux_cuda_ctx_set_gemm_trace.restype = c_int
    L.flux_cuda_ctx_set_gemm_trace.argtypes = [c_void_p, c_void_p]
    L.flux_cuda_ctx_saturated_stores.restype = c_int
    L.flux_cuda_ctx_saturated_stores.argtypes = [c_void_p, ctypes.POINTER(c_ll), c_int]
    L.flux_cuda_selftest_wait_timeout.restype = c_int
    L.flux_cuda_selftest_wait_timeout.argtypes = [c_void_p, c_ll, c_void_p]
    L.flux_cuda_group_create.restype = c_int
    L.flux_cuda_group_create.argtypes = [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_void_p)]
    L.flux_cuda_group_destroy.restype = None
    L.flux_cuda_group_destroy.argtypes = [c_void_p]
    L.flux_cuda_group_size.restype = c_int
    L.flux_cuda_group_size.argtypes = [c_void_p]
    L.flux_cuda_group_context.restype = c_void_p
    L.flux_cuda_group_context.argtypes = [c_void_p, c_int]
    L.flux_cuda_group_load_safetensors.restype = c_int
    L.flux_cuda_group_load_safetensors.argtypes = [c_void_p, c_char_p]
    L.flux_cuda_group_set_models.restype = c_int
    L.flux_cuda_group_set_models.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
    L.flux_cuda_group_sample_batch.restype = c_int
    L.flux_cuda_group_sample_batch.argtypes = [c_void_p, ctypes.POINTER(CSampleParams), c_int, ctypes.POINTER(fp),
                                               ctypes.POINTER(fp), ctypes.POINTER(fp)]
    L.flux_cuda_group_sample_cfg_pair.restype = c_int
    L.flux_cuda_group_sample_cfg_pair.argtypes = [c_void_p, ctypes.POINTER(CSampleParams), fp, fp]
    L.flux_cuda_rendezvous_create.restype = c_int
    L.flux_cuda_rendezvous_create.argtypes = [c_int, ctypes.POINTER(c_void_p)]
    L.flux_cuda_rendezvous_destroy.restype = None
    L.flux_cuda_rendezvous_destroy.argtypes = [c_void_p]
    L.flux_cuda_rendezvous_arrive_and_wait.restype = c_int
    L.flux_cuda_rendezvous_arrive_and_wait.argtypes = [c_void_p, c_int, c_ll, c_int]
    L.flux_cuda_rendezvous_abandon.restype = None
    L.flux_cuda_rendezvous_abandon.argtypes = [c_void_p, c_int]
    L.flux_cuda_official_schedule.restype = None
    L.flux_cuda_official_schedule.argtypes = [c_int, c_int, fp]
    L.flux_cuda_linear_schedule.restype = None
    L.flux_cuda_linear_schedule.argtypes = [c_int, fp]
    L.flux_cuda_power_schedule.restype = None
    L.flux_cuda_power_schedule.argtypes = [c_int, ctypes.c_float, fp]
    L.flux_cuda_init_noise.restype = None
    L.flux_cuda_init_noise.argtypes = [c_int, c_int, c_int, c_ll, fp]


class CDims(ctypes.Structure):  # flux_cuda_dims
    _fields_ = [(n, ctypes.c_int) for n in ("hidden", "heads", "head_dim", "mlp", "n_double", "n_single", "text_dim",
                                            "latent_ch", "time_dim")] + [("rope_theta", ctypes.c_float),
                                                                         ("axis_dim", ctypes.c_int)]


class CQwenDims(ctypes.Structure):  # flux_cuda_qwen3_dims
    _fields_ = [(n, ctypes.c_int) for n in ("hidden", "heads", "kv_heads", "head_dim", "inter", "layers", "vocab")] + [
        ("rope_theta", ctypes.c_float), ("out_layers", ctypes.c_int * 3)]


class CRef(ctypes.Structure):  # flux_cuda_ref
    _fields_ = [("latent", ctypes.POINTER(ctypes.c_float)), ("h", ctypes.c_int), ("w", ctypes.c_int),
                ("t_offset", ctypes.c_int)]


class CRefShape(ctypes.Structure):  # flux_cuda_ref_shape
    _fields_ = [("h", ctypes.c_int), ("w", ctypes.c_int), ("t_offset", ctypes.c_int)]


class CSampleParams(ctypes.Structure):  # flux_cuda_sample_params
    _fields_ = [("h", ctypes.c_int), ("w", ctypes.c_int), ("num_steps", ctypes.c_int),
                ("schedule", ctypes.POINTER(ctypes.c_float)), ("ctx", ctypes.POINTER(ctypes.c_float)),
                ("ctx_uncond", ctypes.POINTER(ctypes.c_float)), ("txt_seq", ctypes.c_int),
                ("guidance", ctypes.c_float), ("refs", ctypes.POINTER(CRef)), ("num_refs", ctypes.c_int)]


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

    def saturated_stores(self, reset=False):
        """f16 stores that hit the +-65504 clamp, as seen by the synchronising calls so far."""
        n = ctypes.c_longlong()
        check(lib().flux_cuda_ctx_saturated_stores(self.handle, ctypes.byref(n), int(reset)))
        return n.value

    def selftest_wait_timeout(self, limit_cycles, waited_ptr=None):
        check(lib().flux_cuda_selftest_wait_timeout(self.handle, limit_cycles, waited_ptr))

    def set_half_format(self, name):
        """'f16' (default) or 'bf16': storage format of models created afterwards."""
        check(lib().flux_cuda_ctx_set_half_format(self.handle, {"f16": 1, "bf16": 2}[name]))

    def set_gemm_trace(self, stamps_ptr):
        check(lib().flux_cuda_ctx_set_gemm_trace(self.handle, stamps_ptr))

    def set_gemm_pair(self, on):
        check(lib().flux_cuda_ctx_set_gemm_pair(self.handle, int(on)))

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
            ld_out = N // 2 if (epilogue & 0xFF) == EPI_SWIGLU_BF16 else N
        check(lib().flux_cuda_gemm_bf16(self.handle, x_ptr, w_ptr, out_ptr, M, N, K, epilogue, ld_out, gate_ptr,
                                        tile_n))

    def gemm_qkv_norm_rope(self, x_ptr, w_ptr, out_ptr, M, hidden, K, wq_ptr, wk_ptr, cos_ptr, sin_ptr, seq,
                           f16=False):
        check(lib().flux_cuda_gemm_qkv_norm_rope(self.handle, x_ptr, w_ptr, out_ptr, M, hidden, K, wq_ptr, wk_ptr,
                                                 cos_ptr, sin_ptr, seq, int(f16)))

    def attention(self, qkv_ptr, batch, seq, ld, q_col, k_col, v_col, heads, out_ptr, out_ld, out_col=0, f16=False):
        check(lib().flux_cuda_attention(self.handle, qkv_ptr, batch, seq, ld, q_col, k_col, v_col, heads, out_ptr,
                                        out_ld, out_col, int(f16)))

    def adaln(self, x_ptr, out_ptr, rows, hidden, shift_ptr, scale_ptr, f16=False):
        check(lib().flux_cuda_adaln(self.handle, x_ptr, out_ptr, rows, hidden, shift_ptr, scale_ptr, int(f16)))

    def conv3x3(self, x_ptr, n_img, H, W, cin, w_ptr, cout, bias_ptr, mode, out_ptr, ld, f16=True, stride2=False):
        fn = lib().flux_cuda_conv3x3_stride2 if stride2 else lib().flux_cuda_conv3x3
        check(fn(self.handle, x_ptr, n_img, H, W, cin, w_ptr, cout, bias_ptr, mode, out_ptr, ld, int(f16)))

    def gemm_bias(self, x_ptr, ldx, w_ptr, ldw, M, N, K, bias_ptr, mode, out_ptr, ld, w_rows=None, f16=True):
        check(lib().flux_cuda_gemm_bias(self.handle, x_ptr, ldx, w_ptr, ldw, M, N, K, N if w_rows is None else w_rows,
                                        bias_ptr, mode, out_ptr, ld, int(f16)))

    def group_norm(self, x_ptr, in16, out_ptr, n_img, pixels, C, gamma_ptr, beta_ptr, eps, swish, f16=True):
        check(lib().flux_cuda_group_norm(self.handle, x_ptr, int(in16), out_ptr, n_img, pixels, C, gamma_ptr, beta_ptr,
                                         eps, int(swish), int(f16)))

    def group_norm_noalloc(self, x_ptr, in16, out_ptr, n_img, pixels, C, gamma_ptr, beta_ptr, eps, swish, f16=True):
        check(lib().flux_cuda_group_norm_noalloc(self.handle, x_ptr, int(in16), out_ptr, n_img, pixels, C, gamma_ptr,
                                                 beta_ptr, eps, int(swish), int(f16)))

    def patchify(self, out_ptr, in_ptr, batch, channels, H, W, patch):
        check(lib().flux_cuda_patchify(self.handle, out_ptr, in_ptr, batch, channels, H, W, patch))

    def unpatchify(self, out_ptr, in_ptr, batch, channels, H, W, patch):
        check(lib().flux_cuda_unpatchify(self.handle, out_ptr, in_ptr, batch, channels, H, W, patch))

    def qk_norm_rope(self, qkv_ptr, ld, q_col, k_col, seq, batch, heads, wq_ptr, wk_ptr, cos_ptr, sin_ptr):
        check(lib().flux_cuda_qk_norm_rope(self.handle, qkv_ptr, ld, q_col, k_col, seq, batch, heads, wq_ptr, wk_ptr,
                                           cos_ptr, sin_ptr))


# ------------------------------------------------------------------------------------------------ host helpers
def _np():
    import numpy as np
    return np


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def official_schedule(num_steps, image_seq_len):
    """flux_official_schedule: num_steps + 1 timesteps from 1 to 0 (computed by the C library's host code)."""
    np = _np()
    out = np.zeros(num_steps + 1, dtype=np.float32)
    lib().flux_cuda_official_schedule(num_steps, image_seq_len, _fp(out))
    return out


def linear_schedule(num_steps):
    np = _np()
    out = np.zeros(num_steps + 1, dtype=np.float32)
    lib().flux_cuda_linear_schedule(num_steps, _fp(out))
    return out


def power_schedule(num_steps, alpha):
    np = _np()
    out = np.zeros(num_steps + 1, dtype=np.float32)
    lib().flux_cuda_power_schedule(num_steps, alpha, _fp(out))
    return out


def init_noise(channels, h, w, seed):
    """flux_init_noise: the reference's size-independent seeded noise, f32 [channels, h, w]."""
    np = _np()
    out = np.zeros((channels, h, w), dtype=np.float32)
    lib().flux_cuda_init_noise(channels, h, w, seed, _fp(out))
    return out


_DTYPES = {"float32": 0, "float16": 1, "uint16": 2}  # uint16 arrays carry bf16 bit patterns


class Model:
    """The DiT on one GPU. Mirrors flux_transformer_load_safetensors / flux_transformer_forward* / flux_sample_euler*."""

    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle

    @staticmethod
    def load_safetensors(ctx, path):
        h = ctypes.c_void_p()
        check(lib().flux_cuda_model_load_safetensors(ctx.handle, path.encode(), ctypes.byref(h)))
        return Model(ctx, h)

    @staticmethod
    def from_tensors(ctx, dims, tensors):
        """dims: object with the fields of flux_cuda_dims; tensors: name -> numpy array (uint16 = bf16 bits)."""
        cd = CDims()
        for name, _ in CDims._fields_:
            setattr(cd, name, getattr(dims, name))
        h = ctypes.c_void_p()
        check(lib().flux_cuda_model_create(ctx.handle, ctypes.byref(cd), ctypes.byref(h)))
        m = Model(ctx, h)
        np = _np()
        for name, arr in tensors.items():
            arr = np.ascontiguousarray(arr)
            shape = (ctypes.c_longlong * arr.ndim)(*arr.shape)
            check(lib().flux_cuda_model_set_tensor(h, name.encode(), arr.ctypes.data, _DTYPES[str(arr.dtype)], shape,
                                                   arr.ndim))
        check(lib().flux_cuda_model_finalize(h))
        return m

    def dims(self):
        cd = CDims()
        check(lib().flux_cuda_model_dims(self.handle, ctypes.byref(cd)))
        return cd

    @staticmethod
    def _refs(refs):
        np = _np()
        keep = [np.ascontiguousarray(lat, dtype=np.float32) for lat, _ in refs]
        arr = (CRef * max(1, len(refs)))()
        for i, (lat, toff) in enumerate(refs):
            arr[i].latent = _fp(keep[i])
            arr[i].h, arr[i].w, arr[i].t_offset = keep[i].shape[1], keep[i].shape[2], toff
        return arr, keep

    def forward(self, z, h, w, ctx_emb, t, refs=()):
        """Velocity [C, h, w] for latent z at timestep t; refs = [(latent [C, rh, rw], t_offset), ...]."""
        np = _np()
        z = np.ascontiguousarray(z, dtype=np.float32)
        ctx_emb = np.ascontiguousarray(ctx_emb, dtype=np.float32)
        out = np.empty_like(z)
        arr, keep = self._refs(refs)
        check(lib().flux_cuda_forward(self.handle, _fp(z), h, w, arr, len(refs), _fp(ctx_emb), ctx_emb.shape[0], t,
                                      _fp(out)))
        return out

    def sample(self, z0, h, w, ctx_emb, schedule, ctx_uncond=None, guidance=1.0, refs=(), return_velocities=False):
        """Euler loop on the device; with ctx_uncond the guidance pair runs as a batch of two."""
        np = _np()
        z0 = np.ascontiguousarray(z0, dtype=np.float32)
        ctx_emb = np.ascontiguousarray(ctx_emb, dtype=np.float32)
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        steps = len(sch) - 1
        p = CSampleParams()
        p.h, p.w, p.num_steps, p.schedule, p.ctx, p.txt_seq = h, w, steps, _fp(sch), _fp(ctx_emb), ctx_emb.shape[0]
        if ctx_uncond is not None:
            ctx_uncond = np.ascontiguousarray(ctx_uncond, dtype=np.float32)
            p.ctx_uncond = _fp(ctx_uncond)
        p.guidance = guidance
        arr, keep = self._refs(refs)
        p.refs, p.num_refs = arr, len(refs)
        out = np.empty_like(z0)
        vel = np.empty((steps,) + z0.shape, dtype=np.float32) if return_velocities else None
        check(lib().flux_cuda_sample(self.handle, ctypes.byref(p), _fp(z0), _fp(out),
                                     _fp(vel) if vel is not None else None))
        return (out, vel) if return_velocities else out

    def close(self):
        if self.handle:
            lib().flux_cuda_model_free(self.handle)
            self.handle = ctypes.c_void_p()


class TextEncoder:
    """The Qwen3 text encoder on one GPU. Mirrors qwen3_model_load / qwen3_forward / qwen3_model_free."""

    def __init__(self, ctx, handle, dims):
        self.ctx, self.handle, self.dims = ctx, handle, dims

    @staticmethod
    def load_dir(ctx, model_dir, max_seq=512):
        h = ctypes.c_void_p()
        check(lib().flux_cuda_qwen3_load_dir(ctx.handle, model_dir.encode(), max_seq, ctypes.byref(h)))
        return TextEncoder(ctx, h, None)

    @staticmethod
    def from_tensors(ctx, dims, tensors, max_seq=512):
        cd = CQwenDims()
        for name in ("hidden", "heads", "kv_heads", "head_dim", "inter", "layers", "vocab", "rope_theta"):
            setattr(cd, name, getattr(dims, name))
        for i in range(3):
            cd.out_layers[i] = dims.out_layers[i]
        h = ctypes.c_void_p()
        check(lib().flux_cuda_qwen3_create(ctx.handle, ctypes.byref(cd), max_seq, ctypes.byref(h)))
        np = _np()
        for name, arr in tensors.items():
            arr = np.ascontiguousarray(arr)
            shape = (ctypes.c_longlong * arr.ndim)(*arr.shape)
            check(lib().flux_cuda_qwen3_set_tensor(h, name.encode(), arr.ctypes.data, _DTYPES[str(arr.dtype)], shape,
                                                   arr.ndim))
        check(lib().flux_cuda_qwen3_finalize(h))
        return TextEncoder(ctx, h, dims)

    def forward(self, ids, mask=None, hidden=None):
        """ids, mask: int sequences of one length; returns f32 [seq, 3 * hidden]."""
        np = _np()
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        ip = ctypes.POINTER(ctypes.c_int)
        mp = None
        if mask is not None:
            mask = np.ascontiguousarray(mask, dtype=np.int32)
            mp = mask.ctypes.data_as(ip)
        hdim = hidden or (self.dims.hidden if self.dims is not None else 2560)
        out = np.empty((len(ids), 3 * hdim), dtype=np.float32)
        check(lib().flux_cuda_qwen3_forward(self.handle, ids.ctypes.data_as(ip), mp, len(ids), _fp(out)))
        return out

    def forward_batch(self, ids, mask=None, hidden=None, device=False):
        """ids, mask: int arrays [batch, seq]. Returns f32 [batch, seq, 3 * hidden], or with device=True the device
        address of that array (queued, no wait, no copy)."""
        np = _np()
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        batch, seq = ids.shape
        ip = ctypes.POINTER(ctypes.c_int)
        mp = None
        if mask is not None:
            mask = np.ascontiguousarray(mask, dtype=np.int32)
            mp = mask.ctypes.data_as(ip)
        if device:
            dev = ctypes.c_void_p()
            check(lib().flux_cuda_qwen3_forward_batch_device(self.handle, ids.ctypes.data_as(ip), mp, batch, seq,
                                                             ctypes.byref(dev)))
            return dev.value
        hdim = hidden or (self.dims.hidden if self.dims is not None else 2560)
        out = np.empty((batch, seq, 3 * hdim), dtype=np.float32)
        check(lib().flux_cuda_qwen3_forward_batch(self.handle, ids.ctypes.data_as(ip), mp, batch, seq, _fp(out)))
        return out

    def forward_device(self, ids, mask=None):
        """Queues the pass and returns the device address of the f32 [seq, 3 * hidden] result (no wait, no copy)."""
        np = _np()
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        ip = ctypes.POINTER(ctypes.c_int)
        mp = None
        if mask is not None:
            mask = np.ascontiguousarray(mask, dtype=np.int32)
            mp = mask.ctypes.data_as(ip)
        dev = ctypes.c_void_p()
        check(lib().flux_cuda_qwen3_forward_device(self.handle, ids.ctypes.data_as(ip), mp, len(ids), ctypes.byref(dev)))
        return dev.value

    def close(self):
        if self.handle:
            lib().flux_cuda_qwen3_free(self.handle)
            self.handle = ctypes.c_void_p()


class Vae:
    """The VAE decoder on one GPU. Mirrors flux_vae_load_safetensors / flux_vae_decode / flux_vae_free."""

    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle

    @staticmethod
    def load_safetensors(ctx, path):
        h = ctypes.c_void_p()
        check(lib().flux_cuda_vae_load_safetensors(ctx.handle, path.encode(), ctypes.byref(h)))
        return Vae(ctx, h)

    @staticmethod
    def from_tensors(ctx, tensors):
        h = ctypes.c_void_p()
        check(lib().flux_cuda_vae_create(ctx.handle, ctypes.byref(h)))
        np = _np()
        for name, arr in tensors.items():
            arr = np.ascontiguousarray(arr)
            shape = (ctypes.c_longlong * arr.ndim)(*arr.shape)
            check(lib().flux_cuda_vae_set_tensor(h, name.encode(), arr.ctypes.data, _DTYPES[str(arr.dtype)], shape,
                                                 arr.ndim))
        check(lib().flux_cuda_vae_finalize(h))
        return Vae(ctx, h)

    def decode(self, latent):
        """latent f32 [128, h, w] -> uint8 RGB [16h, 16w, 3]."""
        np = _np()
        lat = np.ascontiguousarray(latent, dtype=np.float32)
        _, h, w = lat.shape
        out = np.empty((16 * h, 16 * w, 3), dtype=np.uint8)
        check(lib().flux_cuda_vae_decode(self.handle, lat.ctypes.data, h, w, out.ctypes.data))
        return out

    def encode(self, image):
        """image f32 [3, H, W] in [-1, 1] -> latent f32 [128, H/16, W/16]."""
        np = _np()
        img = np.ascontiguousarray(image, dtype=np.float32)
        _, H, W = img.shape
        out = np.empty((128, H // 16, W // 16), dtype=np.float32)
        check(lib().flux_cuda_vae_encode(self.handle, img.ctypes.data, H, W, out.ctypes.data))
        return out

    def has_encoder(self):
        return bool(lib().flux_cuda_vae_has_encoder(self.handle))

    def decode_ptr(self, latent_ptr, h, w, rgb_host_ptr):
        """latent_ptr: host or device address of f32 [128, h, w]; rgb_host_ptr: host address of uint8 [16h, 16w, 3]."""
        check(lib().flux_cuda_vae_decode(self.handle, latent_ptr, h, w, rgb_host_ptr))

    def decode_device(self, latent_ptr, h, w):
        """Queues the decode (no wait); returns the device address of the uint8 [16h, 16w, 3] image."""
        p = ctypes.c_void_p()
        check(lib().flux_cuda_vae_decode_device(self.handle, latent_ptr, h, w, ctypes.byref(p)))
        return p.value

    def last_launches(self):
        return int(lib().flux_cuda_vae_last_launches(self.handle))

    def close(self):
        if self.handle:
            lib().flux_cuda_vae_free(self.handle)
            self.handle = ctypes.c_void_p()


class _BorrowedContext(Context):
    """A context owned by a Group: usable like any other, never destroyed from here."""

    def __init__(self, handle, device):
        self.handle = ctypes.c_void_p(handle)
        self.device = device

    def close(self):
        self.handle = ctypes.c_void_p()


class Group:
    """Several GPUs of one machine driven from one process (flux_cuda_group_*): replicas for independent images, and
    the guidance pair of the base model split over members 0 and 1."""

    def __init__(self, devices):
        devices = list(devices)
        arr = (ctypes.c_int * len(devices))(*devices)
        self.handle = ctypes.c_void_p()
        check(lib().flux_cuda_group_create(len(devices), arr, ctypes.byref(self.handle)))
        self.devices = devices
        self.models = []

    def context(self, member):
        return _BorrowedContext(lib().flux_cuda_group_context(self.handle, member), self.devices[member])

    def load_safetensors(self, path):
        check(lib().flux_cuda_group_load_safetensors(self.handle, path.encode()))

    def set_models(self, models):
        self.models = list(models)  # keep them alive
        arr = (ctypes.c_void_p * len(models))(*[m.handle for m in models])
        check(lib().flux_cuda_group_set_models(self.handle, arr))

    @staticmethod
    def _params(h, w, schedule, txt_seq, ctx_emb=None, ctx_uncond=None, guidance=1.0, refs=()):
        np = _np()
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        p = CSampleParams()
        p.h, p.w, p.num_steps, p.schedule, p.txt_seq, p.guidance = h, w, len(sch) - 1, _fp(sch), txt_seq, guidance
        keep = [sch]
        if ctx_emb is not None:
            ctx_emb = np.ascontiguousarray(ctx_emb, dtype=np.float32)
            p.ctx = _fp(ctx_emb)
            keep.append(ctx_emb)
        if ctx_uncond is not None:
            ctx_uncond = np.ascontiguousarray(ctx_uncond, dtype=np.float32)
            p.ctx_uncond = _fp(ctx_uncond)
            keep.append(ctx_uncond)
        arr, k2 = Model._refs(refs)
        p.refs, p.num_refs = arr, len(refs)
        return p, keep + [arr, k2]

    def sample_batch(self, z0s, ctxs, h, w, schedule, refs=()):
        """Independent images: z0s[i] [C, h, w], ctxs[i] [txt_seq, text_dim]; image i runs on member i % n."""
        np = _np()
        z0s = [np.ascontiguousarray(z, dtype=np.float32) for z in z0s]
        ctxs = [np.ascontiguousarray(c, dtype=np.float32) for c in ctxs]
        outs = [np.empty_like(z) for z in z0s]
        p, keep = self._params(h, w, schedule, ctxs[0].shape[0] if ctxs else 0, refs=refs)
        n = len(z0s)
        fpp = ctypes.POINTER(ctypes.c_float)
        za, ca, oa = (fpp * max(1, n))(*[_fp(z) for z in z0s]), (fpp * max(1, n))(*[_fp(c) for c in ctxs]), \
            (fpp * max(1, n))(*[_fp(o) for o in outs])
        check(lib().flux_cuda_group_sample_batch(self.handle, ctypes.byref(p), n, za, ca, oa))
        return outs

    def sample_cfg_pair(self, z0, h, w, ctx_cond, ctx_uncond, guidance, schedule, refs=()):
        np = _np()
        z0 = np.ascontiguousarray(z0, dtype=np.float32)
        ctx_cond = np.ascontiguousarray(ctx_cond, dtype=np.float32)
        p, keep = self._params(h, w, schedule, ctx_cond.shape[0], ctx_cond, ctx_uncond, guidance, refs)
        out = np.empty_like(z0)
        check(lib().flux_cuda_group_sample_cfg_pair(self.handle, ctypes.byref(p), _fp(z0), _fp(out)))
        return out

    def close(self):
        if self.handle:
            lib().flux_cuda_group_destroy(self.handle)
            self.handle = ctypes.c_void_p()
        self.models = []


class Sampler:
    """Buffers for one (h, w, txt_seq, refs, batch) shape: upload / run / download as separate phases."""

    def __init__(self, model, h, w, txt_seq, ref_shapes=(), batch=1, max_steps=4):
        self.model = model
        arr = (CRefShape * max(1, len(ref_shapes)))()
        for i, (rh, rw, toff) in enumerate(ref_shapes):
            arr[i].h, arr[i].w, arr[i].t_offset = rh, rw, toff
        self.handle = ctypes.c_void_p()
        check(lib().flux_cuda_sampler_create(model.handle, h, w, txt_seq, arr, len(ref_shapes), batch, max_steps,
                                             ctypes.byref(self.handle)))
        self.n_refs = len(ref_shapes)

    def upload(self, z0_ptr, ctx_ptr, ctx_uncond_ptr=None, ref_ptrs=()):
        """Addresses (ints) of f32 buffers, host (pinned memory makes the copies asynchronous) or device."""
        refs = (ctypes.c_void_p * max(1, len(ref_ptrs)))(*ref_ptrs)
        check(lib().flux_cuda_sampler_upload(self.handle, z0_ptr, ctx_ptr, ctx_uncond_ptr, refs))

    def run(self, schedule, guidance=1.0, record_velocities=False, apply_update=True):
        np = _np()
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        check(lib().flux_cuda_sampler_run(self.handle, _fp(sch), len(sch) - 1, guidance, int(record_velocities),
                                          int(apply_update)))

    def run_steps(self, schedule, first, count, guidance=1.0, record_velocities=False):
        np = _np()
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        check(lib().flux_cuda_sampler_run_steps(self.handle, _fp(sch), len(sch) - 1, first, count, guidance,
                                                int(record_velocities)))

    def predict(self, schedule, step):
        """Velocity of the current latent at schedule[step]; the latent is left untouched."""
        np = _np()
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        check(lib().flux_cuda_sampler_predict(self.handle, _fp(sch), len(sch) - 1, step))

    def velocity(self, dst_dev_ptr, scale=1.0):
        check(lib().flux_cuda_sampler_velocity(self.handle, dst_dev_ptr, scale))

    def apply_velocity(self, v_dev_ptr, step):
        check(lib().flux_cuda_sampler_apply_velocity(self.handle, v_dev_ptr, step))

    def latent_device(self):
        """Device address of the current latent (f32 [128, h, w])."""
        p = ctypes.c_void_p()
        check(lib().flux_cuda_sampler_latent_device(self.handle, ctypes.byref(p)))
        return p.value

    def download(self, latent_ptr, velocities_ptr=None):
        check(lib().flux_cuda_sampler_download(self.handle, latent_ptr, velocities_ptr))

    def stage_inputs(self, z0_ptr, ctx_ptr, ctx_uncond_ptr=None, ref_ptrs=()):
        """Inputs of the NEXT image, copied on a second stream while the current image runs; the next run() picks
        them up. The (pinned) host buffers must stay valid until that run has been synchronised."""
        refs = (ctypes.c_void_p * max(1, len(ref_ptrs)))(*ref_ptrs)
        check(lib().flux_cuda_sampler_stage_inputs(self.handle, z0_ptr, ctx_ptr, ctx_uncond_ptr, refs))

    def download_async(self, latent_ptr):
        """Queues the device -> host copy of the latent behind the run; Context.sync() waits for it."""
        check(lib().flux_cuda_sampler_download_async(self.handle, latent_ptr))

    def last_run(self):
        ms = ctypes.c_float()
        n = ctypes.c_longlong()
        check(lib().flux_cuda_sampler_last_run(self.handle, ctypes.byref(ms), ctypes.byref(n)))
        return ms.value, n.value

    def set_profiling(self, on):
        check(lib().flux_cuda_sampler_set_profiling(self.handle, int(on)))

    def profile(self):
        """Device ms and launch count per kernel class of the last profiled run (synchronise first)."""
        ms = (ctypes.c_float * 5)()
        n = (ctypes.c_longlong * 5)()
        check(lib().flux_cuda_sampler_profile(self.handle, ms, n))
        return {k: {"ms": ms[i], "n": n[i]} for i, k in enumerate(("gemm", "attn", "adaln", "qknorm", "other"))}

    def profile_groups(self):
        """Device ms of the last profiled run per part of the forward (the reference's timing globals' split)."""
        ms = (ctypes.c_float * 4)()
        check(lib().flux_cuda_sampler_profile_groups(self.handle, ms))
        return dict(zip(("edges", "double_blocks", "single_blocks", "final_layer"), [ms[i] for i in range(4)]))

    def profile_launches(self, capacity=8192):
        """[(ms, class index)] of the last profiled run, in launch order."""
        ms = (ctypes.c_float * capacity)()
        cls = (ctypes.c_int * capacity)()
        n = ctypes.c_int()
        check(lib().flux_cuda_sampler_profile_launches(self.handle, ms, cls, capacity, ctypes.byref(n)))
        return [(ms[i], cls[i]) for i in range(n.value)]

    def close(self):
        if self.handle:
            lib().flux_cuda_sampler_free(self.handle)
            self.handle = ctypes.c_void_p()
