"""ctypes binding of the reference implementation compiled by oracle/Makefile into oracle/_ref/.

TEST INFRASTRUCTURE ONLY (parity checker and timed CPU baseline). It calls the reference's own
link-seam symbols (declared extern in flux.c:36-119): safetensors_open, flux_transformer_load_safetensors,
flux_transformer_forward[_with_multi_refs], flux_sample_euler[_cfg], flux_official_schedule,
flux_init_noise. The shared objects are built from the reference's sources where they lie; this
file contains none of them.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _openblas_dir():
    """Directory of the wheel-bundled OpenBLAS the BLAS build links: FLUX_REF_OPENBLAS_DIR, else the
    opencv_python_headless.libs folder of whichever site-packages holds it."""
    env = os.environ.get("FLUX_REF_OPENBLAS_DIR")
    if env:
        return env
    import site
    import sysconfig
    roots = [sysconfig.get_paths().get("purelib"), sysconfig.get_paths().get("platlib")]
    try:
        roots += site.getsitepackages()
    except AttributeError:
        pass
    for r in roots:
        if r and os.path.isdir(os.path.join(r, "opencv_python_headless.libs")):
            return os.path.join(r, "opencv_python_headless.libs")
    return os.path.join(roots[0] or "", "opencv_python_headless.libs")


OB_DIR = _openblas_dir()

c_float_p = ctypes.POINTER(ctypes.c_float)


class FluxImage(ctypes.Structure):  # struct flux_image, flux.h:73-78
    _fields_ = [("width", ctypes.c_int), ("height", ctypes.c_int), ("channels", ctypes.c_int),
                ("data", ctypes.POINTER(ctypes.c_uint8))]


class FluxRefT(ctypes.Structure):  # flux_ref_t, flux.c:68-72
    _fields_ = [("latent", c_float_p), ("h", ctypes.c_int), ("w", ctypes.c_int), ("t_offset", ctypes.c_int)]


def _preload(prefix):
    """Loads a wheel-bundled shared object by file-name prefix from any <site-packages>/*.libs directory."""
    site = os.path.dirname(OB_DIR)
    for d in [OB_DIR] + sorted(os.path.join(site, x) for x in os.listdir(site) if x.endswith(".libs")):
        for f in sorted(os.listdir(d)):
            if f.startswith(prefix):
                return ctypes.CDLL(os.path.join(d, f), mode=ctypes.RTLD_GLOBAL)
    raise OSError("no bundled library starting with %s" % prefix)


def available(kind="blas"):
    return os.path.exists(os.path.join(REF_DIR, "libflux_seam.so" if kind == "seam" else "libflux_ref_%s.so" % kind))


def best_kind():
    for k in ("blas", "generic"):
        if available(k):
            try:
                RefLib(k)
                return k
            except OSError:
                continue
    return None


def _fp(a):
    return a.ctypes.data_as(c_float_p)


class RefLib:
    def __init__(self, kind="blas"):
        # kind "seam": the reference's library with flux_transformer.c, flux_sample.c and flux_qwen3.c replaced by the
        # CUDA engine's seam files (oracle/Makefile, libflux_seam.so) - same symbols, same binding, needs a GPU
        path = os.path.join(REF_DIR, "libflux_seam.so" if kind == "seam" else "libflux_ref_%s.so" % kind)
        self.kind = kind
        if kind == "blas":
            # the bundled OpenBLAS needs the libgfortran that sits next to it; load both by full path first
            _preload("libquadmath-2284e583")
            _preload("libgfortran-83c28eba")
            _preload("libopenblasp-")
        # local scope (and -Bsymbolic at link time): several builds of the same sources can live in one process
        self.L = L = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        self.libc = ctypes.CDLL(None)
        self.libc.free.argtypes = [ctypes.c_void_p]
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.safetensors_open.restype = vp
        L.safetensors_open.argtypes = [ctypes.c_char_p]
        L.safetensors_close.argtypes = [vp]
        L.flux_transformer_load_safetensors.restype = vp
        L.flux_transformer_load_safetensors.argtypes = [vp]
        L.flux_transformer_free.argtypes = [vp]
        L.flux_transformer_forward.restype = vp
        L.flux_transformer_forward.argtypes = [vp, c_float_p, ci, ci, c_float_p, ci, cf]
        L.flux_transformer_forward_with_multi_refs.restype = vp
        L.flux_transformer_forward_with_multi_refs.argtypes = [vp, c_float_p, ci, ci, ctypes.POINTER(FluxRefT), ci,
                                                               c_float_p, ci, cf]
        L.flux_sample_euler.restype = vp
        L.flux_sample_euler.argtypes = [vp, vp, c_float_p, ci, ci, ci, ci, c_float_p, ci, c_float_p, ci, vp]
        L.flux_sample_euler_with_multi_refs.restype = vp
        L.flux_sample_euler_with_multi_refs.argtypes = [vp, vp, c_float_p, ci, ci, ci, ci, ctypes.POINTER(FluxRefT),
                                                        ci, c_float_p, ci, c_float_p, ci, vp]
        L.flux_sample_euler_cfg.restype = vp
        L.flux_sample_euler_cfg.argtypes = [vp, vp, c_float_p, ci, ci, ci, ci, c_float_p, ci, c_float_p, ci, cf,
                                            c_float_p, ci, vp]
        L.flux_official_schedule.restype = vp
        L.flux_official_schedule.argtypes = [ci, ci]
        L.flux_linear_schedule.restype = vp
        L.flux_linear_schedule.argtypes = [ci]
        L.flux_power_schedule.restype = vp
        L.flux_power_schedule.argtypes = [ci, cf]
        L.flux_init_noise.restype = vp
        L.flux_init_noise.argtypes = [ci, ci, ci, ci, ctypes.c_int64]
        # exported by flux_sample.c, called from nowhere in the reference (flux_sample.c:75-116, 697-821, 891-919)
        L.flux_sigmoid_schedule.restype = vp
        L.flux_sigmoid_schedule.argtypes = [ci, cf]
        L.flux_resolution_schedule.restype = vp
        L.flux_resolution_schedule.argtypes = [ci, ci, ci]
        L.flux_sample_heun.restype = vp
        L.flux_sample_heun.argtypes = [vp, c_float_p, ci, ci, ci, ci, c_float_p, ci, c_float_p, ci, vp]
        L.flux_sample_euler_ancestral.restype = vp
        L.flux_sample_euler_ancestral.argtypes = [vp, c_float_p, ci, ci, ci, ci, c_float_p, ci, c_float_p, ci, cf, vp]
        L.flux_generate_latent.restype = vp
        L.flux_generate_latent.argtypes = [vp, c_float_p, ci, ci, ci, ci, ctypes.c_int64, vp]
        L.flux_rng_seed.argtypes = [ctypes.c_uint64]
        L.flux_patchify.argtypes = [c_float_p, c_float_p, ci, ci, ci, ci, ci]
        L.flux_unpatchify.argtypes = [c_float_p, c_float_p, ci, ci, ci, ci, ci]
        L.qwen3_model_load.restype = vp
        L.qwen3_model_load.argtypes = [ctypes.c_char_p]
        L.qwen3_model_free.argtypes = [vp]
        L.qwen3_forward.restype = vp
        L.qwen3_forward.argtypes = [vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ci]
        L.flux_vae_encode.restype = vp
        L.flux_vae_encode.argtypes = [vp, c_float_p, ci, ci, ci, ctypes.POINTER(ci), ctypes.POINTER(ci)]
        if kind == "seam":
            L.flux_vae_encode = getattr(L, "__wrap_flux_vae_encode")
            L.flux_vae_encode.restype = vp
            L.flux_vae_encode.argtypes = [vp, c_float_p, ci, ci, ci, ctypes.POINTER(ci), ctypes.POINTER(ci)]
            # the seam redirects these three at link time (-Wl,--wrap); calls from outside the library must name the
            # wrappers themselves to take the path the library's own callers take
            L.flux_vae_load_safetensors = getattr(L, "__wrap_flux_vae_load_safetensors")
            L.flux_vae_decode = getattr(L, "__wrap_flux_vae_decode")
            L.flux_vae_free = getattr(L, "__wrap_flux_vae_free")
        L.flux_vae_load_safetensors.restype = vp
        L.flux_vae_load_safetensors.argtypes = [vp]
        L.flux_vae_free.argtypes = [vp]
        L.flux_vae_decode.restype = ctypes.POINTER(FluxImage)
        L.flux_vae_decode.argtypes = [vp, c_float_p, ci, ci, ci]
        L.flux_image_free.argtypes = [ctypes.POINTER(FluxImage)]
        if kind == "blas":
            try:
                self.blas_threads = L.openblas_get_num_threads()
            except AttributeError:
                ob = ctypes.CDLL([os.path.join(OB_DIR, f) for f in os.listdir(OB_DIR) if f.startswith("libopenblasp")][0])
                self.blas_threads = ob.openblas_get_num_threads()
        else:
            self.blas_threads = 1

    def _take(self, ptr, n):
        if not ptr:
            raise RuntimeError("reference returned NULL")
        out = np.ctypeslib.as_array(ctypes.cast(ptr, c_float_p), shape=(n,)).copy()
        self.libc.free(ptr)
        return out

    def official_schedule(self, steps, seq_len):
        return self._take(self.L.flux_official_schedule(steps, seq_len), steps + 1)

    def linear_schedule(self, steps):
        return self._take(self.L.flux_linear_schedule(steps), steps + 1)

    def power_schedule(self, steps, alpha):
        return self._take(self.L.flux_power_schedule(steps, alpha), steps + 1)

    def sigmoid_schedule(self, steps, shift):
        return self._take(self.L.flux_sigmoid_schedule(steps, shift), steps + 1)

    def resolution_schedule(self, steps, height, width):
        return self._take(self.L.flux_resolution_schedule(steps, height, width), steps + 1)

    def init_noise(self, channels, h, w, seed):
        return self._take(self.L.flux_init_noise(1, channels, h, w, seed), channels * h * w).reshape(channels, h, w)

    def patchify(self, x, p=2):
        x = np.ascontiguousarray(x, dtype=np.float32)
        B, C, H, W = x.shape
        out = np.empty((B, C * p * p, H // p, W // p), dtype=np.float32)
        self.L.flux_patchify(_fp(out), _fp(x), B, C, H, W, p)
        return out

    def unpatchify(self, x, p=2):
        x = np.ascontiguousarray(x, dtype=np.float32)
        B, Cpp, H, W = x.shape
        out = np.empty((B, Cpp // (p * p), H * p, W * p), dtype=np.float32)
        self.L.flux_unpatchify(_fp(out), _fp(x), B, Cpp // (p * p), H, W, p)
        return out

    def qwen3_load(self, model_dir):
        """qwen3_model_load (flux_qwen3.c:1329): directory with the two text-encoder shards."""
        m = self.L.qwen3_model_load(model_dir.encode())
        if not m:
            raise RuntimeError("reference could not load the text encoder from %s" % model_dir)
        return m

    def qwen3_forward(self, model, ids, mask):
        """qwen3_forward (flux_qwen3.c:1041): f32 [seq, 7680]."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        mask = np.ascontiguousarray(mask, dtype=np.int32)
        ip = ctypes.POINTER(ctypes.c_int)
        p = self.L.qwen3_forward(model, ids.ctypes.data_as(ip), mask.ctypes.data_as(ip), len(ids))
        return self._take(p, len(ids) * 7680).reshape(len(ids), 7680)

    def load_vae(self, safetensors_path):
        """flux_vae_load_safetensors (flux_vae.c:1232-1386)."""
        sf = self.L.safetensors_open(safetensors_path.encode())
        if not sf:
            raise RuntimeError("reference could not open %s" % safetensors_path)
        vae = self.L.flux_vae_load_safetensors(sf)
        self.L.safetensors_close(sf)
        if not vae:
            raise RuntimeError("reference could not load the VAE")
        return vae

    def vae_encode(self, vae, image):
        """flux_vae_encode (flux_vae.c:320-440): image f32 [3, H, W] -> latent f32 [128, H/16, W/16]."""
        img = np.ascontiguousarray(image, dtype=np.float32)
        oh, ow = ctypes.c_int(), ctypes.c_int()
        p = self.L.flux_vae_encode(vae, _fp(img), 1, img.shape[1], img.shape[2], ctypes.byref(oh), ctypes.byref(ow))
        return self._take(p, 128 * oh.value * ow.value).reshape(128, oh.value, ow.value)

    def vae_decode(self, vae, latent):
        """flux_vae_decode (flux_vae.c:690-837): latent f32 [128, h, w] -> uint8 RGB [16h, 16w, 3]."""
        lat = np.ascontiguousarray(latent, dtype=np.float32)
        img = self.L.flux_vae_decode(vae, _fp(lat), 1, lat.shape[1], lat.shape[2])
        if not img:
            raise RuntimeError("reference VAE decode failed")
        i = img.contents
        out = np.ctypeslib.as_array(i.data, shape=(i.height, i.width, i.channels)).copy()
        self.L.flux_image_free(img)
        return out

    def load_transformer(self, safetensors_path):
        sf = self.L.safetensors_open(safetensors_path.encode())
        if not sf:
            raise RuntimeError("reference could not open %s" % safetensors_path)
        tf = self.L.flux_transformer_load_safetensors(sf)
        self.L.safetensors_close(sf)
        if not tf:
            raise RuntimeError("reference could not load the transformer")
        return RefTransformer(self, tf)


class RefTransformer:
    def __init__(self, lib, handle):
        self.lib, self.h = lib, handle

    def close(self):
        if self.h:
            self.lib.L.flux_transformer_free(self.h)
            self.h = None

    @staticmethod
    def _refs(refs):
        keep = [np.ascontiguousarray(lat, dtype=np.float32) for lat, _ in refs]
        arr = (FluxRefT * max(1, len(refs)))()
        for i, (lat, toff) in enumerate(refs):
            arr[i].latent = _fp(keep[i])
            arr[i].h, arr[i].w, arr[i].t_offset = lat.shape[1], lat.shape[2], toff
        return arr, keep

    def forward(self, z, h, w, ctx, t, refs=()):
        z = np.ascontiguousarray(z, dtype=np.float32)
        ctx = np.ascontiguousarray(ctx, dtype=np.float32)
        L = self.lib.L
        if refs:
            arr, keep = self._refs(refs)
            p = L.flux_transformer_forward_with_multi_refs(self.h, _fp(z), h, w, arr, len(refs), _fp(ctx),
                                                           ctx.shape[0], t)
        else:
            p = L.flux_transformer_forward(self.h, _fp(z), h, w, _fp(ctx), ctx.shape[0], t)
        return self.lib._take(p, z.size).reshape(z.shape)

    def sample_euler(self, z0, h, w, ctx, schedule, refs=()):
        z0 = np.ascontiguousarray(z0, dtype=np.float32).copy()
        ctx = np.ascontiguousarray(ctx, dtype=np.float32)
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        L = self.lib.L
        C = z0.shape[0]
        if refs:
            arr, keep = self._refs(refs)
            p = L.flux_sample_euler_with_multi_refs(self.h, None, _fp(z0), 1, C, h, w, arr, len(refs), _fp(ctx),
                                                    ctx.shape[0], _fp(sch), len(sch) - 1, None)
        else:
            p = L.flux_sample_euler(self.h, None, _fp(z0), 1, C, h, w, _fp(ctx), ctx.shape[0], _fp(sch),
                                    len(sch) - 1, None)
        return self.lib._take(p, z0.size).reshape(z0.shape)

    def sample_heun(self, z0, h, w, ctx, schedule):
        """flux_sample_heun (flux_sample.c:760-821)."""
        z0 = np.ascontiguousarray(z0, dtype=np.float32).copy()
        ctx = np.ascontiguousarray(ctx, dtype=np.float32)
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        p = self.lib.L.flux_sample_heun(self.h, _fp(z0), 1, z0.shape[0], h, w, _fp(ctx), ctx.shape[0], _fp(sch),
                                        len(sch) - 1, None)
        return self.lib._take(p, z0.size).reshape(z0.shape)

    def sample_euler_ancestral(self, z0, h, w, ctx, schedule, eta, rng_seed):
        """flux_sample_euler_ancestral (flux_sample.c:697-749); the library's global generator (flux_kernels.c:68) is
        seeded first so that the injected noise is reproducible."""
        z0 = np.ascontiguousarray(z0, dtype=np.float32).copy()
        ctx = np.ascontiguousarray(ctx, dtype=np.float32)
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        self.lib.L.flux_rng_seed(rng_seed)
        p = self.lib.L.flux_sample_euler_ancestral(self.h, _fp(z0), 1, z0.shape[0], h, w, _fp(ctx), ctx.shape[0],
                                                   _fp(sch), len(sch) - 1, eta, None)
        return self.lib._take(p, z0.size).reshape(z0.shape)

    def generate_latent(self, ctx, height, width, steps, seed):
        """flux_generate_latent (flux_sample.c:891-919): seeded noise, linear schedule, plain Euler loop."""
        ctx = np.ascontiguousarray(ctx, dtype=np.float32)
        p = self.lib.L.flux_generate_latent(self.h, _fp(ctx), ctx.shape[0], height, width, steps, seed, None)
        return self.lib._take(p, 128 * (height // 16) * (width // 16)).reshape(128, height // 16, width // 16)

    def sample_euler_cfg(self, z0, h, w, ctx_c, ctx_u, guidance, schedule):
        z0 = np.ascontiguousarray(z0, dtype=np.float32).copy()
        ctx_c = np.ascontiguousarray(ctx_c, dtype=np.float32)
        ctx_u = np.ascontiguousarray(ctx_u, dtype=np.float32)
        sch = np.ascontiguousarray(schedule, dtype=np.float32)
        p = self.lib.L.flux_sample_euler_cfg(self.h, None, _fp(z0), 1, z0.shape[0], h, w, _fp(ctx_c), ctx_c.shape[0],
                                             _fp(ctx_u), ctx_u.shape[0], guidance, _fp(sch), len(sch) - 1, None)
        return self.lib._take(p, z0.size).reshape(z0.shape)
