"""CPU restatement (numpy, f32) of the reference's DiT denoising step and Euler samplers.

TEST INFRASTRUCTURE ONLY. This module is the parity oracle: tests, the smoke check and the
benchmark's CPU-baseline leg import it; the product library never does. It restates, in plain
numpy, what the reference computes on its CPU path:

  * flux_transformer_forward / _with_refs / _with_multi_refs   flux_transformer.c:3115-3577, 3605-4043
  * double_block_forward, single_block_forward                 flux_transformer.c:1774-1986, 2992-3109
  * apply_adaln, apply_qk_norm, apply_rope_2d                  flux_transformer.c:979-1048, 1052-1106, 719-741
  * compute_rope_2d[_with_t_offset], compute_rope_text         flux_transformer.c:591-779
  * get_timestep_embedding, time_embed_forward                 flux_transformer.c:940-969
  * flux_official_schedule, flux_linear/power_schedule         flux_sample.c:49-69, 122-155
  * flux_sample_euler*, flux_sample_euler_cfg*                 flux_sample.c:212-290, 303-444, 457-691
  * flux_rng_seed / flux_randn / flux_init_noise               flux_kernels.c:45-102, flux_sample.c:835-877
  * flux_patchify / flux_unpatchify                            flux_kernels.c:1038-1094
  * qwen3_forward and its layers (text encoder)                flux_qwen3.c:176-517, 1041-1156

Parity is PINNED: tests/golden/ holds outputs of the reference itself (compiled from its own
sources by oracle/Makefile and run through oracle/ref_binding.py by tests/golden/make_golden.py),
and tests/test_oracle.py checks this restatement against them.

All arithmetic is f32 like the reference's (weights are bf16 in the file and expanded exactly).
Matrix products go through numpy's BLAS, so summation order differs from the reference at the
1e-6 level, as it does between the reference's own generic and BLAS builds.
"""
import numpy as np

F = np.float32
EPS = F(1e-6)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def silu(x):
    return x / (F(1.0) + np.exp(-x, dtype=np.float32))


# ----------------------------------------------------------------------------------------- schedules
def official_schedule(num_steps, image_seq_len):
    """flux_sample.c:122-155 (compute_empirical_mu, generalized_time_snr_shift with sigma = 1)."""
    a1, b1, a2, b2 = F(8.73809524e-05), F(1.89833333), F(0.00016927), F(0.45666666)
    n = F(image_seq_len)
    if image_seq_len > 4300:
        mu = a2 * n + b2
    else:
        m200 = a2 * n + b2
        m10 = a1 * n + b1
        a = (m200 - m10) / F(190.0)
        b = m200 - F(200.0) * a
        mu = a * F(num_steps) + b
    emu = np.exp(F(mu), dtype=np.float32)
    out = np.zeros(num_steps + 1, dtype=np.float32)
    for i in range(num_steps + 1):
        t = F(1.0) - F(i) / F(num_steps)
        if t <= 0:
            out[i] = 0.0
        elif t >= 1:
            out[i] = 1.0
        else:
            out[i] = emu / (emu + (F(1.0) / t - F(1.0)))
    return out


def linear_schedule(num_steps):
    return (F(1.0) - np.arange(num_steps + 1, dtype=np.float32) / F(num_steps)).astype(np.float32)


def power_schedule(num_steps, alpha):
    t = np.arange(num_steps + 1, dtype=np.float32) / F(num_steps)
    return (F(1.0) - np.power(t, F(alpha), dtype=np.float32)).astype(np.float32)


# ----------------------------------------------------------------------------------------- noise
_M64 = (1 << 64) - 1


def _rotl(x, k):
    return ((x << k) | (x >> (64 - k))) & _M64


class Xoshiro:
    """xoshiro256** seeded through SplitMix64 (flux_kernels.c:45-78). Pure Python: small counts only."""

    def __init__(self, seed):
        s = []
        seed &= _M64
        for _ in range(4):
            seed = (seed + 0x9E3779B97F4A7C15) & _M64
            z = seed
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
            s.append(z ^ (z >> 31))
        self.s = s

    def next_u64(self):
        s = self.s
        result = (_rotl((s[1] * 5) & _M64, 7) * 9) & _M64
        t = (s[1] << 17) & _M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def uniform(self):
        return F((self.next_u64() >> 11) * (1.0 / 9007199254740992.0))

    def normal(self):
        """Box-Muller, cosine branch only, two uniforms per normal (flux_kernels.c:84-91)."""
        u1 = self.uniform()
        u2 = self.uniform()
        while u1 == 0.0:
            u1 = self.uniform()
        return F(np.sqrt(F(-2.0) * np.log(u1, dtype=np.float32), dtype=np.float32) *
                 np.cos(F(2.0) * F(3.14159265358979323846) * u2, dtype=np.float32))


def randn(seed, n):
    r = Xoshiro(seed)
    return np.array([r.normal() for _ in range(n)], dtype=np.float32)


NOISE_MAX = 112


def noise_source_index(channels, h, w):
    """Index into the 112x112 master field that flux_init_noise copies to each target element
    (flux_sample.c:856-872). For h, w >= 112 the field is generated directly at the target size."""
    if h >= NOISE_MAX and w >= NOISE_MAX:
        return np.arange(channels * h * w).reshape(channels, h, w)
    sy = (np.arange(h) * NOISE_MAX) // h
    sx = (np.arange(w) * NOISE_MAX) // w
    c = np.arange(channels)
    return (c[:, None, None] * NOISE_MAX + sy[None, :, None]) * NOISE_MAX + sx[None, None, :]


# ----------------------------------------------------------------------------------------- RoPE tables
def _base_freqs(axis_dim, theta):
    d = np.arange(axis_dim // 2, dtype=np.float32)
    return (F(1.0) / np.power(F(theta), (F(2.0) * d) / F(axis_dim), dtype=np.float32)).astype(np.float32)


def rope_table(pos4, axis_dim=32, theta=2000.0):
    """cos, sin [n, 4*axis_dim] for integer 4-D positions pos4 [n, 4] = (T, Y, X, L); each frequency's value is
    duplicated over the (even, odd) pair it rotates (flux_transformer.c:597-646)."""
    fr = _base_freqs(axis_dim, theta)
    ang = pos4.astype(np.float32)[:, :, None] * fr[None, None, :]
    cos = np.repeat(np.cos(ang, dtype=np.float32), 2, axis=2).reshape(pos4.shape[0], -1)
    sin = np.repeat(np.sin(ang, dtype=np.float32), 2, axis=2).reshape(pos4.shape[0], -1)
    return cos.astype(np.float32), sin.astype(np.float32)


def image_positions(h, w, t_offset=0):
    yy, xx = np.meshgrid(np.arange(h), np.arange(w), indexing="ij")
    p = np.zeros((h * w, 4), dtype=np.int64)
    p[:, 0] = t_offset
    p[:, 1] = yy.reshape(-1)
    p[:, 2] = xx.reshape(-1)
    return p


def text_positions(n):
    p = np.zeros((n, 4), dtype=np.int64)
    p[:, 3] = np.arange(n)
    return p


def apply_rope(x, cos, sin):
    """x [n, H, 128]; consecutive pairs (2j, 2j+1) rotate by (cos, sin)[n, 2j] (flux_transformer.c:719-741)."""
    x0 = x[..., 0::2]
    x1 = x[..., 1::2]
    c = cos[:, None, 0::2]
    s = sin[:, None, 0::2]
    out = np.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * s
    out[..., 1::2] = x1 * c + x0 * s
    return out


# ----------------------------------------------------------------------------------------- patchify
def patchify(x, p=2):
    """[B, C, H, W] -> [B, C p p, H/p, W/p], new channel = c p p + pi p + pj (flux_kernels.c:1038-1065)."""
    B, C, H, W = x.shape
    y = x.reshape(B, C, H // p, p, W // p, p).transpose(0, 1, 3, 5, 2, 4)
    return np.ascontiguousarray(y.reshape(B, C * p * p, H // p, W // p))


def unpatchify(x, p=2):
    """[B, C p p, H, W] -> [B, C, H p, W p] (flux_kernels.c:1067-1094)."""
    B, Cpp, H, W = x.shape
    C = Cpp // (p * p)
    y = x.reshape(B, C, p, p, H, W).transpose(0, 1, 4, 2, 5, 3)
    return np.ascontiguousarray(y.reshape(B, C, H * p, W * p))


# ----------------------------------------------------------------------------------------- layers
def timestep_embedding(t, dim=256, max_period=10000.0):
    """[cos(t*1000*w_i) | sin(t*1000*w_i)], w_i = exp(-ln(max_period) * i / (dim/2)) (flux_transformer.c:940-951, 3140)."""
    half = dim // 2
    tt = F(t) * F(1000.0)
    i = np.arange(half, dtype=np.float32)
    freq = np.exp(-np.log(F(max_period), dtype=np.float32) * i / F(half), dtype=np.float32)
    ang = (tt * freq).astype(np.float32)
    return np.concatenate([np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)]).astype(np.float32)


def adaln(x, shift, scale):
    """LayerNorm without affine (biased variance, eps 1e-6) then (1 + scale) * xhat + shift (flux_transformer.c:1021-1046)."""
    mu = x.mean(axis=1, keepdims=True, dtype=np.float32)
    xc = x - mu
    var = (xc * xc).mean(axis=1, keepdims=True, dtype=np.float32)
    xh = xc / np.sqrt(var + EPS, dtype=np.float32)
    return ((F(1.0) + scale)[None, :] * xh + shift[None, :]).astype(np.float32)


def qk_norm(x, w):
    """x [n, H, 128]: per (token, head) RMSNorm times w[128] (flux_transformer.c:1083-1101)."""
    ms = (x * x).mean(axis=2, keepdims=True, dtype=np.float32)
    return (x * (F(1.0) / np.sqrt(ms + EPS, dtype=np.float32)) * w[None, None, :]).astype(np.float32)


def attention(q, k, v):
    """q [nq, H, d], k, v [nk, H, d] -> [nq, H*d]; softmax(q k^T / sqrt(d)) v per head, no mask
    (flux_transformer.c:1249-1330, 1335-1460)."""
    nq, H, d = q.shape
    scale = F(1.0 / np.sqrt(float(d)))
    out = np.empty((nq, H, d), dtype=np.float32)
    for hh in range(H):
        s = (q[:, hh, :] @ k[:, hh, :].T) * scale
        s -= s.max(axis=1, keepdims=True)
        p = np.exp(s, dtype=np.float32)
        p /= p.sum(axis=1, keepdims=True, dtype=np.float32)
        out[:, hh, :] = p @ v[:, hh, :]
    return out.reshape(nq, H * d)


# ----------------------------------------------------------------------------------------- Qwen3 text encoder
class QwenOracle:
    """numpy f32 restatement of the reference's Qwen3 encoder forward on its CPU path: qwen3_forward
    (flux_qwen3.c:1041-1156), qwen3_layer_forward (484-517), qwen3_attention_forward (313-452: GQA, causal + key
    padding mask with -1e9, softmax), qwen3_mlp_forward (458-478), qwen3_rms_norm / qwen3_head_rms_norm (176-221),
    half-split RoPE with theta 1e6 (253-307). Output: hidden states after the layers in dims.out_layers
    concatenated, [seq, 3 * hidden]. Like the reference's CPU path it can run all layers; the output only depends on
    the first max(out_layers) + 1."""

    def __init__(self, tensors, dims):
        self.t, self.d, self.cache = tensors, dims, {}

    def W(self, name):
        if name not in self.cache:
            a = self.t[name]
            self.cache[name] = bf16_bits_to_f32(a) if a.dtype == np.uint16 else np.asarray(a, dtype=np.float32)
        return self.cache[name]

    @staticmethod
    def rms(x, w, eps=F(1e-6)):
        ms = (x * x).mean(axis=-1, keepdims=True, dtype=np.float32)
        return (x * (F(1.0) / np.sqrt(ms + eps, dtype=np.float32)) * w).astype(np.float32)

    def forward(self, ids, mask=None, num_layers=None):
        d = self.d
        seq = len(ids)
        H, KV, hd = d.heads, d.kv_heads, d.head_dim
        emb = self.W("model.embed_tokens.weight")
        x = np.zeros((seq, d.hidden), dtype=np.float32)
        for s_, tok in enumerate(ids):
            if 0 <= tok < d.vocab:
                x[s_] = emb[tok]
        half = hd // 2
        i = np.arange(half, dtype=np.float32)
        freq = (F(1.0) / np.power(F(d.rope_theta), (F(2.0) * i) / F(hd), dtype=np.float32)).astype(np.float32)
        ang = np.arange(seq, dtype=np.float32)[:, None] * freq[None, :]
        cos, sin = np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)

        def rope(t):  # t [seq, heads, hd], pairs (i, i + half)
            a, b = t[..., :half], t[..., half:]
            c, s = cos[:, None, :], sin[:, None, :]
            return np.concatenate([a * c - b * s, a * s + b * c], axis=-1)

        bias = np.zeros((seq, seq), dtype=np.float32)
        bias[np.triu_indices(seq, 1)] = 1.0
        if mask is not None:
            bias[:, np.asarray(mask) == 0] = 1.0
        masked = bias > 0
        scale = F(1.0 / np.sqrt(float(hd)))
        outs = []
        last = max(d.out_layers) + 1 if num_layers is None else num_layers
        for l in range(last):
            p = "model.layers.%d." % l
            n = self.rms(x, self.W(p + "input_layernorm.weight"))
            q = (n @ self.W(p + "self_attn.q_proj.weight").T).reshape(seq, H, hd)
            k = (n @ self.W(p + "self_attn.k_proj.weight").T).reshape(seq, KV, hd)
            v = (n @ self.W(p + "self_attn.v_proj.weight").T).reshape(seq, KV, hd)
            q = rope(self.rms(q, self.W(p + "self_attn.q_norm.weight")))
            k = rope(self.rms(k, self.W(p + "self_attn.k_norm.weight")))
            att = np.empty((seq, H, hd), dtype=np.float32)
            for h in range(H):
                g = h // (H // KV)
                sc = (q[:, h, :] @ k[:, g, :].T) * scale
                sc[masked] = F(-1e9)
                sc -= sc.max(axis=1, keepdims=True)
                pr = np.exp(sc, dtype=np.float32)
                pr /= pr.sum(axis=1, keepdims=True, dtype=np.float32)
                att[:, h, :] = pr @ v[:, g, :]
            x = x + att.reshape(seq, H * hd) @ self.W(p + "self_attn.o_proj.weight").T
            n = self.rms(x, self.W(p + "post_attention_layernorm.weight"))
            gate = n @ self.W(p + "mlp.gate_proj.weight").T
            up = n @ self.W(p + "mlp.up_proj.weight").T
            x = (x + (silu(gate) * up) @ self.W(p + "mlp.down_proj.weight").T).astype(np.float32)
            if l in d.out_layers:
                outs.append(x.copy())
        return np.concatenate(outs, axis=1).astype(np.float32)


class OracleModel:
    """Holds the DiT weights (name -> array, bf16 bit patterns or f32) and evaluates the reference's forward pass."""

    def __init__(self, tensors, dims, cache_f32=True):
        self.t = tensors
        self.d = dims
        self.cache = {} if cache_f32 else None
        self.taps = None  # set to a dict to record intermediates (block outputs) of the next forward

    def W(self, name):
        if self.cache is not None and name in self.cache:
            return self.cache[name]
        a = self.t[name]
        w = bf16_bits_to_f32(a) if a.dtype == np.uint16 else np.asarray(a, dtype=np.float32)
        if self.cache is not None:
            self.cache[name] = w
        return w

    def preload(self, threads=8):
        """Expands every bf16 tensor to f32 up front, in parallel (the reference does the same at load time,
        flux_transformer.c:4444)."""
        from concurrent.futures import ThreadPoolExecutor
        if self.cache is None:
            self.cache = {}
        names = [n for n in self.t if n not in self.cache]

        def conv(n):
            a = self.t[n]
            if a.dtype != np.uint16:
                return n, np.asarray(a, dtype=np.float32)
            out = np.empty(a.shape, dtype=np.float32)
            o32 = out.view(np.uint32)
            np.copyto(o32, a, casting="unsafe")
            np.left_shift(o32, 16, out=o32)
            return n, out

        with ThreadPoolExecutor(max_workers=threads) as ex:
            for n, w in ex.map(conv, names):
                self.cache[n] = w

    def lin(self, x, name):
        return (x @ self.W(name).T).astype(np.float32)

    # -- one forward pass; refs = [(latent [C, rh, rw], t_offset), ...]
    def forward(self, z, h, w, ctx, t, refs=()):
        d = self.d
        H, hd, hid, m = d.heads, d.head_dim, d.hidden, d.mlp
        n_img = h * w
        n_txt = ctx.shape[0]
        tap = self.taps

        e = timestep_embedding(t, d.time_dim)
        p = "time_guidance_embed.timestep_embedder."
        t_emb = self.lin(silu(self.lin(e[None, :], p + "linear_1.weight")), p + "linear_2.weight")
        s = silu(t_emb)  # [1, hidden]
        mod_img = self.lin(s, "double_stream_modulation_img.linear.weight")[0]
        mod_txt = self.lin(s, "double_stream_modulation_txt.linear.weight")[0]
        mod_single = self.lin(s, "single_stream_modulation.linear.weight")[0]
        mod_final = self.lin(s, "norm_out.linear.weight")[0]

        # tokens: target image first, then each reference's tokens (flux_transformer.c:3157-3161, 3650-3664)
        toks = [np.ascontiguousarray(z.reshape(d.latent_ch, n_img).T)]
        pos = [image_positions(h, w, 0)]
        for lat, toff in refs:
            rh, rw = lat.shape[1], lat.shape[2]
            toks.append(np.ascontiguousarray(lat.reshape(d.latent_ch, rh * rw).T))
            pos.append(image_positions(rh, rw, toff))
        x_img = np.concatenate(toks, axis=0).astype(np.float32)
        img_cos, img_sin = rope_table(np.concatenate(pos, axis=0), d.axis_dim, d.rope_theta)
        txt_cos, txt_sin = rope_table(text_positions(n_txt), d.axis_dim, d.rope_theta)
        n_all_img = x_img.shape[0]

        img = self.lin(x_img, "x_embedder.weight")
        txt = self.lin(ctx.astype(np.float32), "context_embedder.weight")
        if tap is not None:
            tap["img_embed"] = img.copy()
            tap["txt_embed"] = txt.copy()

        def chunks(v, k):
            return [v[i * hid:(i + 1) * hid] for i in range(k)]

        i_sh1, i_sc1, i_g1, i_sh2, i_sc2, i_g2 = chunks(mod_img, 6)
        t_sh1, t_sc1, t_g1, t_sh2, t_sc2, t_g2 = chunks(mod_txt, 6)

        for b in range(d.n_double):
            pre = "transformer_blocks.%d." % b
            ni = adaln(img, i_sh1, i_sc1)
            nt = adaln(txt, t_sh1, t_sc1)
            iq = self.lin(ni, pre + "attn.to_q.weight").reshape(-1, H, hd)
            ik = self.lin(ni, pre + "attn.to_k.weight").reshape(-1, H, hd)
            iv = self.lin(ni, pre + "attn.to_v.weight").reshape(-1, H, hd)
            tq = self.lin(nt, pre + "attn.add_q_proj.weight").reshape(-1, H, hd)
            tk = self.lin(nt, pre + "attn.add_k_proj.weight").reshape(-1, H, hd)
            tv = self.lin(nt, pre + "attn.add_v_proj.weight").reshape(-1, H, hd)
            iq = apply_rope(qk_norm(iq, self.W(pre + "attn.norm_q.weight")), img_cos, img_sin)
            ik = apply_rope(qk_norm(ik, self.W(pre + "attn.norm_k.weight")), img_cos, img_sin)
            tq = apply_rope(qk_norm(tq, self.W(pre + "attn.norm_added_q.weight")), txt_cos, txt_sin)
            tk = apply_rope(qk_norm(tk, self.W(pre + "attn.norm_added_k.weight")), txt_cos, txt_sin)
            k_all = np.concatenate([tk, ik], axis=0)  # [txt ; img]
            v_all = np.concatenate([tv, iv], axis=0)
            io = attention(iq, k_all, v_all)
            to = attention(tq, k_all, v_all)
            img = img + i_g1[None, :] * self.lin(io, pre + "attn.to_out.0.weight")
            txt = txt + t_g1[None, :] * self.lin(to, pre + "attn.to_add_out.weight")
            ni = adaln(img, i_sh2, i_sc2)
            nt = adaln(txt, t_sh2, t_sc2)
            fi = self.lin(ni, pre + "ff.linear_in.weight")
            ft = self.lin(nt, pre + "ff_context.linear_in.weight")
            img = img + i_g2[None, :] * self.lin(silu(fi[:, :m]) * fi[:, m:], pre + "ff.linear_out.weight")
            txt = txt + t_g2[None, :] * self.lin(silu(ft[:, :m]) * ft[:, m:], pre + "ff_context.linear_out.weight")
            if tap is not None:
                tap["double_%d_img" % b] = img.copy()
                tap["double_%d_txt" % b] = txt.copy()

        hs = np.concatenate([txt, img], axis=0).astype(np.float32)
        cos = np.concatenate([txt_cos, img_cos], axis=0)
        sin = np.concatenate([txt_sin, img_sin], axis=0)
        s_sh, s_sc, s_g = chunks(mod_single, 3)
        for j in range(d.n_single):
            pre = "single_transformer_blocks.%d." % j
            n = adaln(hs, s_sh, s_sc)
            f = self.lin(n, pre + "attn.to_qkv_mlp_proj.weight")
            q = f[:, 0:hid].reshape(-1, H, hd)
            k = f[:, hid:2 * hid].reshape(-1, H, hd)
            v = f[:, 2 * hid:3 * hid].reshape(-1, H, hd)
            g = f[:, 3 * hid:3 * hid + m]
            u = f[:, 3 * hid + m:]
            q = apply_rope(qk_norm(q, self.W(pre + "attn.norm_q.weight")), cos, sin)
            k = apply_rope(qk_norm(k, self.W(pre + "attn.norm_k.weight")), cos, sin)
            o = attention(q, k, v)
            cat = np.concatenate([o, silu(g) * u], axis=1)
            hs = hs + s_g[None, :] * self.lin(cat, pre + "attn.to_out.weight")
            if tap is not None:
                tap["single_%d" % j] = hs.copy()

        a = hs[n_txt:n_txt + n_img]  # target tokens only; reference tokens are dropped
        f_scale, f_shift = mod_final[:hid], mod_final[hid:]  # scale first, then shift
        out = self.lin(adaln(a, f_shift, f_scale), "proj_out.weight")
        del n_all_img
        return np.ascontiguousarray(out.T).reshape(d.latent_ch, h, w).astype(np.float32)

    # -- samplers (flux_sample.c:212-290, 381-444, 457-529, 615-691)
    def sample_euler(self, z0, h, w, ctx, schedule, refs=(), record=None):
        z = z0.astype(np.float32).copy()
        for i in range(len(schedule) - 1):
            v = self.forward(z, h, w, ctx, float(schedule[i]), refs)
            if record is not None:
                record.append((z.copy(), v.copy()))
            z = z + F(schedule[i + 1] - schedule[i]) * v
        return z

    def sample_euler_cfg(self, z0, h, w, ctx_cond, ctx_uncond, guidance, schedule, refs=(), record=None):
        z = z0.astype(np.float32).copy()
        g = F(guidance)
        for i in range(len(schedule) - 1):
            vu = self.forward(z, h, w, ctx_uncond, float(schedule[i]), refs)
            vc = self.forward(z, h, w, ctx_cond, float(schedule[i]), refs)
            v = vu + g * (vc - vu)
            if record is not None:
                record.append((z.copy(), v.copy()))
            z = z + F(schedule[i + 1] - schedule[i]) * v
        return z
