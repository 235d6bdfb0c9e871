"""TEST INFRASTRUCTURE ONLY - never imported by the product library.

CPU f32 restatement (torch ops on the CPU) of the reference's VAE decoder, flux_vae_decode (flux_vae.c:690-837):
batch de-normalisation with eps 1e-4 (717-729, 1247), unpatchify (733), post_quant_conv 1x1 (739-741), conv_in (745),
mid block = ResNet block, single-head attention over all pixels, ResNet block (752-767; resblock_forward 179-220,
attnblock_forward 223-314), four up levels of three ResNet blocks with nearest 2x upsampling + 3x3 convolution between
them (773-800), GroupNorm(32) + swish + conv_out (804-811), conversion to uint8 by clamping (v + 1) * 127.5 and
truncating (822-833); and of its encoder, flux_vae_encode (320-440): conv_in, four levels of two ResNet blocks with
a stride-2 convolution over the input padded at the right and bottom between them (146-171, 360-372), the same mid
block, GroupNorm + swish + conv_out, quant_conv 1x1, the mean half of the 64 channels, patchify, batch-norm with the
running statistics. Pinned against the reference build by tests/test_vae_oracle.py. Besides the image it returns the
float tensor before the conversion and, on request, every block's output, which the reference does not expose."""
import numpy as np
import torch
import torch.nn.functional as F

EPS = 1e-4
GROUPS = 32


class VaeOracle:
    def __init__(self, tensors):
        self.t = {k: torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32)) for k, v in tensors.items()}

    def _conv(self, x, name, pad):
        w = self.t[name + ".weight"]
        if w.dim() == 2:
            w = w[:, :, None, None]
        return F.conv2d(x, w, self.t[name + ".bias"], padding=pad)

    def _gn(self, x, name, swish):
        y = F.group_norm(x, GROUPS, self.t[name + ".weight"], self.t[name + ".bias"], eps=EPS)
        return F.silu(y) if swish else y

    def _res(self, x, prefix):
        h = self._conv(self._gn(x, prefix + ".norm1", True), prefix + ".conv1", 1)
        h = self._conv(self._gn(h, prefix + ".norm2", True), prefix + ".conv2", 1)
        if (prefix + ".conv_shortcut.weight") in self.t:
            x = self._conv(x, prefix + ".conv_shortcut", 0)
        return x + h

    def _attn(self, x, prefix):
        b, c, hh, ww = x.shape
        n = self._gn(x, prefix + ".group_norm", False)
        q = self._conv(n, prefix + ".to_q", 0).reshape(b, c, hh * ww).transpose(1, 2)
        k = self._conv(n, prefix + ".to_k", 0).reshape(b, c, hh * ww).transpose(1, 2)
        v = self._conv(n, prefix + ".to_v", 0).reshape(b, c, hh * ww).transpose(1, 2)
        p = torch.softmax((q * (1.0 / np.sqrt(c))) @ k.transpose(1, 2), dim=-1)
        o = (p @ v).transpose(1, 2).reshape(b, c, hh, ww)
        return x + self._conv(o, prefix + ".to_out.0", 0)

    @torch.no_grad()
    def encode(self, image):
        """image f32 [3, H, W] -> latent f32 [128, H/16, W/16]."""
        x = torch.from_numpy(np.ascontiguousarray(image, dtype=np.float32))[None]
        x = self._conv(x, "encoder.conv_in", 1)
        for lvl in range(4):
            for r in range(2):
                x = self._res(x, "encoder.down_blocks.%d.resnets.%d" % (lvl, r))
            if lvl < 3:
                p = "encoder.down_blocks.%d.downsamplers.0.conv" % lvl
                x = F.conv2d(F.pad(x, (0, 1, 0, 1)), self.t[p + ".weight"], self.t[p + ".bias"], stride=2)
        x = self._res(x, "encoder.mid_block.resnets.0")
        x = self._attn(x, "encoder.mid_block.attentions.0")
        x = self._res(x, "encoder.mid_block.resnets.1")
        x = self._conv(self._gn(x, "encoder.conv_norm_out", True), "encoder.conv_out", 1)
        x = self._conv(x, "quant_conv", 0)[:, :32]
        _, _, hl, wl = x.shape
        z = x.reshape(1, 32, hl // 2, 2, wl // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(1, 128, hl // 2, wl // 2)
        mean = self.t.get("bn.running_mean", torch.zeros(128))
        var = self.t.get("bn.running_var", torch.ones(128))
        z = (z - mean[None, :, None, None]) / torch.sqrt(var + EPS)[None, :, None, None]
        return z[0].numpy().copy()

    @torch.no_grad()
    def decode(self, latent, taps=None):
        """latent f32 [128, h, w] -> (uint8 [16h, 16w, 3], float [3, 16h, 16w]); taps: dict filled with block outputs."""
        z = torch.from_numpy(np.ascontiguousarray(latent, dtype=np.float32))[None]
        mean = self.t.get("bn.running_mean", torch.zeros(128))
        var = self.t.get("bn.running_var", torch.ones(128))
        z = z * torch.sqrt(var + EPS)[None, :, None, None] + mean[None, :, None, None]
        _, _, h, w = z.shape
        # channel c * 4 + pi * 2 + pj of the packed latent is pixel (2y + pi, 2x + pj) of channel c
        x = z.reshape(1, 32, 2, 2, h, w).permute(0, 1, 4, 2, 5, 3).reshape(1, 32, 2 * h, 2 * w)
        x = self._conv(x, "post_quant_conv", 0)
        x = self._conv(x, "decoder.conv_in", 1)

        def tap(name):
            if taps is not None:
                taps[name] = x[0].permute(1, 2, 0).contiguous().numpy().copy()  # channels-last, like the engine

        tap("conv_in")
        x = self._res(x, "decoder.mid_block.resnets.0")
        tap("mid0")
        x = self._attn(x, "decoder.mid_block.attentions.0")
        tap("attn")
        x = self._res(x, "decoder.mid_block.resnets.1")
        tap("mid1")
        for ub in range(4):
            for r in range(3):
                x = self._res(x, "decoder.up_blocks.%d.resnets.%d" % (ub, r))
                tap("up%d_%d" % (ub, r))
            if ub < 3:
                x = F.interpolate(x, scale_factor=2, mode="nearest")
                x = self._conv(x, "decoder.up_blocks.%d.upsamplers.0.conv" % ub, 1)
                tap("ups%d" % ub)
        x = self._conv(self._gn(x, "decoder.conv_norm_out", True), "decoder.conv_out", 1)
        f = x[0].numpy().copy()
        img = np.clip((f + 1.0) * 0.5 * 255.0, 0.0, 255.0).astype(np.uint8).transpose(1, 2, 0).copy()
        return img, f
