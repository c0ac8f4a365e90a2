"""The decoder in front of the Kokoro generator, wired from `ops.*_cuda`: five AdainResBlk1d blocks that turn the
aligned text features, the pitch curve and the energy curve into the generator's input x [512, 2F]
(models/kokoro/model.py:158-221 the blocks, :704-717 the stack). Same op sequence as the reference's CPU graph, fused
(stats -> adain_affine -> conv1d_leaky, :205-221) or basic (:158-174).

Its convs have 514 / 1090 / 1024 input channels and kernel size 3. The tensor-core kernel stages 16 input channels at
a time, so the two odd counts are padded here, once, when the weights are uploaded: the row concatenations that build
the block inputs append zero rows up to the next multiple of 16 and the weights / AdaIN parameters get zero columns
to match. A zero row has mean 0 and variance 0, its activation is the finite AdaIN bias, and it meets a zero weight:
the padding contributes exact zeros and every conv of the stack runs on tcgen05.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops
from .synth import DECODER_BLOCKS

SQRT1_2 = 0.7071067811865476


def _pad16(c: int) -> int:
    return -(-c // 16) * 16


class Decoder:
    def __init__(self, sd: dict, device="cuda"):
        self.device = torch.device(device)
        w = {k: ops.to_cuda(np.ascontiguousarray(v, dtype=np.float32), self.device) for k, v in sd.items()}
        self.w, self.state = w, {}
        self.gb_pad = {}  # block -> channels appended to norm1's (gamma, beta)
        for name, cin, cout, up in DECODER_BLOCKS:
            cp = _pad16(cin)
            if cp != cin:  # zero input channels / zero AdaIN parameters for the appended rows
                z = cp - cin
                w[name + ".conv1.weight"] = torch.cat(
                    [w[name + ".conv1.weight"], torch.zeros(cout, z, 3, device=self.device)], 1).contiguous()
                if cin != cout:
                    w[name + ".conv1x1.weight"] = torch.cat(
                        [w[name + ".conv1x1.weight"], torch.zeros(cout, z, 1, device=self.device)], 1).contiguous()
                if up:
                    w[name + ".pool.weight"] = torch.cat(
                        [w[name + ".pool.weight"], torch.zeros(z, 1, 3, device=self.device)], 0).contiguous()
                    w[name + ".pool.bias"] = torch.cat([w[name + ".pool.bias"], torch.zeros(z, device=self.device)])
            self.gb_pad[name] = cp - cin
            for conv in (".conv1", ".conv2"):
                self.state[name + conv] = ops.conv1d_prepare_f32_cuda(w[name + conv + ".weight"])
        # style bank: every `<name>.fc` of the decoder as one GEMV (models/kokoro/model.py:67-81, names sorted)
        names = sorted(k[: -len(".weight")] for k in w if k.endswith(".fc.weight"))
        self.bank_wt = torch.cat([w[n + ".weight"].t() for n in names], dim=1).contiguous()
        self.bank_b = torch.cat([w[n + ".bias"] for n in names]).contiguous()
        self.bank_off, o = {}, 0
        for n in names:
            self.bank_off[n] = (o, int(w[n + ".bias"].shape[0]))
            o += self.bank_off[n][1]
        self._ident = {}

    def _style(self, s):
        bank = ops.gemm_bias_f32_cuda(s.reshape(1, -1), self.bank_wt, self.bank_b).reshape(-1)

        def gb(name, pad=0):
            o, n = self.bank_off[name]
            v = bank[o: o + n]
            if pad:  # (gamma | beta) of the appended zero rows: zeros
                c = n // 2
                z = torch.zeros(pad, device=self.device)
                v = torch.cat([v[:c], z, v[c:], z])
            return v.contiguous()

        return gb

    def _identity(self, c):
        if c not in self._ident:
            self._ident[c] = torch.stack([torch.zeros(c), torch.ones(c), torch.zeros(c)]).to(self.device).contiguous()
        return self._ident[c]

    def _concat(self, parts, cin):
        """concat_rows of the block input, with zero rows up to the next multiple of 16 channels."""
        z = _pad16(cin) - cin
        if z:
            parts = list(parts) + [torch.zeros(z, parts[0].shape[1], device=self.device)]
        return ops.concat_rows_f32_cuda(*parts)

    def adain_resblk(self, x, gb, name, cin, cout, upsample):
        """AdainResBlk1d through the basic ops (models/kokoro/model.py:158-174). x carries the padded rows."""
        w, pad = self.w, self.gb_pad[name]
        r = ops.leaky_relu_f32_cuda(ops.adain1d_f32_cuda(x, gb(name + ".norm1.fc", pad)), slope=0.2)
        if upsample:
            r = ops.conv_transpose1d_dw_f32_cuda(r, w[name + ".pool.weight"], w[name + ".pool.bias"], stride=2,
                                                 padding=1, output_padding=1)
        r = ops.conv1d_f32_cuda(r, w[name + ".conv1.weight"], w[name + ".conv1.bias"], padding=1)
        r = ops.leaky_relu_f32_cuda(ops.adain1d_f32_cuda(r, gb(name + ".norm2.fc")), slope=0.2)
        r = ops.conv1d_f32_cuda(r, w[name + ".conv2.weight"], w[name + ".conv2.bias"], padding=1)
        sc = ops.upsample_nearest1d_f32_cuda(x, scale=2) if upsample else x
        if cin != cout:
            sc = ops.conv1d_nobias_f32_cuda(sc, w[name + ".conv1x1.weight"])
        return ops.scale_f32_cuda(ops.add_f32_cuda(r, sc), scale=SQRT1_2)

    def adain_resblk_fused(self, x, gb, name, cin, cout, upsample):
        """The block through the fused conv kernels (models/kokoro/model.py:205-221)."""
        w, pad = self.w, self.gb_pad[name]
        gb1 = gb(name + ".norm1.fc", pad)
        af = ops.adain_affine_f32_cuda(ops.channel_stats_f32_cuda(x), gb1, length=int(x.shape[1]))
        if upsample:
            r = ops.leaky_relu_f32_cuda(ops.adain1d_f32_cuda(x, gb1), slope=0.2)
            r = ops.conv_transpose1d_dw_f32_cuda(r, w[name + ".pool.weight"], w[name + ".pool.bias"], stride=2,
                                                 padding=1, output_padding=1)
            h, st = ops.conv1d_affine_f32_cuda(r, w[name + ".conv1.weight"], w[name + ".conv1.bias"],
                                               self._identity(int(x.shape[0])), padding=1,
                                               state=self.state[name + ".conv1"])
        else:
            h, st = ops.conv1d_leaky_f32_cuda(x, w[name + ".conv1.weight"], w[name + ".conv1.bias"], af, slope=0.2,
                                              padding=1, state=self.state[name + ".conv1"])
        af = ops.adain_affine_f32_cuda(st, gb(name + ".norm2.fc"), length=int(h.shape[1]))
        sc = ops.upsample_nearest1d_f32_cuda(x, scale=2) if upsample else x
        if cin != cout:
            sc = ops.conv1d_nobias_f32_cuda(sc, w[name + ".conv1x1.weight"])
        out, _ = ops.conv1d_leaky_f32_cuda(h, w[name + ".conv2.weight"], w[name + ".conv2.bias"], af, slope=0.2,
                                           residual=sc, out_scale=SQRT1_2, padding=1,
                                           state=self.state[name + ".conv2"])
        return out

    def forward(self, asr, f0, n_curve, s, fused=True):
        """asr f32[512, F], f0 / n_curve f32[2F], s f32[128] (cuda tensors) -> x f32[512, 2F], the generator's input
        (models/kokoro/model.py:704-717)."""
        w = self.w
        ops.check(asr.dim() == 2 and asr.shape[0] == 512, "asr must be f32[512, F]")
        frames = int(asr.shape[1])
        ops.check(tuple(f0.shape) == (2 * frames,) and tuple(n_curve.shape) == (2 * frames,),
                  "f0 and n_curve must be f32[2F]")
        gb = self._style(s)
        f0d = ops.conv1d_f32_cuda(f0.reshape(1, -1), w["decoder.F0_conv.weight"], w["decoder.F0_conv.bias"], stride=2,
                                  padding=1)
        nd = ops.conv1d_f32_cuda(n_curve.reshape(1, -1), w["decoder.N_conv.weight"], w["decoder.N_conv.bias"],
                                 stride=2, padding=1)
        blk = self.adain_resblk_fused if fused else self.adain_resblk
        name, cin, cout, up = DECODER_BLOCKS[0]
        x = blk(self._concat([asr, f0d, nd], cin), gb, name, cin, cout, up)
        asr_res = ops.conv1d_f32_cuda(asr, w["decoder.asr_res.0.weight"], w["decoder.asr_res.0.bias"])
        for name, cin, cout, up in DECODER_BLOCKS[1:]:
            x = blk(self._concat([x, asr_res, f0d, nd], cin), gb, name, cin, cout, up)
        return x
