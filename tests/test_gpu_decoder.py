"""The decoder AdainResBlk1d stack in front of the generator (models/kokoro/model.py:158-221, 704-717) on the GPU
against the CPU oracle: its three extra ops, each block type (basic and fused), and the whole stack's output dec_x."""
import math

import numpy as np
import pytest
import torch

from lokinfer_b200 import synth
from oracle import kokoro_oracle as O
from util import REL_L2, rel_l2, t32, t64

pytestmark = pytest.mark.gpu


def dev(cuda, *arrs):
    from lokinfer_b200 import ops
    return [ops.to_cuda(a, cuda) for a in arrs]


def test_decoder_side_ops(cuda):
    from lokinfer_b200 import ops
    r = np.random.default_rng(3)
    # depthwise ConvTranspose1d: (C, L, K, stride, padding, output_padding), incl. the pool of the upsampling block
    for c, l, k, s, p, op in [(1090, 37, 3, 2, 1, 1), (5, 1, 3, 2, 1, 1), (8, 33, 4, 2, 1, 0), (3, 10, 5, 3, 0, 2),
                              (16, 700, 3, 1, 1, 0)]:
        x = r.standard_normal((c, l)).astype(np.float32)
        w = r.standard_normal((c, 1, k)).astype(np.float32)
        b = r.standard_normal(c).astype(np.float32)
        got = ops.conv_transpose1d_dw_f32_cuda(*dev(cuda, x, w, b), stride=s, padding=p, output_padding=op).cpu().numpy()
        ref = O.conv_transpose1d_dw(t64(x), t64(w), t64(b), stride=s, padding=p, output_padding=op).numpy()
        assert got.shape == ref.shape == (c, (l - 1) * s - 2 * p + k + op)
        np.testing.assert_allclose(got, ref, atol=1e-5, rtol=1e-5)
    for c, l, sc in [(7, 13, 2), (1104, 40, 2), (3, 5, 1), (2, 9, 3)]:
        x = r.standard_normal((c, l)).astype(np.float32)
        got = ops.upsample_nearest1d_f32_cuda(dev(cuda, x)[0], sc).cpu().numpy()
        np.testing.assert_array_equal(got, O.upsample_nearest1d(t32(x), sc).numpy())
    parts = [r.standard_normal((n, 21)).astype(np.float32) for n in (1024, 64, 1, 1, 14)]
    got = ops.concat_rows_f32_cuda(*dev(cuda, *parts)).cpu().numpy()
    np.testing.assert_array_equal(got, np.concatenate(parts, 0))
    with pytest.raises(ops.OpError):
        ops.concat_rows_f32_cuda(dev(cuda, parts[0])[0])


@pytest.mark.parametrize("frames", [9, 40, 160])
@pytest.mark.parametrize("fused", [True, False])
def test_decoder_vs_oracle(cuda, frames, fused):
    """dec_x [512, 2F] (the generator's input) for F frames. Ten chained convs of 514 .. 1090 input channels: the
    per-op bar compounds, the float64 oracle is the arbiter (GPU error within 2x the float32 oracle's own)."""
    from lokinfer_b200 import Decoder, ops
    sd = synth.decoder_weights(0)
    inp = synth.decoder_inputs(frames, 5 + frames)
    dec = Decoder(sd, cuda)
    a = dev(cuda, inp["asr"], inp["f0"], inp["n"], inp["s"])
    got = dec.forward(*a, fused=fused).cpu().numpy()
    assert got.shape == (512, 2 * frames)
    r32 = O.decoder(sd, *[O.T(inp[k]) for k in ("asr", "f0", "n", "s")], fused=fused).numpy()
    dt = torch.float64
    r64 = O.decoder(sd, *[O.T(inp[k], dt) for k in ("asr", "f0", "n", "s")], fused=fused).numpy()
    assert rel_l2(got, r32) <= 10 * REL_L2
    assert rel_l2(got, r64) <= 2 * rel_l2(r32, r64) + 1e-6
    assert ops.conv_tc_status() == 0
    if fused:  # every conv of the fused stack has a prepared tensor-core state (padded input channels)
        assert all(st is not None for st in dec.state.values())


def test_decoder_feeds_generator(cuda):
    """dec_x goes straight into the generator: decoder -> generator on the device equals the oracle's chain."""
    from lokinfer_b200 import Decoder, Generator, ops
    frames = 8
    dsd, gsd = synth.decoder_weights(0), synth.generator_weights(0)
    inp = synth.decoder_inputs(frames, 2)
    gin = synth.generator_inputs(2 * frames, 4)
    dec, gen = Decoder(dsd, cuda), Generator(gsd, cuda)
    x = dec.forward(*dev(cuda, inp["asr"], inp["f0"], inp["n"], inp["s"]))
    audio = gen.forward(x, *dev(cuda, gin["har"], inp["s"])).cpu().numpy()
    rx = O.decoder(dsd, *[O.T(inp[k]) for k in ("asr", "f0", "n", "s")])
    ref = O.generator(gsd, rx, O.T(gin["har"]), O.T(inp["s"])).numpy()
    assert audio.shape == ref.shape == (600 * frames,)
    assert np.abs(audio - ref).max() <= 1e-4
