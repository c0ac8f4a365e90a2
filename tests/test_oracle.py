"""Pins the CPU oracle against the reference's own kernel-test recipes (seeded inputs, torch float64 compositions,
the reference's tolerances): tests/kernels/test_kokoro_conv_fused.py and tests/kernels/test_kokoro_kernels.py.
Runs without a GPU."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from lokinfer_b200 import synth
from oracle import kokoro_oracle as O
from util import check_stats, rel_l2, t32, t64

torch.set_num_threads(1)


def randn(r, *shape, scale=1.0):
    return (r.standard_normal(shape) * scale).astype(np.float32)


def inorm64(v):
    m = v.mean(dim=-1, keepdim=True)
    return (v - m) / torch.sqrt(((v - m) ** 2).mean(dim=-1, keepdim=True) + 1e-5)


def snake64(x, a):
    return x + (1 / a) * torch.sin(a * x) ** 2


# (Ci, Co, L, K, dilation): the reference's CASES (test_kokoro_conv_fused.py:44-51)
CASES = [(8, 8, 50, 3, 1), (16, 12, 700, 7, 3), (12, 16, 97, 11, 5), (128, 128, 5000, 11, 5), (64, 64, 3000, 3, 1),
         (8, 8, 1, 3, 1)]


def _setup(ci, co, l, k, seed):
    r = np.random.default_rng(seed)
    x = randn(r, ci, l, scale=2)
    w = randn(r, co, ci, k, scale=1 / math.sqrt(ci * k))
    b = randn(r, co)
    affine = np.stack([randn(r, ci, scale=0.5), r.uniform(0.5, 1.5, ci), randn(r, ci, scale=0.3)]).astype(np.float32)
    alpha = r.uniform(0.2, 3.0, ci).astype(np.float32)
    res = randn(r, co, l)
    return x, w, b, affine, alpha, res


@pytest.mark.parametrize("ci,co,l,k,d", CASES)
@pytest.mark.parametrize("variant", ["snake", "snake_res", "leaky", "leaky_res", "affine"])
def test_conv1d_fused_recipe(ci, co, l, k, d, variant):
    x, w, b, affine, alpha, res = _setup(ci, co, l, k, ci * 31 + l + k)
    pad = d * (k - 1) // 2
    af = t64(affine)
    xa = (t64(x) - af[0][:, None]) * af[1][:, None] + af[2][:, None]
    kw = dict(padding=pad, dilation=d)
    if variant.startswith("snake"):
        xa = snake64(xa, t64(alpha)[:, None])
        out, stats = O.conv1d_fused(t32(x), t32(w), t32(b), t32(affine), "snake", alpha=t32(alpha),
                                    residual=t32(res) if variant == "snake_res" else None, **kw)
    elif variant.startswith("leaky"):
        xa = F.leaky_relu(xa, 0.2)
        rk = dict(residual=t32(res), out_scale=0.7071067811865476) if variant == "leaky_res" else {}
        out, stats = O.conv1d_fused(t32(x), t32(w), t32(b), t32(affine), "leaky", slope=0.2, **kw, **rk)
    else:
        out, stats = O.conv1d_fused(t32(x), t32(w), t32(b), t32(affine), "none", **kw)
    ref = F.conv1d(xa[None], t64(w), t64(b), padding=pad, dilation=d)[0]
    if variant == "snake_res":
        ref = ref + t64(res)
    if variant == "leaky_res":
        ref = (ref + t64(res)) * 0.7071067811865476
    assert out.shape == ref.shape
    np.testing.assert_allclose(out.numpy(), ref.numpy(), atol=1e-4, rtol=1e-4)
    check_stats(stats.numpy(), out.numpy())


@pytest.mark.parametrize("c,l", [(4, 1), (16, 700), (128, 5000)])
def test_channel_stats_and_adain_affine_recipe(c, l):
    r = np.random.default_rng(c + l)
    x = randn(r, c, l, scale=3) + 5
    gb = randn(r, 2 * c, scale=0.5)
    stats = O.channel_stats(t32(x))
    check_stats(stats.numpy(), x)
    af = O.adain_affine(stats, t32(gb), l).numpy()
    got = (x - af[0][:, None]) * af[1][:, None] + af[2][:, None]
    ref = (1 + t64(gb[:c])[:, None]) * inorm64(t64(x)[None])[0] + t64(gb[c:])[:, None]
    np.testing.assert_allclose(got, ref.numpy(), atol=2e-5 * max(1, np.abs(ref.numpy()).max()), rtol=1e-4)


def test_resblock1_iteration_recipe():
    """test_kokoro_conv_fused.py:166-199: one AdaINResBlock1 iteration through the fused ops vs torch float64."""
    c, k, d = 16, 7, 3
    r = np.random.default_rng(3)
    w1, w2 = (randn(r, c, c, k, scale=1 / math.sqrt(c * k)) for _ in range(2))
    b1, b2 = randn(r, c), randn(r, c)
    a1, a2 = (r.uniform(0.2, 3.0, c).astype(np.float32) for _ in range(2))
    gb1, gb2 = randn(r, 2 * c, scale=0.5), randn(r, 2 * c, scale=0.5)

    def adain64(v, gb):
        return (1 + t64(gb[:c])[:, None]) * inorm64(v) + t64(gb[c:])[:, None]

    for l in [5, 64, 1000]:
        x = randn(r, c, l)
        st = O.channel_stats(t32(x))
        af1 = O.adain_affine(st, t32(gb1), l)
        y, st = O.conv1d_fused(t32(x), t32(w1), t32(b1), af1, "snake", alpha=t32(a1), padding=d * (k - 1) // 2,
                               dilation=d)
        af2 = O.adain_affine(st, t32(gb2), l)
        z, _ = O.conv1d_fused(y, t32(w2), t32(b2), af2, "snake", alpha=t32(a2), residual=t32(x), padding=(k - 1) // 2)
        xt = t64(x)
        h = snake64(adain64(xt, gb1), t64(a1)[:, None])
        h = F.conv1d(h[None], t64(w1), t64(b1), padding=d * (k - 1) // 2, dilation=d)[0]
        h = snake64(adain64(h, gb2), t64(a2)[:, None])
        ref = (F.conv1d(h[None], t64(w2), t64(b2), padding=(k - 1) // 2)[0] + xt).numpy()
        np.testing.assert_allclose(z.numpy(), ref, atol=2e-4, rtol=2e-4)


# test_kokoro_conv_fused.py:204-212 (Ci, Co, L, K, s, pad_left)
CONVT_CASES = [(8, 32, 5, 4, 2, 0), (16, 40, 37, 8, 4, 1), (512, 256, 26, 20, 10, 0), (512, 256, 294, 20, 10, 0),
               (256, 128, 2940, 12, 6, 1), (256, 128, 1, 12, 6, 1), (64, 64, 700, 12, 6, 1)]


@pytest.mark.parametrize("ci,co,l,k,s,pl", CONVT_CASES)
def test_conv_transpose1d_poly_recipe(ci, co, l, k, s, pl):
    r = np.random.default_rng(ci + l + k)
    x = randn(r, ci, l, scale=2)
    w = randn(r, ci, co, k, scale=1 / math.sqrt(ci * k / s))
    b = randn(r, co)
    p = (k - s) // 2
    res = randn(r, co, l * s + pl)
    y = F.conv_transpose1d(F.leaky_relu(t64(x), 0.1), t64(w), t64(b), stride=s, padding=p)
    if pl:
        y = F.pad(y, (1, 0), mode="reflect") if y.shape[-1] > 1 else torch.cat([y, y], -1)
    ref = (y + t64(res)).numpy()
    out = O.conv_transpose1d_poly(t32(x), t32(w), t32(b), t32(res), s, p, 0.1, pad_left=pl).numpy()
    assert out.shape == ref.shape
    np.testing.assert_allclose(out, ref, atol=1e-4, rtol=1e-4)


def test_mean3_prologues_equal_add3_then_op():
    """test_kokoro_conv_fused.py:236-264: the 3-input-mean prologue equals add3_scale followed by the op."""
    r = np.random.default_rng(7)
    xs = [t32(randn(r, 16, 300)) for _ in range(3)]
    w, b = t32(randn(r, 8, 16, 7, scale=0.1)), t32(randn(r, 8))
    ident = torch.stack([torch.zeros(16), torch.ones(16), torch.zeros(16)])
    got, st = O.conv1d_fused(xs[0], w, b, ident, "leaky", slope=0.01, padding=3, mean3=(xs[1], xs[2], 1 / 3))
    m = O.add3_scale(xs[0], xs[1], xs[2], 1 / 3)
    exp, est = O.conv1d_fused(m, w, b, ident, "leaky", slope=0.01, padding=3)
    assert torch.equal(got, exp) and torch.equal(st, est)


@pytest.mark.parametrize("l", [2, 3, 7, 57, 1201])
def test_istft_two_restatements_agree(l):
    """The explicit DFT / overlap-add of kernels/cpu/kokoro_signal.cpp:275-359 equals torch.istft of
    exp(x[:K]) e^{i sin(x[K:])} (python/lokinfer/ops/kokoro.py:462-465) to 1e-6 * max|y|."""
    g = torch.Generator().manual_seed(l)
    for dt, tol in ((torch.float64, 1e-12), (torch.float32, 1e-6)):
        x = torch.randn(22, l, generator=g, dtype=torch.float64).to(dt)
        a, b = O.istft_logits(x), O.istft_logits_torch(x)
        assert a.shape == (5 * (l - 1),) == b.shape
        assert (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item())


@pytest.mark.parametrize("frames", [1, 3, 30, 119, 300])
def test_harmonic_source_two_restatements_agree(frames):
    """The float32 operation sequence of the reference kernel (kernels/cpu/kokoro_signal.cpp:97-177) and the torch-op
    form that kernel documents (remainder, double cumsum, linear interpolate, sin, Linear, tanh) agree within the
    reference's own tolerance for this op (2e-6, tests/kernels/test_kokoro_kernels.py:522), on its recipe's inputs
    (n = 2 * frames, the f0 curve with unvoiced gaps)."""
    n = 2 * frames
    f0, noise, w, b = synth.source_case(n, frames)
    a = O.harmonic_source(f0, noise, w, b)
    t = O.harmonic_source_torch(f0, noise, w, b)
    assert a.shape == t.shape == (600 * frames,)
    assert (a - t).abs().max().item() <= 2e-6
    assert a.abs().max().item() <= 1.0 and a.abs().max().item() > 1e-3
    # unvoiced first frame: no sine, only noise * 0.1 / 3 through the Linear + tanh
    uv0 = np.tanh((noise[:150] * (np.float32(0.1) / np.float32(3.0))) @ w + b[0])
    np.testing.assert_allclose(a[:150].numpy(), uv0, atol=1e-6)


@pytest.mark.parametrize("s", [11, 25, 600, 6001, 600 * 300])
def test_stft_magphase_recipe(s):
    """tests/kernels/test_kokoro_kernels.py:529-542: magnitude within 1e-5 * max, wrapped phase within 1e-4 where the
    bin is significant, against torch.stft (what TorchSTFT.transform computes); both the torch form and the explicit
    restatement of kernels/cpu/kokoro_signal.cpp:196-272."""
    r = np.random.default_rng(s)
    t = np.arange(s)
    x = (0.3 * np.sin(t * 0.05) + 0.2 * np.sin(t * 0.9) + 0.05 * r.standard_normal(s)).astype(np.float32)
    x[: s // 7] = 0.0  # silent stretch: DC / Nyquist bins with imag == 0
    ref = O.stft_magphase(torch.from_numpy(x).double()).numpy()
    mag, ph = ref[:11], ref[11:]
    for fn in (O.stft_magphase, O.stft_magphase_explicit):
        out = fn(torch.from_numpy(x)).numpy()
        assert out.shape == (22, O.stft_len(s)) == (22, s // 5 + 1)
        np.testing.assert_allclose(out[:11], mag, atol=1e-5 * mag.max(), rtol=0)
        sig = mag > 1e-3 * mag.max()
        dph = np.angle(np.exp(1j * (out[11:].astype(np.float64) - ph)))  # wrapped: the +-pi cut is not an error
        assert np.abs(dph[sig]).max() < 1e-4


def test_stft_frame_algebra():
    """The frame counts the generator relies on: S = 300 T source samples -> 60 T + 1 STFT frames (the length of
    `har`) -> 300 T waveform samples after the iSTFT."""
    for t in (1, 7, 320, 2080):
        s = 300 * t
        assert O.stft_len(s) == 60 * t + 1
        assert O.istft_len(O.stft_len(s)) == s


def test_basic_ops_recipes():
    """test_kokoro_kernels.py: snake (:333-341), add3_scale (:322-330), pad_reflect1d (:460-464), adain1d with a
    large mean (:437-449), conv1d incl. the noise_convs[0] shape (:347-383), conv_transpose1d (:404-424)."""
    r = np.random.default_rng(11)
    x = randn(r, 6, 257, scale=2)
    al = r.uniform(0.2, 3.0, 6).astype(np.float32)
    np.testing.assert_allclose(O.snake(t32(x), t32(al)).numpy(), snake64(t64(x), t64(al)[:, None]).numpy(), atol=1e-6,
                               rtol=1e-6)
    a, b, c = (randn(r, 5, 33) for _ in range(3))
    np.testing.assert_allclose(O.add3_scale(t32(a), t32(b), t32(c), 1 / 3).numpy(), (a + b + c) / 3, atol=1e-6, rtol=1e-6)
    assert torch.equal(O.pad_reflect1d(t32(x), 1, 0)[:, 0], t32(x)[:, 1])
    big = randn(r, 4, 135001) + 100
    gb = randn(r, 8, scale=0.5)
    ref = (1 + t64(gb[:4])[:, None]) * inorm64(t64(big)) + t64(gb[4:])[:, None]
    np.testing.assert_allclose(O.adain1d(t32(big), t32(gb)).numpy(), ref.numpy(), atol=2e-4, rtol=1e-4)
    xx, ww, bb = randn(r, 22, 1201), randn(r, 32, 22, 12, scale=0.1), randn(r, 32)
    ref = F.conv1d(t64(xx)[None], t64(ww), t64(bb), stride=6, padding=3)[0]
    out = O.conv1d(t32(xx), t32(ww), t32(bb), stride=6, padding=3)
    assert out.shape == (32, O.conv_out_len(1201, 12, 6, 3, 1))
    np.testing.assert_allclose(out.numpy(), ref.numpy(), atol=1e-4, rtol=1e-4)
    xt, wt, bt = randn(r, 16, 37), randn(r, 16, 12, 8, scale=0.1), randn(r, 12)
    ref = F.conv_transpose1d(t64(xt)[None], t64(wt), t64(bt), stride=4, padding=2)[0]
    out = O.conv_transpose1d(t32(xt), t32(wt), t32(bt), stride=4, padding=2)
    assert out.shape == (12, O.convt_out_len(37, 8, 4, 2))
    np.testing.assert_allclose(out.numpy(), ref.numpy(), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("t", [1, 4, 320, 2080])
def test_shape_table_is_exact(t):
    """Index / shape logic is integer-exact: L0 = 10 T, L1 = 60 T + 1, S = 300 T (models/kokoro/model.py:754-755)."""
    sh = synth.shapes(t)
    assert sh["L0"] == O.convt_out_len(t, 20, 10, 5) == 10 * t
    assert sh["L1"] == O.convt_out_len(sh["L0"], 12, 6, 3) + 1 == 60 * t + 1
    assert sh["S"] == O.istft_len(sh["L1"]) == 300 * t
    assert O.conv_out_len(sh["L1"], 12, 6, 3, 1) == sh["L0"]  # noise_convs[0] lands on the stage-0 length
    assert O.stat_chunks(sh["L1"]) == -(-sh["L1"] // 128)


def test_generator_fused_equals_basic():
    """The fused graph (model.py:235-247, 741-772) and the basic-kernel graph (:250-260, 750-780) are the same
    function: exact in float64 up to summation order, within f32 rounding in float32."""
    sd = synth.generator_weights(0)
    inp = synth.generator_inputs(6, 1)
    for dt, tol in ((torch.float64, 1e-11), (torch.float32, 2e-5)):
        args = [O.T(inp[k], dt) for k in ("x", "har", "s")]
        a = O.generator(sd, *args, fused=True)
        b = O.generator(sd, *args, fused=False)
        assert a.shape == (300 * 6,)
        assert (a - b).abs().max().item() <= tol
    assert rel_l2(a.numpy(), b.numpy()) < 1e-4


def test_philox_known_answers_and_source_noise():
    """Philox4x32-10 against the known-answer vectors published with the generator (Random123 kat_vectors), and the
    reference's counter layout / Box-Muller pairing (kernels/cpu/kokoro_signal.cpp:66-96): standard normals,
    deterministic per (seed, sample), independent of how many samples are drawn."""
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        got = O.philox4x32_10(np.array([ctr], dtype=np.uint32), key)[0]
        assert [int(v) for v in got] == list(want)
    nz = O.source_noise_philox(1234, 100000)
    assert nz.shape == (100000, 9) and nz.dtype == np.float32 and np.isfinite(nz).all()
    assert abs(float(nz.mean())) < 5e-3 and abs(float(nz.std()) - 1.0) < 5e-3
    np.testing.assert_array_equal(O.source_noise_philox(1234, 1000), nz[:1000])
    assert not np.array_equal(O.source_noise_philox(1235, 1000), nz[:1000])
    # first normal of sample 0, spelled out from its counter block
    c = O.philox4x32_10(np.array([[0, 0, 0, 0x6C6B6E7A]], dtype=np.uint32), (1234, 0))[0]
    u1 = (np.float32(c[0]) + np.float32(0.5)) * np.float32(2.3283064e-10)
    u2 = np.float32(c[1]) * np.float32(2.3283064e-10)
    z0 = np.sqrt(np.float32(-2) * np.log(u1)) * np.cos(np.float32(6.2831853) * u2)
    assert abs(float(nz[0, 0]) - float(z0)) < 1e-6


def test_decoder_fused_equals_basic():
    """The decoder stack through the fused conv contracts (models/kokoro/model.py:205-221) equals the basic-op stack
    (:158-174): the restated graph wiring is consistent (float64 so that only the wiring is tested)."""
    from lokinfer_b200 import synth
    sd = synth.decoder_weights(0)
    inp = synth.decoder_inputs(12, 1)
    a = [O.T(inp[k], torch.float64) for k in ("asr", "f0", "n", "s")]
    fused, basic = O.decoder(sd, *a, fused=True), O.decoder(sd, *a, fused=False)
    assert tuple(fused.shape) == (512, 24)
    assert (fused - basic).abs().max().item() <= 1e-9 * basic.abs().max().item()
