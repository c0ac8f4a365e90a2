"""Seeded synthetic weights and inputs for the Kokoro iSTFTNet generator (random init, no checkpoint).

Weight names and shapes follow the reference graph builder (models/kokoro/model.py:735-781 and the
AdaINResBlock1 wiring at :235-260): weight norm already folded, Snake alphas stored [1, C, 1], every AdaIN
`fc` a Linear(128 -> 2C). Distributions: conv w ~ N(0, 1/(Ci*K)), ConvTranspose w ~ N(0, s/(Ci*K)) (as in
tests/kernels/test_kokoro_conv_fused.py:219), bias ~ N(0, 0.01), alpha ~ U(0.5, 1.5), fc weight ~ N(0, 1/128)
with zero bias, style ~ N(0, 1), activations ~ N(0, 1). Everything is numpy float32 on the host.
"""
from __future__ import annotations

import math

import numpy as np

STYLE_DIM = 128
N_BINS = 22  # n_fft + 2 = 22 logits rows / harmonic-source STFT rows
# (C, upsample kernel, upsample stride, noise-res kernel) per stage
STAGES = ((256, 20, 10, 7), (128, 12, 6, 11))
RES_KERNELS = (3, 7, 11)
DILATIONS = (1, 3, 5)


def shapes(t: int) -> dict:
    """Integer shape table for generator input length t (= 2F in the reference's frame count):
    L0 = 10 t after ups[0]; L1 = 60 t + 1 after ups[1] and its one-sample left reflect pad
    (models/kokoro/model.py:754-755); S = 5 (L1 - 1) = 300 t output samples (ops/kokoro.py:459)."""
    l0 = t * 10
    l1 = l0 * 6 + 1
    return {"T": t, "L0": l0, "L1": l1, "S": 5 * (l1 - 1)}


def _resblock(r, sd, prefix, c, k):
    for j in range(3):
        for n in (1, 2):
            sd[f"{prefix}.convs{n}.{j}.weight"] = (r.standard_normal((c, c, k)) / math.sqrt(c * k)).astype(np.float32)
            sd[f"{prefix}.convs{n}.{j}.bias"] = (r.standard_normal(c) * 0.1).astype(np.float32)
            sd[f"{prefix}.alpha{n}.{j}"] = r.uniform(0.5, 1.5, (1, c, 1)).astype(np.float32)
            sd[f"{prefix}.adain{n}.{j}.fc.weight"] = (
                r.standard_normal((2 * c, STYLE_DIM)) / math.sqrt(STYLE_DIM)).astype(np.float32)
            sd[f"{prefix}.adain{n}.{j}.fc.bias"] = np.zeros(2 * c, np.float32)


def generator_weights(seed: int = 0) -> dict[str, np.ndarray]:
    """Random-init state dict of the generator (weight norm folded). bias ~ N(0, 0.01) means std 0.1."""
    r = np.random.default_rng(seed)
    sd: dict[str, np.ndarray] = {}
    ci = 512
    for i, (c, ku, su, kn) in enumerate(STAGES):
        sd[f"ups.{i}.weight"] = (r.standard_normal((ci, c, ku)) * math.sqrt(su / (ci * ku))).astype(np.float32)
        sd[f"ups.{i}.bias"] = (r.standard_normal(c) * 0.1).astype(np.float32)
        knoise = 12 if i == 0 else 1
        sd[f"noise_convs.{i}.weight"] = (
            r.standard_normal((c, N_BINS, knoise)) / math.sqrt(N_BINS * knoise)).astype(np.float32)
        sd[f"noise_convs.{i}.bias"] = (r.standard_normal(c) * 0.1).astype(np.float32)
        _resblock(r, sd, f"noise_res.{i}", c, kn)
        for j, k in enumerate(RES_KERNELS):
            _resblock(r, sd, f"resblocks.{3 * i + j}", c, k)
        ci = c
    # conv_post is drawn 10x smaller than N(0, 1/(C K)): its output is a log-magnitude that the iSTFT tail
    # exponentiates, and the resblock mean feeding it has std ~5 at random init; with the plain init the waveform
    # reaches ~5e4 and an absolute waveform tolerance would mean nothing. This keeps |audio| of order 1.
    sd["conv_post.weight"] = (0.1 * r.standard_normal((N_BINS, 128, 7)) / math.sqrt(128 * 7)).astype(np.float32)
    sd["conv_post.bias"] = (r.standard_normal(N_BINS) * 0.1).astype(np.float32)
    # Linear(9 -> 1) of the harmonic source that produces `har` (models/kokoro/model.py:720-726); drawn last so that
    # the weights above do not depend on it
    sd["m_source.l_linear.weight"] = (r.standard_normal((1, 9)) * 0.5).astype(np.float32)
    sd["m_source.l_linear.bias"] = (r.standard_normal(1) * 0.1).astype(np.float32)
    return sd


def generator_inputs(t: int, seed: int = 1) -> dict[str, np.ndarray]:
    """x f32[512, t] ~ N(0,1) (decoder features), har f32[22, 60 t + 1] ~ N(0,1) (stand-in for the harmonic-source
    STFT that feeds noise_convs), s f32[128] ~ N(0,1) (style)."""
    r = np.random.default_rng(seed)
    sh = shapes(t)
    return {
        "x": r.standard_normal((512, t)).astype(np.float32),
        "har": r.standard_normal((N_BINS, sh["L1"])).astype(np.float32),
        "s": r.standard_normal(STYLE_DIM).astype(np.float32),
    }


def fc_names(sd) -> list[str]:
    """Sorted `<...>.fc` prefixes: the style-bank order (models/kokoro/model.py:67-81)."""
    return sorted(k[: -len(".weight")] for k in sd if k.endswith(".fc.weight"))


def resblock_case(c: int, l: int, k: int, seed: int):
    """One AdaINResBlock1 (kernel k, dilations 1/3/5) at C channels: weights under prefix 'rb' + input + style."""
    r = np.random.default_rng(seed)
    sd: dict[str, np.ndarray] = {}
    _resblock(r, sd, "rb", c, k)
    x = r.standard_normal((c, l)).astype(np.float32)
    s = r.standard_normal(STYLE_DIM).astype(np.float32)
    return sd, x, s


def conv_case(ci: int, co: int, l: int, k: int, seed: int, big: bool = True):
    """Operands of one fused conv in the reference's own test distribution
    (tests/kernels/test_kokoro_conv_fused.py:54-62): x*2, affine mean N(0,.5) / scale U(.5,1.5) / beta N(0,.3),
    alpha U(.2,3); big=False gives the unit-scale variant (alpha U(.5,1.5))."""
    r = np.random.default_rng(seed)
    x = (r.standard_normal((ci, l)) * (2 if big else 1)).astype(np.float32)
    w = (r.standard_normal((co, ci, k)) / math.sqrt(ci * k)).astype(np.float32)
    b = r.standard_normal(co).astype(np.float32)
    affine = np.stack([r.standard_normal(ci) * 0.5, r.uniform(0.5, 1.5, ci), r.standard_normal(ci) * 0.3]).astype(
        np.float32)
    alpha = (r.uniform(0.2, 3.0, ci) if big else r.uniform(0.5, 1.5, ci)).astype(np.float32)
    res = r.standard_normal((co, max(l, 1))).astype(np.float32)
    return x, w, b, affine, alpha, res


def f0_curve(n: int, seed: int) -> np.ndarray:
    """An F0 contour at 80 Hz with the features the reference's test recipe exercises
    (tests/kernels/test_kokoro_kernels.py:477-488): smooth 70..400 Hz voiced stretches, unvoiced (0) gaps, values
    below the voicing threshold (10 Hz), first frame unvoiced."""
    r = np.random.default_rng(seed)
    t = np.arange(n)
    f0 = 180 + 90 * np.sin(t / 17.0 + seed) + 40 * np.sin(t / 5.3) + r.normal(0, 5, n)
    f0 = np.clip(f0, 70, 400)
    for _ in range(max(1, n // 40)):
        a = int(r.integers(0, n))
        f0[a:a + int(r.integers(2, 12))] = 0.0
    f0[r.integers(0, n, max(1, n // 50))] = r.uniform(0, 10)
    f0[0] = 0.0
    return f0.astype(np.float32)


def source_case(n: int, seed: int):
    """Seeded operands of the harmonic source for n frames: f0[n], noise[300n, 9], w[9], b[1]
    (distributions of tests/kernels/test_kokoro_kernels.py:511-516)."""
    r = np.random.default_rng(seed)
    f0 = f0_curve(n, seed)
    noise = r.standard_normal((300 * n, 9)).astype(np.float32)
    w = (r.standard_normal(9) * 0.5).astype(np.float32)
    b = (r.standard_normal(1) * 0.1).astype(np.float32)
    return f0, noise, w, b


DECODER_BLOCKS = (("decoder.encode", 514, 1024, False), ("decoder.decode.0", 1090, 1024, False),
                  ("decoder.decode.1", 1090, 1024, False), ("decoder.decode.2", 1090, 1024, False),
                  ("decoder.decode.3", 1090, 512, True))


def decoder_weights(seed: int = 0) -> dict[str, np.ndarray]:
    """Random-init weights of the decoder in front of the generator (names and shapes of models/kokoro/model.py:
    158-221, 704-717): five AdainResBlk1d (norm1.fc / norm2.fc Linear(128 -> 2C), conv1 / conv2 k 3, conv1x1 where the
    channel count changes, the depthwise pool of the upsampling block), asr_res (512 -> 64, k 1), F0_conv / N_conv
    (1 -> 1, k 3, stride 2). Conv weights ~ N(0, 1 / (Ci K)), biases ~ N(0, 0.01), fc weights ~ N(0, 1 / 128)."""
    r = np.random.default_rng(1000 + seed)
    sd = {}

    def conv(name, co, ci, k, bias=True):
        sd[name + ".weight"] = (r.standard_normal((co, ci, k)) / np.sqrt(ci * k)).astype(np.float32)
        if bias:
            sd[name + ".bias"] = (r.standard_normal(co) * 0.1).astype(np.float32)

    for name, cin, cout, up in DECODER_BLOCKS:
        for fc, c in ((".norm1.fc", cin), (".norm2.fc", cout)):
            sd[name + fc + ".weight"] = (r.standard_normal((2 * c, 128)) / np.sqrt(128)).astype(np.float32)
            sd[name + fc + ".bias"] = (r.standard_normal(2 * c) * 0.1).astype(np.float32)
        conv(name + ".conv1", cout, cin, 3)
        conv(name + ".conv2", cout, cout, 3)
        if cin != cout:
            conv(name + ".conv1x1", cout, cin, 1, bias=False)
        if up:
            sd[name + ".pool.weight"] = (r.standard_normal((cin, 1, 3)) / np.sqrt(3)).astype(np.float32)
            sd[name + ".pool.bias"] = (r.standard_normal(cin) * 0.1).astype(np.float32)
    conv("decoder.asr_res.0", 64, 512, 1)
    conv("decoder.F0_conv", 1, 1, 3)
    conv("decoder.N_conv", 1, 1, 3)
    return sd


def decoder_inputs(frames: int, seed: int = 1) -> dict[str, np.ndarray]:
    """asr f32[512, F] ~ N(0, 1), the F0 curve f32[2F] (Hz, voiced / unvoiced stretches), the energy curve f32[2F]
    ~ U(0, 4), style f32[128] ~ N(0, 1)."""
    r = np.random.default_rng(2000 + seed)
    return {"asr": r.standard_normal((512, frames)).astype(np.float32), "f0": f0_curve(2 * frames, seed),
            "n": r.uniform(0.0, 4.0, 2 * frames).astype(np.float32), "s": r.standard_normal(128).astype(np.float32)}
