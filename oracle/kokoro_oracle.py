"""CPU oracle for the Kokoro iSTFTNet generator path. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this module; the
product package never does. It is a torch/numpy restatement (public torch ops only) of the reference's f32 CPU
kernels and graph for this path, each function citing the reference file:line it follows.

Pinning: the reference's own implementation cannot be built or imported on an x86-64 Linux host (Apple-only
headers, aarch64 intrinsics, a nanobind extension for Python >= 3.14) and the repo stores no golden vectors for
this path; its kernel tests are seeded recipes that compare each op with a torch float64 composition
(tests/kernels/test_kokoro_conv_fused.py, tests/kernels/test_kokoro_kernels.py). This oracle is pinned per op
and per AdaINResBlock1 iteration against those same recipes (tests/test_oracle.py). Whole-generator parity is
UNPINNED: the reference checks it against the third-party `kokoro==0.7.16` PyTorch modules, which are absent; the
same holds for harmonic_source (parity unpinned: two independent restatements are checked against each other), while
stft_magphase is pinned against torch.stft.

Every function takes/returns torch CPU tensors and works in the dtype of its inputs (float32 = the reference's
precision, float64 = golden).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

STAT_CHUNK = 128  # include/lokinfer/kernels/cpu_kokoro.h:96 (kStatChunk)
DILATIONS = (1, 3, 5)
RES_KERNELS = (3, 7, 11)


def T(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(np.asarray(a))).to(dtype)


# ----------------------------------------------------------------------------- shape rules (integers, exact)

def conv_out_len(l, k, stride, padding, dilation):
    """python/lokinfer/ops/kokoro.py:223-224."""
    return (l + 2 * padding - dilation * (k - 1) - 1) // stride + 1


def convt_out_len(l, k, stride, padding, output_padding=0):
    """python/lokinfer/ops/kokoro.py:264-265."""
    return (l - 1) * stride - 2 * padding + k + output_padding


def stat_chunks(l):
    """kernels/cpu/kokoro_conv_fused.cpp:78."""
    return (l + STAT_CHUNK - 1) // STAT_CHUNK


def istft_len(l, hop=5):
    """python/lokinfer/ops/kokoro.py:459."""
    return (l - 1) * hop


# ----------------------------------------------------------------------------- basic ops (the unfused layer)

def conv1d(x, w, b=None, stride=1, padding=0, dilation=1):
    """F.conv1d over x [Ci, L] (kernels/cpu/kokoro_conv.cpp:32-69)."""
    return F.conv1d(x[None], w, b, stride=stride, padding=padding, dilation=dilation)[0]


def conv_transpose1d(x, w, b=None, stride=1, padding=0, output_padding=0):
    """F.conv_transpose1d over x [Ci, L], w [Ci, Co, K] (kernels/cpu/kokoro_conv.cpp:71-95)."""
    return F.conv_transpose1d(x[None], w, b, stride=stride, padding=padding, output_padding=output_padding)[0]


def leaky_relu(x, slope):
    """kernels/cpu/kokoro_misc.cpp:172-180."""
    return F.leaky_relu(x, slope)


def snake(x, alpha):
    """x + (1/alpha) sin(alpha x)^2, alpha [C] (kernels/cpu/kokoro_misc.cpp:197-214)."""
    a = alpha.reshape(-1, 1)
    return x + (1.0 / a) * torch.sin(a * x) ** 2


def add(a, b):
    return a + b


def add3_scale(a, b, c, scale):
    """((a + b) + c) * scale (kernels/cpu/kokoro_misc.cpp:189-195)."""
    return ((a + b) + c) * scale


def pad_reflect1d(x, left, right):
    """F.pad(mode='reflect') (kernels/cpu/kokoro_conv.cpp:249-258)."""
    return F.pad(x[None], (left, right), mode="reflect")[0]


def instance_norm(x, eps=1e-5):
    m = x.mean(dim=-1, keepdim=True)
    return (x - m) / torch.sqrt(((x - m) ** 2).mean(dim=-1, keepdim=True) + eps)


def adain1d(x, gb, eps=1e-5):
    """(1 + gb[:C]) * instance_norm(x) + gb[C:], biased variance (kernels/cpu/kokoro_norm.cpp:49-58)."""
    c = x.shape[0]
    return (1 + gb[:c, None]) * instance_norm(x, eps) + gb[c:, None]


# ----------------------------------------------------------------------------- fused-layer ops

def channel_stats(x):
    """Per-(channel, 128-sample chunk) (mean, M2 = sum (v - mean)^2): [C, L] -> [C, ceil(L/128), 2]
    (kernels/cpu/kokoro_conv_fused.cpp:41-46, 631-639). Sums are taken in double and rounded to the working dtype,
    as the reference's blocked sums are; the deviation pass uses the rounded mean."""
    c, l = x.shape
    n = stat_chunks(l)
    out = torch.empty(c, n, 2, dtype=x.dtype)

    def seg_stats(seg):  # seg [c, m, len]
        mean = (seg.double().sum(dim=-1) / seg.shape[-1]).to(x.dtype)
        dev = seg - mean[..., None]
        return mean, (dev * dev).double().sum(dim=-1).to(x.dtype)

    full = l // STAT_CHUNK
    if full:
        out[:, :full, 0], out[:, :full, 1] = seg_stats(x[:, :full * STAT_CHUNK].reshape(c, full, STAT_CHUNK))
    if full < n:
        m, q = seg_stats(x[:, None, full * STAT_CHUNK:])
        out[:, full, 0], out[:, full, 1] = m[:, 0], q[:, 0]
    return out


def adain_affine(stats, gb, length, eps=1e-5):
    """Chan combine of the chunk partials in double, then affine rows (mean, (1 + g) / sqrt(var + eps), b):
    -> [3, C] (kernels/cpu/kokoro_conv_fused.cpp:641-664). var is biased and rounded to the working dtype before
    the rsqrt, as in the reference."""
    c, n, _ = stats.shape
    assert n == stat_chunks(length)
    dt = stats.dtype
    cnt = torch.full((n,), float(STAT_CHUNK), dtype=torch.float64)
    cnt[-1] = length - (n - 1) * STAT_CHUNK
    m = stats[:, :, 0].double()
    mean = (m * cnt).sum(dim=1) / length
    m2 = stats[:, :, 1].double().sum(dim=1) + (cnt * (m - mean[:, None]) ** 2).sum(dim=1)
    var = (m2 / length).to(dt)
    mean = mean.to(dt)
    scale = (1 + gb[:c]) * (1.0 / torch.sqrt(var + torch.tensor(eps, dtype=dt)))
    return torch.stack([mean, scale, gb[c:].clone()])


def conv1d_fused(x, w, b, affine, act="none", alpha=None, slope=0.0, residual=None, out_scale=1.0, padding=0,
                 dilation=1, mean3=None):
    """(conv1d(act((x - mean) * scale + beta), w) + b [+ residual]) * out_scale and the output's chunk stats
    (kernels/cpu/kokoro_conv_fused.cpp:117-150; zero padding is applied after the activation, :127-135).
    mean3 = (x2, x3, in_scale): the input is ((x + x2) + x3) * in_scale first (cpu_kokoro.h:113-115)."""
    if mean3 is not None:
        x = add3_scale(x, mean3[0], mean3[1], mean3[2])
    xa = (x - affine[0][:, None]) * affine[1][:, None] + affine[2][:, None]
    if act == "snake":
        xa = snake(xa, alpha)
    elif act == "leaky":
        xa = F.leaky_relu(xa, slope)
    else:
        assert act == "none"
    out = conv1d(xa, w, b, padding=padding, dilation=dilation)
    if residual is not None:
        out = out + residual
        if out_scale != 1.0:
            out = out * out_scale
    return out, channel_stats(out)


def conv_transpose1d_poly(x, w, b, res, stride, padding, slope, pad_left=0, mean3=None):
    """reflect_pad_left(conv_transpose1d(leaky(xin, slope), w, b, stride, padding), pad_left) + res with
    xin = x or ((x + x2) + x3) * in_scale (kernels/cpu/kokoro_conv.cpp:139-229; out[:, 0] = unpadded[:, 1] at :226).
    w is the torch ConvTranspose1d weight [Ci, Co, K], K = taps * stride, 2 p = (taps - 1) * stride."""
    k = w.shape[2]
    taps = k // stride
    assert taps * stride == k and 2 * padding == (taps - 1) * stride and 0 <= padding < stride
    if mean3 is not None:
        x = add3_scale(x, mean3[0], mean3[1], mean3[2])
    y = conv_transpose1d(F.leaky_relu(x, slope), w, b, stride=stride, padding=padding)
    assert y.shape[1] == x.shape[1] * stride
    if pad_left:
        y = torch.cat([y[:, 1:2], y], dim=1)
    return y + res


def hann_periodic(n, dtype):
    """kernels/cpu/kokoro_signal.cpp:33-36: computed in double, rounded to the working dtype."""
    i = torch.arange(n, dtype=torch.float64)
    return (0.5 - 0.5 * torch.cos(2.0 * math.pi * i / n)).to(dtype)


def istft_logits(x, n_fft=20, hop=5):
    """Explicit restatement of kernels/cpu/kokoro_signal.cpp:275-359: X_k = exp(x[k]) e^{i sin(x[K+k])},
    windowed inverse real DFT per frame, overlap-add as a gather per output sample with frames in ascending
    order, divided by the window-square envelope: [n_fft+2, L] -> [hop (L-1)]."""
    bins, pad = n_fft // 2 + 1, n_fft // 2
    l = x.shape[1]
    dt = x.dtype
    win = hann_periodic(n_fft, dt)
    k = torch.arange(bins, dtype=torch.float64)[:, None]
    m = torch.arange(n_fft, dtype=torch.float64)[None, :]
    ang = 2.0 * math.pi * torch.remainder(k * m, n_fft) / n_fft
    edge = ((k == 0) | (2 * k == n_fft)).double()
    cw = (2.0 - edge) * win.double()[None, :] / n_fft
    tab_re = (cw * torch.cos(ang)).to(dt)  # [bins, n_fft]
    tab_im = ((1.0 - edge) * (-cw) * torch.sin(ang)).to(dt)
    mag = torch.exp(x[:bins])
    ph = torch.sin(x[bins:])
    re, im = mag * torch.cos(ph), mag * torch.sin(ph)  # [bins, L]
    fr = tab_re.t() @ re + tab_im.t() @ im  # [n_fft, L] frame-minor like the kernel's fr[m][t]
    length = hop * (l - 1)
    i = torch.arange(length)
    p = pad + i
    t_hi = torch.clamp(p // hop, max=l - 1)
    t_lo = torch.where(p >= n_fft, (p - n_fft) // hop + 1, torch.zeros_like(p))
    y = torch.zeros(length, dtype=dt)
    env = torch.zeros(length, dtype=dt)
    w2 = win * win
    span = n_fft // hop
    for j in range(span):  # ascending t = t_lo + j
        t = t_lo + j
        ok = t <= t_hi
        tt = torch.where(ok, t, t_lo)
        mm = p - tt * hop
        y = y + torch.where(ok, fr[mm, tt], torch.zeros((), dtype=dt))
        env = env + torch.where(ok, w2[mm], torch.zeros((), dtype=dt))
    return y / env


def istft_logits_torch(x, n_fft=20, hop=5):
    """The documented equivalent (python/lokinfer/ops/kokoro.py:462-465):
    torch.istft(exp(x[:K]) e^{i sin(x[K:])}, periodic hann, center)."""
    bins = n_fft // 2 + 1
    mag, ph = torch.exp(x[:bins]), torch.sin(x[bins:])
    spec = torch.complex(mag * torch.cos(ph), mag * torch.sin(ph))
    win = torch.hann_window(n_fft, periodic=True, dtype=x.dtype, device=x.device)
    return torch.istft(spec[None], n_fft, hop_length=hop, win_length=n_fft, window=win, center=True)[0]


# ----------------------------------------------------------------------------- graph (models/kokoro/model.py)

# --- harmonic source + STFT: the producer of the generator's `har` input (kernels/cpu/kokoro_signal.cpp:97-272) ----
# The reference pins these two ops against the third-party kokoro modules (SourceModuleHnNSF, TorchSTFT), which are
# absent here. harmonic_source below restates the reference KERNEL's float32 operation sequence (its header comment
# spells out the torch ops it mirrors); stft_magphase is pinned against torch.stft (tests/test_oracle.py).

SOURCE_UP = 300          # kokoro_signal.cpp:19 (kUp = prod(upsample_rates) * hop)
SOURCE_HARMONICS = 9     # :18
SOURCE_RATE = 24000.0    # :20
SOURCE_VOICED = 10.0     # :21
SOURCE_SINE_AMP = 0.1    # :22
SOURCE_NOISE_STD = 0.003  # :23


def _fma32(a, b, c):
    """float32 fused multiply-add of numpy arrays: the product of two float32 is exact in float64."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def harmonic_phase_table(f0):
    """p300[j, h] = phase of harmonic h at frame j times 300 (kokoro_signal.cpp:103-115): rad = remainder(f0 (h+1) /
    24000, 1) in float32, running sum in float64, phase = (float32(sum) * 2) * float32(pi), all in float32."""
    f0 = np.asarray(f0, np.float32)
    h = np.arange(1, SOURCE_HARMONICS + 1, dtype=np.float32)
    fn = f0[:, None] * h[None, :]
    rad = np.fmod(fn / np.float32(SOURCE_RATE), np.float32(1.0)).astype(np.float32)
    rad = np.where((rad != 0) & (rad < 0), rad + np.float32(1.0), rad).astype(np.float32)  # torch.remainder (:26-30)
    acc = np.cumsum(rad.astype(np.float64), axis=0)  # sequential float64 adds, like the reference's loop
    phase = (acc.astype(np.float32) * np.float32(2.0)) * np.float32(math.pi)
    return (phase * np.float32(SOURCE_UP)).astype(np.float32)


def harmonic_source(f0, noise, w, b):
    """Kokoro SourceModuleHnNSF as the reference kernel computes it (kokoro_signal.cpp:97-177): f0 f32[n] (one value
    per 80 Hz frame), noise f32[300 n, 9], w f32[9], b f32[1] -> f32[300 n]. Linear x300 upsampling of the phase table
    (align_corners = False: source index fma(1/300, i + 0.5, -0.5), value fma(t0, l0, t1 * l1)), sine * 0.1 where
    voiced (f0 > 10) plus noise * (0.003 voiced | 0.1 / 3 unvoiced), Linear(9 -> 1) accumulated harmonic by harmonic,
    tanh. numpy float32 throughout (torch tensors in, torch tensor out)."""
    f0 = np.asarray(f0, np.float32)
    noise = np.asarray(noise, np.float32)
    w = np.asarray(w, np.float32)
    b = np.asarray(b, np.float32)
    n = f0.shape[0]
    s = n * SOURCE_UP
    p300 = harmonic_phase_table(f0)
    i = np.arange(s, dtype=np.float32)  # exact below 2^24 samples (the reference converts i to float as well)
    scale = np.float32(1.0 / float(SOURCE_UP))
    real = np.maximum(_fma32(np.full(s, scale, np.float32), i + np.float32(0.5), np.full(s, -0.5, np.float32)),
                      np.float32(0.0))
    i0 = np.minimum(np.floor(real).astype(np.int64), n - 1)
    l1 = np.clip(real - i0.astype(np.float32), np.float32(0.0), np.float32(1.0)).astype(np.float32)
    l0 = (np.float32(1.0) - l1).astype(np.float32)
    i1 = i0 + (i0 < n - 1)
    voiced = f0[np.arange(s) // SOURCE_UP] > np.float32(SOURCE_VOICED)
    uv = voiced.astype(np.float32)
    amp = np.where(voiced, np.float32(SOURCE_NOISE_STD), np.float32(SOURCE_SINE_AMP) / np.float32(3.0)).astype(np.float32)
    y = np.zeros(s, np.float32)
    for h in range(SOURCE_HARMONICS):
        t0, t1 = p300[i0, h], p300[i1, h]
        phase = _fma32(t0, l0, (t1 * l1).astype(np.float32))
        sine = (np.sin(phase.astype(np.float64)).astype(np.float32) * np.float32(SOURCE_SINE_AMP)).astype(np.float32)
        v = ((sine * uv).astype(np.float32) + (amp * noise[:, h]).astype(np.float32)).astype(np.float32)
        y = (y + (v * w[h]).astype(np.float32)).astype(np.float32)
    return torch.from_numpy(np.tanh((y + b[0]).astype(np.float64)).astype(np.float32))


def philox4x32_10(counters, key):
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11), vectorised:
    counters uint32[..., 4], key (k0, k1) -> uint32[..., 4]. The round function and constants are the published ones;
    the reference uses the same (kernels/cpu/kokoro_signal.cpp:42-64)."""
    c = [counters[..., i].astype(np.uint64) for i in range(4)]
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    m0, m1, mask = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = c[0] * m0, c[2] * m1
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ k0, lo1, hi0 ^ c[3] ^ k1, lo0]
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & mask, (k1 + np.uint64(0xBB67AE85)) & mask
    return np.stack(c, axis=-1).astype(np.uint32)


def source_noise_philox(seed, samples):
    """The normal draw of harmonic_source_rng_f32_cpu (kernels/cpu/kokoro_signal.cpp:66-96): sample i, block blk in
    0..2: counters (i_lo, i_hi, blk, 0x6C6B6E7A), key = the 64-bit seed; Box-Muller in float32 on the word pairs
    (c0, c1), (c2, c3) -> normals 4 blk + (0, 1) and 4 blk + (2, 3); the first 9 are used. -> float32[samples, 9]."""
    i = np.arange(samples, dtype=np.uint64)
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    key = (seed & 0xFFFFFFFF, seed >> 32)
    out = np.zeros((samples, 12), dtype=np.float32)
    scale = np.float32(2.3283064e-10)
    for blk in range(3):
        ctr = np.stack([i & np.uint64(0xFFFFFFFF), i >> np.uint64(32), np.full(samples, blk, np.uint64),
                        np.full(samples, 0x6C6B6E7A, np.uint64)], axis=-1).astype(np.uint32)
        c = philox4x32_10(ctr, key)
        for q in range(2):
            u1 = (c[:, 2 * q].astype(np.float32) + np.float32(0.5)) * scale
            u2 = c[:, 2 * q + 1].astype(np.float32) * scale
            r = np.sqrt(np.float32(-2.0) * np.log(u1)).astype(np.float32)
            t = (np.float32(6.2831853) * u2).astype(np.float32)
            out[:, 4 * blk + 2 * q] = r * np.cos(t)
            out[:, 4 * blk + 2 * q + 1] = r * np.sin(t)
    return out[:, :SOURCE_HARMONICS].copy()


def harmonic_source_rng(f0, w, b, seed):
    """harmonic_source with the noise drawn from `seed` (python/lokinfer/ops/kokoro.py:429-435)."""
    f0 = np.asarray(f0, dtype=np.float32)
    return harmonic_source(f0, source_noise_philox(seed, f0.shape[0] * SOURCE_UP), w, b)


def harmonic_source_torch(f0, noise, w, b):
    """The torch-op form the reference kernel says it mirrors (kokoro_signal.cpp:98-103): remainder, cumsum (double),
    F.interpolate(linear, align_corners=False), sin, Linear, tanh. Agrees with harmonic_source except where this
    host's interpolate rounds the phase (~1e5 rad) differently by one ulp (no fused multiply-add)."""
    f0, noise, w, b = (torch.as_tensor(np.asarray(v, np.float32)) for v in (f0, noise, w, b))
    h = torch.arange(1, SOURCE_HARMONICS + 1, dtype=torch.float32)
    rad = torch.remainder(f0[:, None] * h[None, :] / SOURCE_RATE, 1.0)
    phase = (torch.cumsum(rad.double(), 0).float() * 2.0) * torch.tensor(math.pi, dtype=torch.float32)
    up = F.interpolate((phase * SOURCE_UP).t()[None], scale_factor=SOURCE_UP, mode="linear", align_corners=False)[0].t()
    uv = (f0.repeat_interleave(SOURCE_UP) > SOURCE_VOICED).float()[:, None]
    amp = uv * SOURCE_NOISE_STD + (1 - uv) * SOURCE_SINE_AMP / 3
    v = torch.sin(up) * SOURCE_SINE_AMP * uv + amp * noise
    return torch.tanh(v @ w + b)


def stft_len(s, hop=5):
    return s // hop + 1


def stft_magphase(x, n_fft=20, hop=5):
    """torch.stft(center, reflect, periodic hann(n_fft), onesided) -> cat(abs, angle): [S] -> [n_fft + 2, S // hop + 1]
    (python/lokinfer/ops/kokoro.py:447-449; the restated kernel is stft_magphase_explicit)."""
    win = hann_periodic(n_fft, x.dtype).to(x.device)
    z = torch.stft(x, n_fft, hop_length=hop, win_length=n_fft, window=win, center=True, pad_mode="reflect",
                   onesided=True, return_complex=True)
    return torch.cat([z.abs(), z.angle()], 0)


def stft_magphase_explicit(x, n_fft=20, hop=5):
    """The reference kernel (kokoro_signal.cpp:196-272): reflect-padded frames times a windowed DFT basis built in
    double and rounded to the working dtype, re / im accumulated over m = 0..n_fft-1 in order, imaginary part exactly 0
    at DC and Nyquist, mag = sqrt(re^2 + im^2), phase = atan2(im, re)."""
    s = x.shape[0]
    bins, pad, frames = n_fft // 2 + 1, n_fft // 2, s // hop + 1
    win = hann_periodic(n_fft, torch.float64).to(x.dtype).double()
    m = torch.arange(n_fft, dtype=torch.float64)
    k = torch.arange(bins, dtype=torch.float64)
    ang = 2.0 * math.pi * ((k[:, None] * m[None, :]) % n_fft) / n_fft
    cr = (win[None, :] * torch.cos(ang)).to(x.dtype)
    ci = (-win[None, :] * torch.sin(ang)).to(x.dtype)
    q = torch.arange(frames)[:, None] * hop + torch.arange(n_fft)[None, :] - pad
    q = torch.where(q < 0, -q, q)
    q = torch.where(q >= s, 2 * (s - 1) - q, q)
    fr = x[q]  # [frames, n_fft]
    re = torch.zeros(bins, frames, dtype=x.dtype)
    im = torch.zeros(bins, frames, dtype=x.dtype)
    for mm in range(n_fft):
        re = re + cr[:, mm:mm + 1] * fr[None, :, mm]
        im = im + ci[:, mm:mm + 1] * fr[None, :, mm]
    im[0] = 0.0
    if n_fft % 2 == 0:
        im[n_fft // 2] = 0.0
    return torch.cat([torch.sqrt(re * re + im * im), torch.atan2(im, re)], 0)


def style_bank(sd, s, names=None):
    """gb = Linear(128 -> 2C)(s) for every `<name>.fc` (models/kokoro/model.py:67-81, 135-144)."""
    names = names or sorted(k[: -len(".weight")] for k in sd if k.endswith(".fc.weight"))
    return {n: sd[n + ".weight"] @ s + sd[n + ".bias"] for n in names}


def adain_resblock1(x, gbs, sd, prefix, k):
    """Basic AdaINResBlock1 (models/kokoro/model.py:250-260)."""
    for j, d in enumerate(DILATIONS):
        xt = adain1d(x, gbs[f"{prefix}.adain1.{j}.fc"])
        xt = snake(xt, sd[f"{prefix}.alpha1.{j}"].reshape(-1))
        xt = conv1d(xt, sd[f"{prefix}.convs1.{j}.weight"], sd[f"{prefix}.convs1.{j}.bias"], padding=d * (k - 1) // 2,
                    dilation=d)
        xt = adain1d(xt, gbs[f"{prefix}.adain2.{j}.fc"])
        xt = snake(xt, sd[f"{prefix}.alpha2.{j}"].reshape(-1))
        xt = conv1d(xt, sd[f"{prefix}.convs2.{j}.weight"], sd[f"{prefix}.convs2.{j}.bias"], padding=(k - 1) // 2)
        x = xt + x
    return x


def adain_resblock1_fused(x, gbs, sd, prefix, k, x_stats=None):
    """Fused AdaINResBlock1 (models/kokoro/model.py:235-247): per dilation adain_affine -> conv1d_snake ->
    adain_affine -> conv1d_snake(+x); every conv emits the chunk stats of its output. Returns (x, stats)."""
    n = x.shape[1]
    st = channel_stats(x) if x_stats is None else x_stats
    for j, d in enumerate(DILATIONS):
        af = adain_affine(st, gbs[f"{prefix}.adain1.{j}.fc"], n)
        xt, st1 = conv1d_fused(x, sd[f"{prefix}.convs1.{j}.weight"], sd[f"{prefix}.convs1.{j}.bias"], af, "snake",
                               alpha=sd[f"{prefix}.alpha1.{j}"].reshape(-1), padding=d * (k - 1) // 2, dilation=d)
        af = adain_affine(st1, gbs[f"{prefix}.adain2.{j}.fc"], n)
        x, st = conv1d_fused(xt, sd[f"{prefix}.convs2.{j}.weight"], sd[f"{prefix}.convs2.{j}.bias"], af, "snake",
                             alpha=sd[f"{prefix}.alpha2.{j}"].reshape(-1), padding=(k - 1) // 2, residual=x)
    return x, st


SQRT1_2 = 0.7071067811865476


def conv_transpose1d_dw(x, w, b, stride=1, padding=0, output_padding=0):
    """Depthwise F.conv_transpose1d (python/lokinfer/ops/kokoro.py:367-371)."""
    return F.conv_transpose1d(x[None], w, b, stride=stride, padding=padding, output_padding=output_padding,
                              groups=x.shape[0])[0]


def upsample_nearest1d(x, scale):
    """F.interpolate(mode='nearest') with an integer scale (python/lokinfer/ops/kokoro.py:399-402)."""
    return x.repeat_interleave(scale, dim=1)


def adain_resblk(x, gb1, gb2, sd, prefix, cin, cout, upsample):
    """AdainResBlk1d through the basic ops (models/kokoro/model.py:158-174)."""
    r = leaky_relu(adain1d(x, gb1), 0.2)
    if upsample:
        r = conv_transpose1d_dw(r, sd[prefix + ".pool.weight"], sd[prefix + ".pool.bias"], stride=2, padding=1,
                                output_padding=1)
    r = conv1d(r, sd[prefix + ".conv1.weight"], sd[prefix + ".conv1.bias"], padding=1)
    r = leaky_relu(adain1d(r, gb2), 0.2)
    r = conv1d(r, sd[prefix + ".conv2.weight"], sd[prefix + ".conv2.bias"], padding=1)
    sc = upsample_nearest1d(x, 2) if upsample else x
    if cin != cout:
        sc = conv1d(sc, sd[prefix + ".conv1x1.weight"])
    return (r + sc) * SQRT1_2


def adain_resblk_fused(x, gb1, gb2, sd, prefix, cin, cout, upsample):
    """The same block through the fused conv contracts (models/kokoro/model.py:205-221): stats -> adain_affine ->
    conv1d_leaky -> adain_affine -> conv1d_leaky(+shortcut, x 1/sqrt 2); the upsample block keeps the basic AdaIN /
    leaky / depthwise-convT front and an identity affine on conv1."""
    dt = x.dtype
    af = adain_affine(channel_stats(x), gb1, x.shape[1])
    if upsample:
        r = leaky_relu(adain1d(x, gb1), 0.2)
        r = conv_transpose1d_dw(r, sd[prefix + ".pool.weight"], sd[prefix + ".pool.bias"], stride=2, padding=1,
                                output_padding=1)
        ident = torch.stack([torch.zeros(cin), torch.ones(cin), torch.zeros(cin)]).to(dt)
        h, st = conv1d_fused(r, sd[prefix + ".conv1.weight"], sd[prefix + ".conv1.bias"], ident, "none", padding=1)
    else:
        h, st = conv1d_fused(x, sd[prefix + ".conv1.weight"], sd[prefix + ".conv1.bias"], af, "leaky", slope=0.2,
                             padding=1)
    af = adain_affine(st, gb2, h.shape[1])
    sc = upsample_nearest1d(x, 2) if upsample else x
    if cin != cout:
        sc = conv1d(sc, sd[prefix + ".conv1x1.weight"])
    out, _ = conv1d_fused(h, sd[prefix + ".conv2.weight"], sd[prefix + ".conv2.bias"], af, "leaky", slope=0.2,
                          residual=sc, out_scale=SQRT1_2, padding=1)
    return out


DECODER_BLOCKS = (("decoder.encode", 514, 1024, False), ("decoder.decode.0", 1090, 1024, False),
                  ("decoder.decode.1", 1090, 1024, False), ("decoder.decode.2", 1090, 1024, False),
                  ("decoder.decode.3", 1090, 512, True))


def decoder(sd, asr, f0, n_curve, s, fused=True):
    """The decoder in front of the generator (models/kokoro/model.py:704-717): asr [512, F] aligned text features,
    f0 / n_curve [2F] pitch and energy curves, s [128] style -> x [512, 2F]."""
    dt = asr.dtype
    sd = {k: (v if torch.is_tensor(v) else T(v)).to(dt) for k, v in sd.items()}
    gbs = style_bank(sd, s)
    f0d = conv1d(f0.reshape(1, -1), sd["decoder.F0_conv.weight"], sd["decoder.F0_conv.bias"], stride=2, padding=1)
    nd = conv1d(n_curve.reshape(1, -1), sd["decoder.N_conv.weight"], sd["decoder.N_conv.bias"], stride=2, padding=1)
    blk = adain_resblk_fused if fused else adain_resblk
    x = torch.cat([asr, f0d, nd], 0)
    name, cin, cout, up = DECODER_BLOCKS[0]
    x = blk(x, gbs[name + ".norm1.fc"], gbs[name + ".norm2.fc"], sd, name, cin, cout, up)
    asr_res = conv1d(asr, sd["decoder.asr_res.0.weight"], sd["decoder.asr_res.0.bias"])
    for name, cin, cout, up in DECODER_BLOCKS[1:]:
        x = torch.cat([x, asr_res, f0d, nd], 0)
        x = blk(x, gbs[name + ".norm1.fc"], gbs[name + ".norm2.fc"], sd, name, cin, cout, up)
    return x


def generator(sd, x, har, s, fused=True, stages=False):
    """The generator part of the reference graph (models/kokoro/model.py:735-781): x [512, T] decoder features,
    har [22, 60 T + 1] harmonic-source STFT, s [128] style -> audio [300 T]. fused=False is the basic-kernel
    graph (:750-764, 779-780). stages=True also returns named intermediates."""
    dt = x.dtype
    sd = {k: (v if torch.is_tensor(v) else T(v)).to(dt) for k, v in sd.items()}
    gbs = style_bank(sd, s)
    st = {}
    rb = None
    for i, (k_up, u, k_noise) in enumerate(((20, 10, 7), (12, 6, 11))):
        if i == 0:
            xs = conv1d(har, sd["noise_convs.0.weight"], sd["noise_convs.0.bias"], stride=6, padding=3)
        else:
            xs = conv1d(har, sd["noise_convs.1.weight"], sd["noise_convs.1.bias"])
        if fused:
            xs, _ = adain_resblock1_fused(xs, gbs, sd, f"noise_res.{i}", k_noise)
            x = conv_transpose1d_poly(x if i == 0 else rb[0], sd[f"ups.{i}.weight"], sd[f"ups.{i}.bias"], xs, stride=u,
                                      padding=(k_up - u) // 2, slope=0.1, pad_left=1 if i == 1 else 0,
                                      mean3=None if i == 0 else (rb[1], rb[2], 1.0 / 3.0))
            xst = channel_stats(x)
            rb = [adain_resblock1_fused(x, gbs, sd, f"resblocks.{3 * i + j}", kk, xst)[0]
                  for j, kk in enumerate(RES_KERNELS)]
        else:
            xs = adain_resblock1(xs, gbs, sd, f"noise_res.{i}", k_noise)
            x = leaky_relu(x, 0.1)
            x = conv_transpose1d(x, sd[f"ups.{i}.weight"], sd[f"ups.{i}.bias"], stride=u, padding=(k_up - u) // 2)
            if i == 1:
                x = pad_reflect1d(x, 1, 0)
            x = x + xs
            rb = [adain_resblock1(x, gbs, sd, f"resblocks.{3 * i + j}", kk) for j, kk in enumerate(RES_KERNELS)]
            x = add3_scale(rb[0], rb[1], rb[2], 1.0 / 3.0)
        st[f"stage{i}"] = x if not fused else rb
    if fused:
        c = rb[0].shape[0]
        ident = torch.stack([torch.zeros(c), torch.ones(c), torch.zeros(c)]).to(dt)
        post, _ = conv1d_fused(rb[0], sd["conv_post.weight"], sd["conv_post.bias"], ident, "leaky", slope=0.01,
                               padding=3, mean3=(rb[1], rb[2], 1.0 / 3.0))
    else:
        post = conv1d(leaky_relu(x, 0.01), sd["conv_post.weight"], sd["conv_post.bias"], padding=3)
    audio = istft_logits(post)
    if stages:
        st["post"] = post
        st["audio"] = audio
        return st
    return audio
