"""Shared helpers for the parity tests: error metrics and the tolerances used throughout.

REL_L2 (<= 1e-5 per op) and WAVE_MAXABS (<= 1e-4 on the final waveform) are the bars for the CUDA path against the
float32 oracle on identical seeded inputs. The float64 recipes use the reference's own tolerances
(tests/kernels/test_kokoro_conv_fused.py:1-7, tests/kernels/test_kokoro_kernels.py:3-14)."""
import numpy as np
import torch

REL_L2 = 1e-5
WAVE_MAXABS = 1e-4


def rel_l2(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    d = np.linalg.norm((got - ref).ravel())
    n = np.linalg.norm(ref.ravel())
    return d / n if n > 0 else d


def t32(a):
    return torch.from_numpy(np.ascontiguousarray(np.asarray(a, dtype=np.float32)))


def t64(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float64))


def stats_ref64(y, tile=128):
    """Chunk (mean, M2) in float64 numpy (tests/kernels/test_kokoro_conv_fused.py:65-73)."""
    y = np.asarray(y, dtype=np.float64)
    out = []
    for t0 in range(0, y.shape[1], tile):
        seg = y[:, t0:t0 + tile]
        m = seg.mean(axis=1)
        out.append(np.stack([m, ((seg - m[:, None]) ** 2).sum(axis=1)], axis=1))
    return np.stack(out, axis=1)


def check_stats(stats, y):
    ref = stats_ref64(y)
    stats = np.asarray(stats)
    assert stats.shape == ref.shape
    np.testing.assert_allclose(stats[..., 0], ref[..., 0], atol=2e-5, rtol=2e-5)
    np.testing.assert_allclose(stats[..., 1], ref[..., 1], atol=2e-4, rtol=1e-4)
