"""Host logic of the polyphase form of a strided conv (ops.polyphase_conv_weights + the space-to-depth view): pure
numpy, no GPU. conv1d(x, w, stride s, padding p) with K = taps * s equals the stride-1 conv of y[ci * s + r, t] =
x[ci, s t + r - p] with w'[co, ci * s + r, j] = w[co, ci, s j + r]."""
import numpy as np
import pytest
import torch

from lokinfer_b200 import ops


def _space_to_depth(x, s, p, taps, rows):
    ci, l = x.shape
    lo = (l + 2 * p - taps * s) // s + 1
    y = np.zeros((rows, lo + taps - 1), dtype=x.dtype)
    for c in range(ci):
        for r in range(s):
            for t in range(y.shape[1]):
                pos = s * t + r - p
                if 0 <= pos < l:
                    y[c * s + r, t] = x[c, pos]
    return y


@pytest.mark.parametrize("ci,co,l,k,s,p", [(22, 8, 61, 12, 6, 3), (22, 8, 40, 1, 1, 0), (5, 4, 50, 6, 3, 2),
                                           (3, 2, 33, 4, 2, 0)])
def test_polyphase_weights_and_view_reproduce_the_strided_conv(ci, co, l, k, s, p):
    rng = np.random.default_rng(k * 100 + l)
    x = rng.standard_normal((ci, l))
    w = rng.standard_normal((co, ci, k))
    rows = -(-ci * s // 16) * 16
    wp = ops.polyphase_conv_weights(w.astype(np.float32), s, rows).astype(np.float64)
    assert wp.shape == (co, rows, k // s) and not wp[:, ci * s:, :].any()
    y = _space_to_depth(x, s, p, k // s, rows)
    want = torch.nn.functional.conv1d(torch.from_numpy(x)[None], torch.from_numpy(w), stride=s, padding=p)[0].numpy()
    got = torch.nn.functional.conv1d(torch.from_numpy(y)[None], torch.from_numpy(wp))[0].numpy()
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-5)  # w' went through float32


def test_polyphase_weights_reject_a_kernel_that_is_not_a_multiple_of_the_stride():
    with pytest.raises(ops.OpError):
        ops.polyphase_conv_weights(np.zeros((2, 3, 7), np.float32), 3)
    with pytest.raises(ops.OpError):
        ops.polyphase_conv_weights(np.zeros((2, 3, 6), np.float32), 3, rows=8)
