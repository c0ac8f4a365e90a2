"""The device-side harness (RUN2 data path): oracle pins on the CPU, GPU kernels against the oracle."""
import math

import numpy as np
import pytest
import torch

from oracle import run2_oracle as R


def test_splitmix_stream_matches_the_published_vector():
    """splitmix64 started at state 0: the first three outputs of the published reference implementation."""
    got = R.splitmix_at(0, np.arange(1, 4, dtype=np.uint64))
    assert [int(v) for v in got] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_oracle_generate_ranges_and_moments():
    """The checks the reference makes on its own generator (tests/python/test_remote.py:150-159)."""
    gx = R.generate([1000], 42)
    gy = R.generate([1000], 43, dist="uniform", a=-2, b=3)
    assert -2 <= gy.min() and gy.max() < 3 and abs(gx.mean()) < 0.1 and abs(gx.std() - 1) < 0.1
    ints = R.generate([10000], 5, np.int64, "int", 3, 9)
    assert ints.min() == 3 and ints.max() == 8
    assert R.generate([3, 4], 7).shape == (3, 4) and R.generate([], 7).shape == ()
    # element i depends on (seed, i) only
    np.testing.assert_array_equal(R.generate([10], 9)[:5], R.generate([5], 9))


def test_oracle_compare_stats_rules():
    ref = np.arange(8, dtype=np.float32)
    got = ref.copy()
    got[3] += 1.0
    got[6] += 1.0  # same excess as index 3: the first one is the worst
    s = R.compare_stats(got, ref, 0.0, 1e-3)
    assert (s["count"], s["nonfinite"], s["mismatches"], s["worst"]) == (8, 0, 2, 3)
    assert s["max_abs_err"] == 1.0 and s["max_abs_ref"] == 7.0 and s["sum_sq_err"] == 2.0 and s["sum_sq_ref"] == 140.0
    got = ref.copy()
    got[1], got[2] = np.nan, np.inf
    refn = ref.copy()
    refn[1] = np.nan
    s = R.compare_stats(got, refn, 0.0, 0.0)
    assert s["nonfinite"] == 2 and s["mismatches"] == 1  # NaN against NaN is not a mismatch, inf against 2 is
    assert s["sum_sq_ref"] == float((ref ** 2).sum() - 1 - 4)  # non-finite elements take no part in the sums
    assert R.compare_stats(np.zeros(0, np.float32), np.zeros(0, np.float32), 0, 0)["worst"] == -1


# ------------------------------------------------------------------------------------------------------------ GPU


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 1000, 300001])
def test_generate_matches_oracle(cuda, n):
    from lokinfer_b200 import run2
    for seed in (0, 42, 2 ** 63 + 5):
        u = run2.generate([n], seed, dist="uniform", a=-2, b=3, device=cuda).cpu().numpy()
        np.testing.assert_array_equal(u, R.generate([n], seed, dist="uniform", a=-2, b=3))
        i64 = run2.generate([n], seed, torch.int64, "int", 3, 9, device=cuda).cpu().numpy()
        np.testing.assert_array_equal(i64, R.generate([n], seed, np.int64, "int", 3, 9))
        i32 = run2.generate([n], seed, torch.int32, "int", -5.5, 1000.2, device=cuda).cpu().numpy()
        np.testing.assert_array_equal(i32, R.generate([n], seed, np.int32, "int", -5.5, 1000.2))
        g = run2.generate([n], seed, dist="normal", a=0.5, b=2.0, device=cuda).cpu().numpy()
        want = R.generate([n], seed, dist="normal", a=0.5, b=2.0)
        # to an ulp of f32: the device's double log / cos may round differently from the host's libm
        assert np.all(np.abs(g - want) <= np.spacing(np.abs(want)))
        assert np.mean(g != want) < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 77, 100003, 4000000])
def test_compare_matches_oracle(cuda, n):
    from lokinfer_b200 import run2
    rng = np.random.default_rng(n)
    ref = rng.standard_normal(n).astype(np.float32)
    got = ref + (rng.standard_normal(n) * 1e-6).astype(np.float32)
    if n > 50:
        got[17] += 1.0
        got[n // 2] += 1.0          # a tie for the worst excess only if ref is equal there: make it so
        ref[n // 2] = ref[17]
        got[n // 2] = got[17]
        got[5], ref[5] = np.nan, np.nan
        got[6] = np.inf
        got[n - 1] = -np.inf
        ref[n - 1] = -np.inf
    want = R.compare_stats(got, ref, 1e-5, 1e-5)
    s = run2.compare(torch.from_numpy(got).to(cuda), torch.from_numpy(ref).to(cuda), 1e-5, 1e-5)
    assert (s.count, s.nonfinite, s.mismatches, s.worst) == (want["count"], want["nonfinite"], want["mismatches"],
                                                             want["worst"])
    assert s.max_abs_err == want["max_abs_err"] and s.max_abs_ref == want["max_abs_ref"]
    # the device sums in a tree, the reference (and the oracle) sequentially: both are held to the exactly rounded sum
    fin = np.isfinite(got)
    e64, r64 = np.abs(got[fin].astype(np.float64) - ref[fin].astype(np.float64)), ref[fin].astype(np.float64)
    sse, ssr = math.fsum(e64 * e64), math.fsum(r64 * r64)
    assert abs(s.sum_sq_err - sse) <= 1e-12 * max(sse, 1e-300) and abs(want["sum_sq_err"] - sse) <= 1e-9 * max(sse, 1e-300)
    assert abs(s.sum_sq_ref - ssr) <= 1e-12 * ssr and abs(want["sum_sq_ref"] - ssr) <= 1e-9 * ssr
    assert s.ok == (want["mismatches"] == 0 and want["nonfinite"] == 0)


@pytest.mark.gpu
def test_compare_integers_and_empty(cuda):
    from lokinfer_b200 import run2
    a = torch.arange(1000, dtype=torch.int64, device=cuda)
    b = a.clone()
    b[400] += 3
    s = run2.compare(b, a, 0.0, 0.0)
    assert (s.mismatches, s.worst, s.max_abs_err) == (1, 400, 3.0)
    s = run2.compare(a.to(torch.int32), a.to(torch.int32))
    assert s.ok and s.count == 1000 and s.sum_sq_err == 0.0
    e = torch.empty(0, dtype=torch.float32, device=cuda)
    s = run2.compare(e, e)
    assert s.ok and s.count == 0 and s.worst == -1


@pytest.mark.gpu
def test_run2_tensor_core_conv_against_cuda_core_conv_on_the_device(cuda):
    """The reference's on-device sweeps (tests/python/test_device_sweeps.py): an optimized kernel and its oracle side
    by side in one call, inputs generated on the device, outputs compared on the device. Here: the tcgen05 fused conv
    against the CUDA-core kernel of the same contract."""
    from lokinfer_b200 import ops, run2
    c, l, k, d = 128, 5000, 11, 5
    store = run2.BlobStore(cuda)
    w = (np.random.default_rng(3).standard_normal((c, c, k)) / np.sqrt(c * k)).astype(np.float32)
    wb = store.put_tensor(w)
    assert store.put_tensor(w.copy()) == wb and store.uploads == 1  # same content, same handle, one upload
    state = ops.conv1d_prepare_f32_cuda(store.get(wb))
    affine = torch.stack([torch.zeros(c), torch.ones(c), torch.zeros(c)]).to(cuda)

    def both(x, wt, bias, alpha, res):
        kw = dict(residual=res, padding=d * (k - 1) // 2, dilation=d)
        fast, _ = ops.conv1d_snake_f32_cuda(x, wt, bias, affine, alpha, state=state, **kw)
        slow, _ = ops.conv1d_snake_f32_cuda(x, wt, bias, affine, alpha, **kw)
        return fast, slow

    inputs = [run2.Generated((c, l), seed=1), wb, run2.Generated((c,), seed=2, b=0.01),
              run2.Generated((c,), seed=3, dist="uniform", a=0.5, b=1.5), run2.Generated((c, l), seed=4)]
    outs, stats, times = run2.run2(both, inputs, compare=[(0, 1, 1e-5, 1e-5)], warmup=1, iters=2, store=store)
    assert len(outs) == 2 and len(times) == 2 and all(t > 0 for t in times)
    assert stats[0].ok and stats[0].count == c * l and stats[0].rel_rms <= 1e-5 and stats[0].snr_db > 100
    # the same call without returning tensors, against a stored reference, with one element disturbed
    wrong = outs[1].clone()
    wrong[0, 17] += 1
    rb = store.put_tensor(wrong)
    outs2, stats2, _ = run2.run2(both, inputs, compare=[(0, rb, 0.0, 1e-3)], return_outputs=False, store=store)
    assert outs2 == [] and stats2[0].mismatches == 1 and stats2[0].worst == 17 and abs(stats2[0].max_abs_err - 1) < 1e-4
    assert ops.conv_tc_status() == 0
