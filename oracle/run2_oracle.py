"""CPU oracle for the data path of the reference's RUN2 message. TEST INFRASTRUCTURE ONLY.

Only tests/ may import this module; the product package never does. Two numpy restatements:

generate       the device-side input generator (src/remote/server.cpp:739-782, mirrored by
               python/lokinfer/remote.py:96-119): element i draws from the splitmix64 stream at positions 2 i + 1 and
               2 i + 2 of a stream started at `seed` (state += golden ratio constant, then the published splitmix64
               finaliser), top 53 bits as a double in [0, 1).
compare_stats  the on-device comparison (src/remote/server.cpp:686-736).

Pinning: the reference stores no vectors for its generator (tests/python/test_remote.py:150-159 checks ranges and
moments only). The integer stream is pinned here against the published splitmix64 test vector (seed 0 ->
0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F), the value ranges against the reference's own test.
"""
from __future__ import annotations

import numpy as np

GOLDEN = 0x9E3779B97F4A7C15
MASK = (1 << 64) - 1


def splitmix_at(seed: int, pos: np.ndarray) -> np.ndarray:
    """Output number `pos` (1-based) of the splitmix64 stream whose state starts at `seed`: uint64 array."""
    pos = np.asarray(pos, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = np.uint64(seed & MASK) + pos * np.uint64(GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _unit(bits: np.ndarray) -> np.ndarray:
    return (bits >> np.uint64(11)).astype(np.float64) * 2.0 ** -53


def generate(shape, seed: int, dtype=np.float32, dist: str = "normal", a: float = 0.0, b: float = 1.0) -> np.ndarray:
    """dist "normal": a + b sqrt(-2 log(1 - u1)) cos(2 pi u2); "uniform": a + (b - a) u1 in [a, b); "int": floor(a) +
    floor(u1 (floor(b) - floor(a))). Computed in double, converted to dtype at the end (src/remote/server.cpp:768-781)."""
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    i = np.arange(n, dtype=np.uint64)
    u1 = _unit(splitmix_at(seed, np.uint64(2) * i + np.uint64(1)))
    if dist == "normal":
        u2 = _unit(splitmix_at(seed, np.uint64(2) * i + np.uint64(2)))
        x = a + b * np.sqrt(-2.0 * np.log(1.0 - u1)) * np.cos(6.283185307179586 * u2)
    elif dist == "uniform":
        x = a + (b - a) * u1
    elif dist == "int":
        x = np.floor(a) + np.floor(u1 * (np.floor(b) - np.floor(a)))
    else:
        raise ValueError(dist)
    return x.astype(dtype).reshape(shape)


def compare_stats(got: np.ndarray, ref: np.ndarray, rtol: float, atol: float) -> dict:
    """count, nonfinite, mismatches, worst, max_abs_err, max_abs_ref, sum_sq_err, sum_sq_ref, with the reference's
    rules: a non-finite `got` is counted as nonfinite (and as a mismatch unless both are NaN or equal), and is left out
    of every other figure; worst = index of the largest excess e - (atol + rtol |ref|), the first one on a tie, -1 when
    no element took part. The two sums run sequentially over the elements, as in the reference."""
    g = np.asarray(got, dtype=np.float64).ravel()
    r = np.asarray(ref, dtype=np.float64).ravel()
    assert g.shape == r.shape
    fin = np.isfinite(g)
    bad = ~fin
    nonfinite = int(bad.sum())
    with np.errstate(invalid="ignore"):
        mism = int((bad & ~(np.isnan(g) & np.isnan(r)) & (g != r)).sum())
        e = np.abs(g[fin] - r[fin])
        ar = np.abs(r[fin])
        excess = e - (atol + rtol * ar)
        mism += int((excess > 0).sum())
    idx = np.nonzero(fin)[0]
    worst = -1
    if e.size:
        ex = np.where(np.isnan(excess), -np.inf, excess)
        if np.isfinite(ex).any() or (ex == np.inf).any():
            worst = int(idx[int(np.argmax(ex))])  # argmax returns the first maximum
    sse = ssr = 0.0
    for v in e:
        sse += float(v) * float(v)
    for v in r[fin]:
        ssr += float(v) * float(v)
    return {"count": int(g.size), "nonfinite": nonfinite, "mismatches": mism, "worst": worst,
            "max_abs_err": float(np.fmax.reduce(e, initial=0.0)) if e.size else 0.0,
            "max_abs_ref": float(np.fmax.reduce(ar, initial=0.0)) if e.size else 0.0,
            "sum_sq_err": sse, "sum_sq_ref": ssr}
