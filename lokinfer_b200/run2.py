"""Device-side test harness: the data path of the reference's RUN2 message (include/lokinfer/remote/server.h:30-47,
python/lokinfer/remote.py `RemoteDevice.run2`) without its wire protocol. Inputs are generated on the GPU from a seed
(`Generated`) or kept on the GPU under their content hash (`BlobStore.put_tensor` -> `Blob`), the callable under test
runs `warmup + iters` times, and outputs are compared on the GPU against a blob or against another output, so that
only a few numbers per comparison come back to the host:

    store = BlobStore(device)
    outs, stats, times = run2(fn, [Generated((128, 5000), seed=1), store.put_tensor(w)],
                              compare=[(0, 1, 1e-5, 1e-5)], iters=3, store=store)
    assert stats[0].ok

`generate` / `compare` are the two kernels on their own (csrc/harness.cu). Networking, model upload and the `.lkm`
container of the reference are not part of this repository.
"""
from __future__ import annotations

import ctypes
import hashlib
import time
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib, ops

_DTYPES = {torch.float32: 0, torch.int32: 1, torch.int64: 2}
_DISTS = {"normal": 0, "uniform": 1, "int": 2}
_WORKSPACE_BYTES = 32768  # LKC_COMPARE_WORKSPACE_BYTES


def _call(fn, ptrs, ints, floats):
    p = (ctypes.c_void_p * len(ptrs))(*ptrs)
    i = (ctypes.c_int64 * len(ints))(*ints)
    f = (ctypes.c_double * len(floats))(*floats)
    a = _lib.LkcArgs(p, i, f, None, len(ptrs), len(ints))
    fn.argtypes = [ctypes.POINTER(_lib.LkcArgs), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    if fn(ctypes.byref(a), ctypes.c_void_p(ops._stream())) != 0:
        raise _lib.LkcError(_lib.last_error())


def generate(shape, seed: int, dtype=torch.float32, dist: str = "normal", a: float = 0.0, b: float = 1.0,
             device=None) -> torch.Tensor:
    """A tensor filled on the device by the reference's RUN2 generator (splitmix64 + Box-Muller in double,
    src/remote/server.cpp:739-782): "normal" = normal(mean a, std b), "uniform" = [a, b), "int" = integers in
    [floor a, floor b). dtype float32, int32 or int64."""
    ops.check(dtype in _DTYPES, "generated tensors are float32, int32 or int64")
    ops.check(dist in _DISTS, "dist must be 'normal', 'uniform' or 'int'")
    ops.check(np.isfinite(a) and np.isfinite(b), "a and b must be finite")
    ops.check(dist != "int" or (b > a and b - a < 9.0e15), "bad integer range")
    device = torch.device(device if device is not None else "cuda")
    ops.check(device.type == "cuda", "generate runs on a cuda device (there is no CPU path)")
    out = torch.empty(tuple(int(d) for d in shape), dtype=dtype, device=device)
    seed_slot = ctypes.c_uint64(int(seed) & (2 ** 64 - 1))
    with torch.cuda.device(device):
        _call(_lib.lib().lkc_generate_cuda, [ctypes.addressof(seed_slot), out.data_ptr()],
              [out.numel(), _DTYPES[dtype], _DISTS[dist]], [float(a), float(b)])
    return out


@dataclass
class Stats:
    """On-device comparison of one output (the reference's `Stats`, python/lokinfer/remote.py:122-143)."""
    output: int
    count: int
    nonfinite: int
    mismatches: int
    worst: int
    max_abs_err: float
    max_abs_ref: float
    sum_sq_err: float
    sum_sq_ref: float

    @property
    def ok(self) -> bool:
        return self.mismatches == 0 and self.nonfinite == 0

    @property
    def rel_rms(self) -> float:
        return float(np.sqrt(self.sum_sq_err / self.sum_sq_ref)) if self.sum_sq_ref > 0 else float(np.sqrt(self.sum_sq_err))

    @property
    def snr_db(self) -> float:
        return float(10 * np.log10(self.sum_sq_ref / self.sum_sq_err)) if self.sum_sq_err > 0 else float("inf")


def compare_async(got: torch.Tensor, ref: torch.Tensor, rtol: float, atol: float):
    """Queues the comparison on the current stream; returns the 64-byte device record (see Stats / include/lkc.h)."""
    ops.check(got.is_cuda and ref.is_cuda and got.device == ref.device, "compare: both tensors on one cuda device")
    ops.check(got.dtype == ref.dtype and got.numel() == ref.numel(), "compare: shape or dtype differs")
    ops.check(got.dtype in _DTYPES, "compare: float32, int32 or int64 tensors")
    ops.check(rtol >= 0 and atol >= 0, "compare: bad tolerance")
    got, ref = got.contiguous(), ref.contiguous()
    rec = torch.empty(8, dtype=torch.int64, device=got.device)
    ws = torch.empty(_WORKSPACE_BYTES, dtype=torch.uint8, device=got.device)
    with torch.cuda.device(got.device):
        _call(_lib.lib().lkc_compare_stats_cuda, [got.data_ptr(), ref.data_ptr(), rec.data_ptr(), ws.data_ptr()],
              [got.numel(), _DTYPES[got.dtype]], [float(rtol), float(atol)])
    rec._keep = (got, ref, ws)  # the kernels read them after this function returns
    return rec


def stats_from_record(rec: torch.Tensor, output: int = 0) -> Stats:
    host = rec.cpu()  # synchronises with the stream that produced it
    ints = host[:4].tolist()
    dbl = host[4:].view(torch.float64).tolist()
    return Stats(output, ints[0], ints[1], ints[2], ints[3], dbl[0], dbl[1], dbl[2], dbl[3])


def compare(got: torch.Tensor, ref: torch.Tensor, rtol: float = 0.0, atol: float = 0.0) -> Stats:
    """mismatches = #(|got - ref| > atol + rtol |ref|), worst index, max errors and sums of squares, computed on the
    device (src/remote/server.cpp:686-736)."""
    return stats_from_record(compare_async(got, ref, rtol, atol))


@dataclass(frozen=True)
class Generated:
    """An input generated on the device (RUN2 input kind 2)."""
    shape: tuple
    seed: int
    dtype: torch.dtype = torch.float32
    dist: str = "normal"
    a: float = 0.0
    b: float = 1.0


@dataclass(frozen=True)
class Blob:
    """A tensor kept on the device under the sha256 of its bytes, dtype and shape (RUN2 input / reference kind 1)."""
    sha: str


class BlobStore:
    """Content-addressed device tensors: the same content is stored (and would be sent) once."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._blobs: dict[str, torch.Tensor] = {}
        self.uploads = 0

    def put_tensor(self, x) -> Blob:
        a = np.ascontiguousarray(x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else x)
        h = hashlib.sha256(str((a.dtype.str, a.shape)).encode() + a.tobytes()).hexdigest()
        if h not in self._blobs:
            self._blobs[h] = torch.from_numpy(a).to(self.device)
            self.uploads += 1
        return Blob(h)

    def get(self, blob: Blob) -> torch.Tensor:
        ops.check(blob.sha in self._blobs, f"unknown blob {blob.sha[:12]}")
        return self._blobs[blob.sha]


def run2(fn, inputs, compare=(), warmup: int = 0, iters: int = 1, return_outputs: bool = True, store: BlobStore = None,
         device=None):
    """Runs fn(*device_inputs) `warmup` + `iters` times (RemoteDevice.run2, python/lokinfer/remote.py). inputs: a
    Generated, a Blob of `store`, a torch tensor or a numpy array each. compare: (output index, Blob or other output
    index, rtol, atol) each. Returns (outputs or [], [Stats], [wall ns of every timed iteration]); an iteration is
    timed on the host around a stream synchronise, as the reference times a call."""
    device = torch.device(device if device is not None else (store.device if store is not None else "cuda"))
    args = []
    for x in inputs:
        if isinstance(x, Generated):
            args.append(generate(x.shape, x.seed, x.dtype, x.dist, x.a, x.b, device))
        elif isinstance(x, Blob):
            ops.check(store is not None, "a Blob input needs the store it was put into")
            args.append(store.get(x))
        elif isinstance(x, torch.Tensor):
            args.append(x.to(device))
        else:
            args.append(torch.from_numpy(np.ascontiguousarray(x)).to(device))
    outs = None
    times = []
    for it in range(warmup + iters):
        torch.cuda.synchronize(device)
        t0 = time.perf_counter_ns()
        outs = fn(*args)
        torch.cuda.synchronize(device)
        if it >= warmup:
            times.append(time.perf_counter_ns() - t0)
    outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
    records = []
    for out_idx, ref, rtol, atol in compare:
        ops.check(0 <= out_idx < len(outs), f"comparison: no output {out_idx}")
        if isinstance(ref, Blob):
            ops.check(store is not None, "a Blob reference needs the store it was put into")
            r = store.get(ref)
        else:
            ops.check(0 <= int(ref) < len(outs), f"comparison: no output {ref}")
            r = outs[int(ref)]
        records.append((out_idx, compare_async(outs[out_idx], r, rtol, atol)))
    stats = [stats_from_record(rec, i) for i, rec in records]
    return (outs if return_outputs else []), stats, times
