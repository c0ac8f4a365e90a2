"""lkc_harmonic_source_noalloc_f32_cuda: the harmonic source with its phase table in a fixed device array of the
library (no allocation on any path). It has to give exactly what lkc_harmonic_source_f32_cuda gives, call after call,
whether this file runs alone or after every other GPU test of the suite (it is collected last)."""
import ctypes

import numpy as np
import pytest
import torch

from lokinfer_b200 import synth

pytestmark = pytest.mark.gpu


def _call(fn, tensors, ints, stream):
    from lokinfer_b200 import _lib
    ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    iarr = (ctypes.c_int64 * len(ints))(*ints)
    farr = (ctypes.c_double * 1)()
    args = _lib.LkcArgs(ptrs, iarr, farr, None, len(tensors), len(ints))
    return fn(ctypes.byref(args), ctypes.c_void_p(stream))


@pytest.mark.parametrize("n", [1, 7, 238, 2080, 4096])
def test_noalloc_matches_the_allocating_entry_point(cuda, n):
    from lokinfer_b200 import _lib, ops
    lib = _lib.lib()
    fn = lib.lkc_harmonic_source_noalloc_f32_cuda
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_lib.LkcArgs), ctypes.c_void_p]
    f0, noise, w, b = synth.source_case(n, n + 3)
    d = [ops.to_cuda(v, cuda) for v in (f0, noise, w, b)]
    ref = ops.harmonic_source_f32_cuda(*d)
    ints = [n, 300 * n, 9, 9, 1, 300 * n]
    stream = torch.cuda.current_stream(cuda).cuda_stream
    outs = []
    for _ in range(2):  # two calls in a row reuse the fixed table
        out = torch.full((300 * n,), float("nan"), device=cuda)
        assert _call(fn, d + [out], ints, stream) == 0, _lib.last_error()
        outs.append(out)
    torch.cuda.synchronize(cuda)
    assert torch.equal(outs[0], ref) and torch.equal(outs[1], ref)
    # a different, shorter input right after: nothing of the previous call's table may leak into it
    f0s, noises, ws, bs = synth.source_case(3, 17)
    ds = [ops.to_cuda(v, cuda) for v in (f0s, noises, ws, bs)]
    out = torch.empty(900, device=cuda)
    assert _call(fn, ds + [out], [3, 900, 9, 9, 1, 900], stream) == 0, _lib.last_error()
    assert torch.equal(out, ops.harmonic_source_f32_cuda(*ds))


def test_noalloc_rejects_inputs_beyond_its_table(cuda):
    from lokinfer_b200 import _lib, ops
    lib = _lib.lib()
    fn = lib.lkc_harmonic_source_noalloc_f32_cuda
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(_lib.LkcArgs), ctypes.c_void_p]
    n = 4097
    d = [torch.zeros(n, device=cuda), torch.zeros(300 * n, 9, device=cuda), torch.zeros(9, device=cuda),
         torch.zeros(1, device=cuda)]
    out = torch.full((300 * n,), 7.0, device=cuda)
    rc = _call(fn, d + [out], [n, 300 * n, 9, 9, 1, 300 * n], torch.cuda.current_stream(cuda).cuda_stream)
    assert rc != 0 and "4096" in _lib.last_error()
    torch.cuda.synchronize(cuda)
    assert bool((out == 7.0).all())  # nothing was launched
    assert ops.conv_tc_status() == 0
