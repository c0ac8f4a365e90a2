"""The C-ABI boundary without a GPU: the library loads, exports every symbol include/lkc.h declares, its registry
matches the Python `ops` surface (the reference's registry rule, tests/python/test_registry.py), shape rules raise
OpError like the reference's type rules, and a compute call without a CUDA device fails loudly (no CPU path)."""
import ctypes
import inspect
import re
from pathlib import Path

import pytest
import torch

from lokinfer_b200 import _lib, ops

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "lkc.h").read_text()
    return sorted(set(re.findall(r"LKC_API[^;]*?\b(lkc_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    syms = declared_symbols()
    assert len(syms) >= 25
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/lkc.h but not exported by liblkc.so"


def test_registry_matches_ops_surface():
    names = _lib.registered_kernels()
    assert names == sorted(names) and len(set(names)) == len(names)
    for n in names:
        assert n.endswith("_f32_cuda") and _lib.find_kernel(n) is not None
        assert hasattr(_lib.lib(), "lkc_" + n)
    assert _lib.find_kernel("conv1d_snake_f32_cpu") is None
    src = inspect.getsource(ops)
    used = set(re.findall(r'(?:_run|_lib\.run)\(\s*"(\w+)"', src))
    assert used == set(names), (used ^ set(names))


def test_shape_rules_raise_op_error():
    z = torch.zeros
    with pytest.raises(ops.OpError, match="w must be"):
        ops.conv1d_snake_f32_cuda(z(8, 50), z(8, 7, 3), z(8), z(3, 8), z(8))
    with pytest.raises(ops.OpError, match="affine must be"):
        ops.conv1d_snake_f32_cuda(z(8, 50), z(8, 8, 3), z(8), z(2, 8), z(8))
    with pytest.raises(ops.OpError, match="empty conv output"):
        ops.conv1d_affine_f32_cuda(z(8, 2), z(8, 8, 7), z(8), z(3, 8))
    with pytest.raises(ops.OpError, match="out_scale needs a residual"):
        ops.conv1d_leaky_f32_cuda(z(8, 50), z(8, 8, 3), z(8), z(3, 8), out_scale=0.5, padding=1)
    with pytest.raises(ops.OpError, match="tile must be"):
        ops.conv1d_affine_f32_cuda(z(8, 50), z(8, 8, 3), z(8), z(3, 8), padding=1, tile=100)
    with pytest.raises(ops.OpError, match="2p"):
        ops.conv_transpose1d_poly_f32_cuda(z(8, 5), z(8, 2, 2, 4), z(4), z(4, 10), stride=2, padding=0, taps=2,
                                           slope=0.1)
    with pytest.raises(ops.OpError, match="stats chunks"):
        ops.adain_affine_f32_cuda(z(4, 3, 2), z(8), length=1000)
    with pytest.raises(ops.OpError, match="n_fft"):
        ops.istft_logits_f32_cuda(z(22, 8), n_fft=21)
    with pytest.raises(ops.OpError, match="need at least 2 frames"):
        ops.istft_logits_f32_cuda(z(22, 1))
    with pytest.raises(ops.OpError, match="reflect padding"):
        ops.pad_reflect1d_f32_cuda(z(2, 1), 1, 0)
    with pytest.raises(ops.OpError, match="noise must be"):
        ops.harmonic_source_f32_cuda(z(4), z(1200, 8), z(9), z(1))
    with pytest.raises(ops.OpError, match="w must be"):
        ops.harmonic_source_f32_cuda(z(4), z(1200, 9), z(8), z(1))
    with pytest.raises(ops.OpError, match="longer than n_fft/2"):
        ops.stft_magphase_f32_cuda(z(10))
    with pytest.raises(ops.OpError, match="n_fft"):
        ops.stft_magphase_f32_cuda(z(100), n_fft=128)
    with pytest.raises(ops.OpError, match="must be an int"):
        ops.conv1d_f32_cuda(z(2, 8), z(2, 2, 3), z(2), stride=1.0)


def test_no_cpu_path():
    with pytest.raises(ops.OpError, match="no CPU path"):
        ops.channel_stats_f32_cuda(torch.zeros(4, 300))


def test_entry_point_rejects_bad_packing_without_touching_the_gpu():
    """Argument validation happens on the host before any launch: a wrong operand count returns non-zero and
    lkc_last_error() names the kernel."""
    fn = _lib.find_kernel("istft_logits_f32_cuda")
    ints = (ctypes.c_int64 * 5)(22, 1, 0, 5, 20)
    ptrs = (ctypes.c_void_p * 2)(None, None)
    args = _lib.LkcArgs(ptrs, ints, None, None, 2, 5)
    assert fn(ctypes.byref(args), None) != 0
    assert "istft_logits_f32_cuda" in _lib.last_error()
    args = _lib.LkcArgs(ptrs, ints, None, None, 1, 5)
    assert fn(ctypes.byref(args), None) != 0
