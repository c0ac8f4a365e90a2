"""ctypes binding of liblkc.so (the C-ABI CUDA library). There is no CPU fallback: if the library is missing
or a call fails, the caller gets an exception."""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "liblkc.so"


class LkcArgs(ctypes.Structure):
    """struct LkcArgs of include/lkc.h (the reference's KernelArgs packing, include/lokinfer/runtime/kernel.h:31-39)."""
    _fields_ = [
        ("ptrs", ctypes.POINTER(ctypes.c_void_p)),
        ("ints", ctypes.POINTER(ctypes.c_int64)),
        ("floats", ctypes.POINTER(ctypes.c_double)),
        ("state", ctypes.c_void_p),
        ("numPtrs", ctypes.c_uint32),
        ("numInts", ctypes.c_uint32),
    ]


RUN_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(LkcArgs), ctypes.c_void_p)

_lib = None
_kernels: dict = {}


class LkcError(RuntimeError):
    """A kernel entry point returned non-zero; the message is lkc_last_error()."""


def lib():
    """The loaded library (loads it on first use). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m lokinfer_b200.build` "
                "(there is no CPU fallback for the CUDA kernels)")
        l = ctypes.CDLL(str(LIB_PATH))
        l.lkc_kernel_count.restype = ctypes.c_int
        l.lkc_kernel_name.restype = ctypes.c_char_p
        l.lkc_kernel_name.argtypes = [ctypes.c_int]
        l.lkc_find_kernel.restype = ctypes.c_void_p
        l.lkc_find_kernel.argtypes = [ctypes.c_char_p]
        l.lkc_last_error.restype = ctypes.c_char_p
        l.lkc_build_info.restype = ctypes.c_char_p
        l.lkc_conv1d_tc_pack_floats.restype = ctypes.c_int64
        l.lkc_conv1d_tc_pack_floats.argtypes = [ctypes.c_int64] * 3
        l.lkc_conv1d_state_create.restype = ctypes.c_void_p
        l.lkc_conv1d_state_create.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
        l.lkc_convt_tc_pack_floats.restype = ctypes.c_int64
        l.lkc_convt_tc_pack_floats.argtypes = [ctypes.c_int64] * 5
        l.lkc_convt_state_create.restype = ctypes.c_void_p
        l.lkc_convt_state_create.argtypes = [ctypes.c_void_p] + [ctypes.c_int64] * 5
        l.lkc_conv1d_state_destroy.restype = None
        l.lkc_conv1d_state_destroy.argtypes = [ctypes.c_void_p]
        l.lkc_conv1d_tc_status.restype = ctypes.c_int
        l.lkc_conv1d_tc_status.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int]
        l.lkc_conv1d_tc_status_async.restype = ctypes.c_int
        l.lkc_conv1d_tc_status_async.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        l.lkc_conv1d_tc_profile.restype = ctypes.c_int
        l.lkc_conv1d_tc_profile.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int64)]
        l.lkc_set_conv_io.restype = ctypes.c_int
        l.lkc_set_conv_io.argtypes = [ctypes.c_int]
        l.lkc_set_conv_path.restype = ctypes.c_int
        l.lkc_set_conv_path.argtypes = [ctypes.c_int]
        _lib = l
    return _lib


def registered_kernels() -> list[str]:
    """Names of every kernel in the library's registry (sorted), like registeredKernels() in the reference."""
    l = lib()
    return [l.lkc_kernel_name(i).decode() for i in range(l.lkc_kernel_count())]


def find_kernel(name: str):
    """The run function registered under `name` (looked up through lkc_find_kernel), or None."""
    fn = _kernels.get(name)
    if fn is None:
        addr = lib().lkc_find_kernel(name.encode())
        if not addr:
            return None
        fn = RUN_FN(addr)
        _kernels[name] = fn
    return fn


def last_error() -> str:
    return lib().lkc_last_error().decode(errors="replace")


def run(name: str, ptrs, ints, floats=(), state: int | None = None, stream: int = 0) -> None:
    """Calls kernel `name` with the reference's argument packing: ptrs = operand then out device addresses,
    ints = shape dims then integer attrs in name order, floats = float attrs in name order."""
    fn = find_kernel(name)
    if fn is None:
        raise LkcError(f"kernel {name} is not registered in liblkc")
    n_p, n_i, n_f = len(ptrs), len(ints), len(floats)
    p_arr = (ctypes.c_void_p * max(n_p, 1))(*ptrs)
    i_arr = (ctypes.c_int64 * max(n_i, 1))(*ints)
    f_arr = (ctypes.c_double * max(n_f, 1))(*floats)
    args = LkcArgs(p_arr, i_arr, f_arr, state, n_p, n_i)
    rc = fn(ctypes.byref(args), ctypes.c_void_p(stream))
    if rc != 0:
        raise LkcError(f"{name}: {last_error()}")
