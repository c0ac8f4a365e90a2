"""`ops.*` surface of the Kokoro generator path on the `cuda` device.

Each function mirrors one op of the reference's Python front end (python/lokinfer/ops/kokoro.py; elementwise ops
python/lokinfer/ops/elementwise.py) with the same positional operands, keyword attributes, defaults, shape rules
and error messages, under the name `<op>_f32_cuda` instead of `<op>_f32_cpu`. Operands are contiguous float32
torch tensors on a CUDA device; results are new tensors (the wrapper plays the runtime's role of allocating the
outs, src/runtime/executable.cpp:583-654) and every launch goes to torch's current stream through the C-ABI in
include/lkc.h. Shape errors raise OpError before anything is launched (python/lokinfer/ops/_def.py:12-19).

Padded rows (no counterpart in the reference, whose tensors are always contiguous): inside `with padded_rows():`
every [C, L] result is allocated with its row pitch rounded up to 4 floats and returned as the [:, :L] view, and the
ops that take a row pitch (the conv family, channel_stats, conv_transpose1d_poly, istft_logits, add3_scale) accept
such views as operands. Rows then start on 16-byte boundaries, which lets the tensor-core kernels move them with
the TMA unit; values never depend on the pitch. Outs come from `allocator` (default: torch.empty), the hook a
planned arena plugs into.
"""
from __future__ import annotations

import contextlib

import torch

from . import _lib

STAT_CHUNK = 128  # python/lokinfer/ops/kokoro.py:470


class OpError(ValueError):
    pass


def check(cond: bool, msg: str = "invalid operands") -> None:
    if not cond:
        raise OpError(msg)


def _float(v, name):
    check(isinstance(v, (int, float)) and not isinstance(v, bool), f"{name} must be a number")
    return float(v)


def _int(v, name):
    check(isinstance(v, int) and not isinstance(v, bool), f"{name} must be an int")
    return int(v)


def _row_pitched(x) -> bool:
    """[C, L] view of a [C, pitch] buffer: unit stride along time, rows at least L apart."""
    return x.dim() == 2 and x.stride(1) == 1 and x.stride(0) >= x.shape[1]


def _f32(*xs, rank=None):
    for x in xs:
        check(isinstance(x, torch.Tensor) and x.dtype == torch.float32, "expected f32 tensor operands")
        check(x.is_contiguous() or _row_pitched(x), "expected contiguous tensors (or [C, L] views with padded rows)")
        if rank is not None:
            check(x.dim() == rank, f"expected rank-{rank} operands, got {tuple(x.shape)}")


def ceildiv(a, b):
    return -(-a // b)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class Profile:
    """Per-kernel recorder (the reference's Executable::setProfile / LOKINFER_PROFILE, runtime.h:69-74): while one is
    active every kernel launch is bracketed by a CUDA event pair on the launching stream and counted. Zero cost
    when off. rows() -> [(kernel name, ints, milliseconds)] after a synchronize."""

    def __init__(self, time_kernels=True, repeat=1, graph=False):
        """repeat > 1 launches every kernel `repeat` times back to back inside its event pair and reports the
        average: the ops are pure (outs never alias operands), and the host's enqueue latency between the start
        event and the first launch stops inflating the figure for short kernels. graph=True goes one step further:
        the repeats are captured into a small CUDA graph (on a side stream, right after the kernel's real launch) and
        that graph is replayed inside the event pair, so the host's launch path (ctypes, tensor-map encoding) is out
        of the timed region altogether, as it is when the forward itself runs as a captured graph."""
        self.time_kernels = time_kernels
        self.repeat = max(1, int(repeat))
        self.graph = bool(graph)
        self._graphs = []  # kept alive until rows() has read the events
        self._side = None
        self.calls = []  # (name, ints, start event, end event)
        self.count = 0

    def __enter__(self):
        global _profile
        self._prev, _profile = _profile, self
        return self

    def __exit__(self, *exc):
        global _profile
        _profile = self._prev

    def rows(self):
        torch.cuda.synchronize()
        out = [(n, i, a.elapsed_time(b) / self.repeat) for n, i, a, b in self.calls]
        self._graphs.clear()
        return out


_profile = None


# Kernels that take row pitches: positions (in operands + outs order) of their [C, L] activation tensors. The
# pitches are appended to the ints only when one of them differs from the row length.
_PITCHED = {
    "conv1d_f32_cuda": (0, 3), "conv1d_nobias_f32_cuda": (0, 2), "channel_stats_f32_cuda": (0,),
    "conv1d_snake_f32_cuda": (0, 5), "conv1d_snake_res_f32_cuda": (0, 5, 6),
    "conv1d_leaky_f32_cuda": (0, 4), "conv1d_leaky_res_f32_cuda": (0, 4, 5), "conv1d_affine_f32_cuda": (0, 4),
    "conv_transpose1d_poly_f32_cuda": (0, 3, 4), "istft_logits_f32_cuda": (0,),
    "space_to_depth_f32_cuda": (0, 1),
}


def _run(name, operands, outs, attrs_int=(), attrs_float=(), state=None, window=None):
    """window: the ints of the window extension of include/lkc.h (time-sharded tensors, see timeshard.py); the row
    pitches are then always passed and the caller vouches for the layout of every operand."""
    ts = list(operands) + list(outs)
    check(all(t.is_cuda and t.device == ts[0].device for t in ts),
          f"{name}: operands must live on one cuda device (use to_cuda); there is no CPU path")
    ints = [d for t in ts for d in t.shape] + list(attrs_int)
    pitched = _PITCHED.get(name, ())
    if window is None:
        for i, t in enumerate(ts):
            check(t.is_contiguous() or i in pitched, f"{name}: operand {i} must be contiguous")
    if window is not None or any(not ts[i].is_contiguous() for i in pitched):
        ints += [int(ts[i].stride(0)) for i in pitched]
    if window is not None:
        ints += [int(v) for v in window]
    if _tracer is not None:
        _tracer.on_run(ts, _stream())
    with torch.cuda.device(ts[0].device):
        prof = _profile
        if prof is None:
            _lib.run(name, [t.data_ptr() for t in ts], ints, attrs_float, state, _stream())
            return
        prof.count += 1
        if not prof.time_kernels:
            _lib.run(name, [t.data_ptr() for t in ts], ints, attrs_float, state, _stream())
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ptrs = [t.data_ptr() for t in ts]
        _lib.run(name, ptrs, ints, attrs_float, state, _stream())  # untimed first launch: absorbs the enqueue gap
        if prof.graph:
            if prof._side is None:
                prof._side = torch.cuda.Stream(device=ts[0].device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(prof._side):
                with torch.cuda.graph(g, stream=prof._side):
                    for _ in range(prof.repeat):
                        _lib.run(name, ptrs, ints, attrs_float, state, _stream())
            g.replay()  # untimed: first replay of a graph pays its upload
            a.record()
            g.replay()
            b.record()
            prof._graphs.append(g)
        else:
            a.record()
            for _ in range(prof.repeat):
                _lib.run(name, ptrs, ints, attrs_float, state, _stream())
            b.record()
        prof.calls.append((name, ints, a, b))


ROW_ALIGN = 4  # floats: 16-byte rows


def _torch_alloc(shape, device):
    return torch.empty(shape, dtype=torch.float32, device=device)


allocator = _torch_alloc  # (shape, device) -> contiguous f32 tensor; replaced by a planned arena (see arena.py)
_pad_rows = False
_tracer = None  # arena.Tracer while a forward is being traced for the memory plan


def _alloc(shape, device):
    t = allocator(tuple(int(d) for d in shape), device)
    if _tracer is not None:
        _tracer.on_alloc(t, _stream())
    return t


@contextlib.contextmanager
def tracing(tracer):
    """Records every result allocation, kernel call and stream join inside the block into `tracer`."""
    global _tracer
    prev, _tracer = _tracer, tracer
    try:
        yield tracer
    finally:
        _tracer = prev


def join(waiter, waited):
    """waiter.wait_stream(waited), visible to the tracer (the memory plan needs the fork / join structure)."""
    waiter.wait_stream(waited)
    if _tracer is not None:
        _tracer.on_join(waiter.cuda_stream, waited.cuda_stream)


@contextlib.contextmanager
def padded_rows(enable=True):
    """Inside the block [C, L] results get a row pitch rounded up to ROW_ALIGN floats (see the module docstring)."""
    global _pad_rows
    prev, _pad_rows = _pad_rows, bool(enable)
    try:
        yield
    finally:
        _pad_rows = prev


@contextlib.contextmanager
def use_allocator(fn):
    """Routes the allocation of every result inside the block through fn(shape, device)."""
    global allocator
    prev, allocator = allocator, fn
    try:
        yield
    finally:
        allocator = prev


def empty_rows(c, l, device):
    """f32[c, l] with padded rows when padded_rows() is active (else contiguous)."""
    if _pad_rows:
        pitch = ceildiv(int(l), ROW_ALIGN) * ROW_ALIGN
        return _alloc((int(c), pitch), device)[:, :int(l)]
    return _alloc((int(c), int(l)), device)


def _new(like, shape, rows=False):
    """Storage of one result. rows=True marks a [C, L] activation of an op that takes row pitches: it gets padded
    rows inside padded_rows()."""
    # Shape rules run on any device (so they can be exercised without a GPU); storage is only made on cuda.
    if not like.is_cuda:
        return torch.empty(tuple(shape), dtype=torch.float32, device="meta")
    if rows:
        return empty_rows(shape[0], shape[1], like.device)
    return _alloc(shape, like.device)


def _full_rows(x):
    """The [C, pitch] buffer behind a [C, L] view with padded rows (the view must start at its first element)."""
    c, pitch = int(x.shape[0]), int(x.stride(0))
    check(x.untyped_storage().nbytes() >= (x.storage_offset() + c * pitch) * 4, "padded view without its full rows")
    return torch.as_strided(x, (c, pitch), (pitch, 1))


def to_cuda(a, device="cuda", rows=False):
    """Host array / tensor -> contiguous f32 tensor on the cuda device (the `sync cpu_to_cuda` copy). rows=True: a
    [C, L] array goes into a buffer with padded rows when padded_rows() is active."""
    t = torch.as_tensor(a, dtype=torch.float32)
    if rows and t.dim() == 2 and _pad_rows:
        out = empty_rows(t.shape[0], t.shape[1], torch.device(device))
        out.copy_(t)
        return out
    return t.to(device).contiguous()


def to_cpu(t):
    return t.detach().cpu()


# --- elementwise ---------------------------------------------------------------------------------------------

def leaky_relu_f32_cuda(x, slope):
    """F.leaky_relu(x, slope), any shape."""
    _f32(x)
    out = _new(x, x.shape)
    _run("leaky_relu_f32_cuda", [x], [out], attrs_float=[_float(slope, "slope")])
    return out


def scale_f32_cuda(x, scale):
    """x * scale, any shape."""
    _f32(x)
    out = _new(x, x.shape)
    _run("scale_f32_cuda", [x], [out], attrs_float=[_float(scale, "scale")])
    return out


def add_f32_cuda(a, b):
    """a + b, same shapes."""
    _f32(a, b)
    check(a.shape == b.shape, f"shape mismatch: {tuple(a.shape)}, {tuple(b.shape)}")
    out = _new(a, a.shape)
    _run("add_f32_cuda", [a, b], [out])
    return out


def add3_scale_f32_cuda(a, b, c, scale):
    """(a + b + c) * scale, any shape. [C, L] views with padded rows of one pitch are processed with their padding
    (the op is elementwise, so the padding columns only cost their bandwidth)."""
    _f32(a, b, c)
    check(a.shape == b.shape and a.shape == c.shape,
          f"shape mismatch: {tuple(a.shape)}, {tuple(b.shape)}, {tuple(c.shape)}")
    if a.is_cuda and not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
        check(a.stride() == b.stride() == c.stride(), "padded operands must share one row pitch")
        fa, fb, fc = _full_rows(a), _full_rows(b), _full_rows(c)
        out = _alloc(tuple(fa.shape), a.device)
        _run("add3_scale_f32_cuda", [fa, fb, fc], [out], attrs_float=[_float(scale, "scale")])
        return out[:, :a.shape[1]]
    out = _new(a, a.shape)
    _run("add3_scale_f32_cuda", [a, b, c], [out], attrs_float=[_float(scale, "scale")])
    return out


def gemm_bias_f32_cuda(x, wt, b):
    """x @ wt + b: x f32[M, K], wt f32[K, N], b f32[N] -> f32[M, N] (the style-bank GEMV)."""
    _f32(x, wt, rank=2)
    _f32(b, rank=1)
    check(wt.shape[0] == x.shape[1] and b.shape[0] == wt.shape[1], "gemm_bias: x[M,K] wt[K,N] b[N]")
    out = _new(x, (x.shape[0], wt.shape[1]))
    _run("gemm_bias_f32_cuda", [x, wt, b], [out])
    return out


# --- frame-rate ([C, L]) ------------------------------------------------------------------------------------

def _conv_out(l, k, stride, padding, dilation):
    return (l + 2 * padding - dilation * (k - 1) - 1) // stride + 1


def _conv_rule(x, w, *, dilation, padding, stride):
    _f32(x, rank=2)
    _f32(w, rank=3)
    check(w.shape[1] == x.shape[0], f"w must be [Co, Ci, K]: x {tuple(x.shape)}, w {tuple(w.shape)}")
    check(stride >= 1 and dilation >= 1 and padding >= 0, "invalid stride/padding/dilation")
    lo = _conv_out(x.shape[1], w.shape[2], stride, padding, dilation)
    check(lo >= 1, "empty conv output")
    return (w.shape[0], lo)


def conv1d_f32_cuda(x, w, b, stride=1, padding=0, dilation=1):
    """F.conv1d: x f32[Ci, L], w f32[Co, Ci, K], b f32[Co] -> f32[Co, Lo]."""
    stride, padding, dilation = _int(stride, "stride"), _int(padding, "padding"), _int(dilation, "dilation")
    shape = _conv_rule(x, w, dilation=dilation, padding=padding, stride=stride)
    _f32(b, rank=1)
    check(b.shape[0] == w.shape[0], "bias must be f32[Co]")
    out = _new(x, shape, rows=True)
    _run("conv1d_f32_cuda", [x, w, b], [out], attrs_int=[dilation, padding, stride])
    return out


def conv1d_nobias_f32_cuda(x, w, stride=1, padding=0, dilation=1):
    """F.conv1d without bias."""
    stride, padding, dilation = _int(stride, "stride"), _int(padding, "padding"), _int(dilation, "dilation")
    shape = _conv_rule(x, w, dilation=dilation, padding=padding, stride=stride)
    out = _new(x, shape, rows=True)
    _run("conv1d_nobias_f32_cuda", [x, w], [out], attrs_int=[dilation, padding, stride])
    return out


def _convt_out(l, k, stride, padding, output_padding):
    return (l - 1) * stride - 2 * padding + k + output_padding


def conv_transpose1d_f32_cuda(x, w, b, stride=1, padding=0, output_padding=0):
    """F.conv_transpose1d: x f32[Ci, L], w f32[Ci, Co, K], b f32[Co] -> f32[Co, (L-1)s - 2p + K + op]."""
    stride, padding = _int(stride, "stride"), _int(padding, "padding")
    output_padding = _int(output_padding, "output_padding")
    _f32(x, rank=2)
    _f32(w, rank=3)
    _f32(b, rank=1)
    check(w.shape[0] == x.shape[0], f"w must be [Ci, Co, K]: x {tuple(x.shape)}, w {tuple(w.shape)}")
    check(b.shape[0] == w.shape[1], "bias must be f32[Co]")
    check(stride >= 1 and padding >= 0 and 0 <= output_padding < stride, "invalid stride/padding/output_padding")
    lo = _convt_out(x.shape[1], w.shape[2], stride, padding, output_padding)
    check(lo >= 1, "empty conv_transpose output")
    out = _new(x, (w.shape[1], lo))
    _run("conv_transpose1d_f32_cuda", [x, w, b], [out], attrs_int=[output_padding, padding, stride])
    return out


def convt_poly_weights_cuda(w, stride: int, padding: int):
    """torch ConvTranspose1d weight f32[Ci, Co, K] (K = taps*s, 2p = (taps-1)*s) -> the polyphase pack of
    conv_transpose1d_poly_f32_cuda: f32[Ci, s, taps, Co], entry [c, r, tt, co] = w[c, co, (r + p) % s + (taps-1-tt)*s]
    (the counterpart of convt_poly_weights_cpu, python/lokinfer/ops/kokoro.py:289-314; run once on constants)."""
    _f32(w, rank=3)
    s, p = _int(stride, "stride"), _int(padding, "padding")
    ci, co, k = w.shape
    taps = k // s
    check(taps * s == k and 2 * p == (taps - 1) * s and 0 <= p < s, "needs K = taps*s and 2p = (taps-1)*s")
    wp = _new(w, (ci, s, taps, co))
    _run("convt_poly_pack_f32_cuda", [w], [wp], attrs_int=[p, s])
    return wp


def conv_transpose1d_poly_f32_cuda(x, wp, b, res, stride, padding, taps, slope, pad_left=0, mean3=None, state=None):
    """reflect_pad_left(conv_transpose1d(leaky_relu(x, slope), w, b, stride, padding), pad_left) + res, polyphase
    (wp = convt_poly_weights_cuda(w, stride, padding), K = taps * stride): x f32[Ci, L] -> f32[Co, L*s + pad_left].
    mean3 = (x2, x3, scale): the input is ((x + x2) + x3) * scale. state = conv_transpose1d_prepare_f32_cuda(w, ...)
    runs the same contract on the tensor cores (ignored with mean3)."""
    pad_left, padding, stride = _int(pad_left, "pad_left"), _int(padding, "padding"), _int(stride, "stride")
    taps, slope = _int(taps, "taps"), _float(slope, "slope")
    _f32(x, res, rank=2)
    _f32(wp, rank=4)
    _f32(b, rank=1)
    check(wp.shape[0] == x.shape[0] and wp.shape[1] == stride and wp.shape[2] == taps and wp.shape[3] == b.shape[0],
          "wp must come from convt_poly_weights_cuda")
    check(2 * padding == (taps - 1) * stride and 0 <= padding < stride, "needs 2p = (taps-1)*s")
    check(pad_left in (0, 1), "pad_left must be 0 or 1")
    lo = x.shape[1] * stride + pad_left
    check(res.shape[0] == b.shape[0] and res.shape[1] == lo, "residual must be f32[Co, L*s + pad_left]")
    # padded rows only on the tensor-core route (the CUDA-core kernels of this op take contiguous rows)
    out = _new(x, (b.shape[0], lo), rows=state is not None and mean3 is None)
    at = [pad_left, padding, stride, taps]
    if mean3 is not None:
        x2, x3, sc = mean3
        _f32(x2, x3, rank=2)
        check(x2.shape == x.shape and x3.shape == x.shape, "x2 / x3 must match x")
        _run("conv_transpose1d_poly_mean3_f32_cuda", [x, x2, x3, wp, b, res], [out], attrs_int=at,
             attrs_float=[_float(sc, "in_scale"), slope])
    else:
        if state is not None:
            check(isinstance(state, ConvState) and state.shape == (int(x.shape[0]), int(b.shape[0]), taps * stride, stride),
                  "state must come from conv_transpose1d_prepare_f32_cuda of this weight")
        _run("conv_transpose1d_poly_f32_cuda", [x, wp, b, res], [out], attrs_int=at, attrs_float=[slope],
             state=None if state is None else state.handle)
    return out


def conv_transpose1d_dw_f32_cuda(x, w, b, stride=1, padding=0, output_padding=0):
    """Depthwise F.conv_transpose1d(groups=C): x f32[C, L], w f32[C, 1, K], b f32[C]
    (python/lokinfer/ops/kokoro.py:349-371)."""
    stride, padding = _int(stride, "stride"), _int(padding, "padding")
    output_padding = _int(output_padding, "output_padding")
    _f32(x, rank=2)
    _f32(w, rank=3)
    _f32(b, rank=1)
    check(w.shape[0] == x.shape[0] and w.shape[1] == 1, "w must be [C, 1, K]")
    check(b.shape[0] == x.shape[0], "bias must be f32[C]")
    check(stride >= 1 and padding >= 0 and 0 <= output_padding < stride, "invalid stride/padding/output_padding")
    lo = _convt_out(x.shape[1], w.shape[2], stride, padding, output_padding)
    check(lo >= 1, "empty conv_transpose output")
    out = _new(x, (x.shape[0], lo))
    _run("conv_transpose1d_dw_f32_cuda", [x, w, b], [out], attrs_int=[output_padding, padding, stride])
    return out


def upsample_nearest1d_f32_cuda(x, scale):
    """F.interpolate(mode='nearest', scale_factor=scale) (integer scale): f32[C, L] -> f32[C, L*scale]
    (python/lokinfer/ops/kokoro.py:392-402)."""
    scale = _int(scale, "scale")
    _f32(x, rank=2)
    check(scale >= 1, "scale must be >= 1")
    out = _new(x, (x.shape[0], x.shape[1] * scale))
    _run("upsample_nearest1d_f32_cuda", [x], [out], attrs_int=[scale])
    return out


def concat_rows_f32_cuda(*xs):
    """torch.cat(xs, dim=0) for 2..8 f32[R_i, C] (python/lokinfer/ops/kokoro.py:152-161)."""
    check(2 <= len(xs) <= 8, "concat takes 2..8 operands")
    _f32(*xs, rank=2)
    check(all(x.shape[1] == xs[0].shape[1] for x in xs), "column counts differ")
    out = _new(xs[0], (sum(int(x.shape[0]) for x in xs), xs[0].shape[1]))
    _run("concat_rows_f32_cuda", list(xs), [out])
    return out


def adain1d_f32_cuda(x, gb, eps=1e-5):
    """(1 + gb[:C, None]) * instance_norm(x) + gb[C:, None] (biased var) over x f32[C, L]."""
    _f32(x, rank=2)
    _f32(gb, rank=1)
    check(gb.shape[0] == x.shape[0] * 2, "gb must be f32[2C]")
    out = _new(x, x.shape)
    _run("adain1d_f32_cuda", [x, gb], [out], attrs_float=[_float(eps, "eps")])
    return out


def snake_f32_cuda(x, alpha):
    """x + (1/alpha) * sin(alpha * x)^2, alpha f32[C] per channel of x f32[C, L]."""
    _f32(x, rank=2)
    _f32(alpha, rank=1)
    check(alpha.shape[0] == x.shape[0], "alpha must be f32[C]")
    out = _new(x, x.shape)
    _run("snake_f32_cuda", [x, alpha], [out])
    return out


def space_to_depth_f32_cuda(x, stride, padding, taps, rows=None):
    """Polyphase view of the input of a strided conv (no counterpart in the reference): y[ci * stride + r, t] =
    x[ci, stride * t + r - padding], zero outside x, t in [0, Lo + taps - 1) where Lo is the length of
    conv1d(x, w[Co, Ci, taps * stride], stride, padding); rows beyond Ci * stride (up to `rows`) are zero. With
    polyphase_conv_weights(w, stride, rows), conv1d(y, w') at stride 1 and no padding is that strided conv."""
    stride, padding, taps = _int(stride, "stride"), _int(padding, "padding"), _int(taps, "taps")
    _f32(x, rank=2)
    check(stride >= 1 and padding >= 0 and taps >= 1, "invalid stride / padding / taps")
    ci, l = int(x.shape[0]), int(x.shape[1])
    lo = _conv_out(l, taps * stride, stride, padding, 1)
    check(lo >= 1, "empty conv output")
    rows = ci * stride if rows is None else _int(rows, "rows")
    check(rows >= ci * stride, "rows must be >= Ci * stride")
    y = _new(x, (rows, lo + taps - 1), rows=True)
    _run("space_to_depth_f32_cuda", [x], [y], attrs_int=[padding, stride])
    return y


def polyphase_conv_weights(w, stride, rows=None):
    """w f32[Co, Ci, taps * stride] (numpy) -> w' f32[Co, rows, taps] with w'[co, ci * stride + r, j] =
    w[co, ci, stride * j + r] and zeros in the rows beyond Ci * stride: the weights of the stride-1 conv over
    space_to_depth_f32_cuda(x, stride, ...)."""
    import numpy as np
    co, ci, k = w.shape
    check(k % stride == 0, "K must be a multiple of the stride")
    taps = k // stride
    rows = ci * stride if rows is None else int(rows)
    check(rows >= ci * stride, "rows must be >= Ci * stride")
    out = np.zeros((co, rows, taps), dtype=np.float32)
    out[:, : ci * stride, :] = np.asarray(w, dtype=np.float32).reshape(co, ci, taps, stride).transpose(0, 1, 3, 2).reshape(
        co, ci * stride, taps)
    return out


def pad_reflect1d_f32_cuda(x, left, right):
    """F.pad(x, (left, right), mode='reflect') over f32[C, L] (left, right < L)."""
    left, right = _int(left, "left"), _int(right, "right")
    _f32(x, rank=2)
    check(left >= 0 and right >= 0, "negative padding")
    check(x.shape[1] >= max(left, right) + 1, "reflect padding must be < L")
    out = _new(x, (x.shape[0], x.shape[1] + left + right))
    _run("pad_reflect1d_f32_cuda", [x], [out], attrs_int=[left, right])
    return out


def istft_logits_f32_cuda(x, n_fft=20, hop=5):
    """torch.istft(exp(x[:K]) * e^{i sin(x[K:])}, periodic hann, center), K = n_fft/2+1:
    f32[n_fft+2, L] -> f32[hop*(L-1)]."""
    n_fft, hop = _int(n_fft, "n_fft"), _int(hop, "hop")
    _f32(x, rank=2)
    check(n_fft >= 2 and n_fft % 2 == 0 and hop >= 1, "n_fft must be even, hop >= 1")
    check(n_fft <= 126, "n_fft must be <= 126 (the kernel keeps n_fft/2 + 1 <= 64 bins on the stack)")
    check(x.shape[0] == n_fft + 2, f"x must be f32[n_fft+2, L], got {tuple(x.shape)}")
    check(x.shape[1] >= 2, "need at least 2 frames")
    out = _new(x, ((x.shape[1] - 1) * hop,))
    _run("istft_logits_f32_cuda", [x], [out], attrs_int=[hop, n_fft])
    return out


def harmonic_source_f32_cuda(f0, noise, w, b):
    """Kokoro SourceModuleHnNSF (SineGen x300, 9 harmonics, Linear 9->1, tanh) in the reference kernel's op order.
    f0 f32[n] (80 Hz curve), noise f32[300n, 9] (the randn_like draw), w f32[9], b f32[1] -> f32[300n]
    (python/lokinfer/ops/kokoro.py:417-426)."""
    _f32(f0, w, b, rank=1)
    _f32(noise, rank=2)
    s = f0.shape[0] * 300
    check(noise.shape[0] == s and noise.shape[1] == 9, f"noise must be f32[300n, 9], got {tuple(noise.shape)}")
    check(w.shape[0] == 9 and b.shape[0] == 1, "w must be f32[9], b f32[1]")
    check(1 <= f0.shape[0] <= 27962, "f0 must hold 1..27962 frames")
    out = _new(f0, (s,))
    _run("harmonic_source_f32_cuda", [f0, noise, w, b], [out])
    return out


def harmonic_source_rng_f32_cuda(f0, w, b, seed):
    """Same as harmonic_source_f32_cuda, with the noise generated in-kernel from `seed` (an i64 scalar), like
    torch's randn_like after manual_seed (Philox4x32-10 + Box-Muller; deterministic per seed, not torch's bit stream)
    (python/lokinfer/ops/kokoro.py:429-435). The seed travels as the reference packs scalar operands: a pointer to an
    8-byte host slot."""
    import ctypes
    _f32(f0, w, b, rank=1)
    check(isinstance(seed, int) and not isinstance(seed, bool) and -(1 << 63) <= seed < (1 << 64),
          "seed must be an i64 scalar")
    check(w.shape[0] == 9 and b.shape[0] == 1, "w must be f32[9], b f32[1]")
    check(1 <= f0.shape[0] <= 27962, "f0 must hold 1..27962 frames")
    out = _new(f0, (f0.shape[0] * 300,))
    if not f0.is_cuda:
        return out
    check(all(t.is_cuda and t.device == f0.device and t.is_contiguous() for t in (f0, w, b)),
          "harmonic_source_rng_f32_cuda: operands must be contiguous tensors of one cuda device; there is no CPU path")
    slot = ctypes.c_int64(seed if seed < (1 << 63) else seed - (1 << 64))
    ptrs = [f0.data_ptr(), w.data_ptr(), b.data_ptr(), ctypes.addressof(slot), out.data_ptr()]
    ints = [f0.shape[0], 9, 1, out.shape[0]]
    with torch.cuda.device(f0.device):
        _lib.run("harmonic_source_rng_f32_cuda", ptrs, ints, (), None, _stream())
    if _profile is not None:
        _profile.count += 1
    return out


def stft_magphase_f32_cuda(x, n_fft=20, hop=5):
    """torch.stft(center, reflect, periodic hann(n_fft), onesided) -> cat(abs, angle):
    f32[S] -> f32[n_fft+2, S//hop+1] (python/lokinfer/ops/kokoro.py:438-449)."""
    n_fft, hop = _int(n_fft, "n_fft"), _int(hop, "hop")
    _f32(x, rank=1)
    check(n_fft >= 2 and n_fft % 2 == 0 and hop >= 1, "n_fft must be even, hop >= 1")
    check(n_fft <= 64, "n_fft must be <= 64 (the windowed basis is kept in shared memory)")
    check(x.shape[0] >= n_fft // 2 + 1, "signal must be longer than n_fft/2 (reflect pad)")
    out = _new(x, (n_fft + 2, x.shape[0] // hop + 1))
    _run("stft_magphase_f32_cuda", [x], [out], attrs_int=[hop, n_fft])
    return out


# --- fused frame-rate conv -----------------------------------------------------------------------------------

def conv_tile(ci: int, k: int) -> int:
    """The reference's default time tile (python/lokinfer/ops/kokoro.py:474-479). The CUDA kernels pick their own
    tiling; the attribute is packed for ABI compatibility and ignored."""
    t = (3 << 20) // (4 * ci * k) // STAT_CHUNK * STAT_CHUNK
    return max(STAT_CHUNK, min(768, t))


def _fused_rule(x, w, b, affine, extra, *, dilation, padding, tile):
    shape = _conv_rule(x, w, dilation=dilation, padding=padding, stride=1)
    _f32(b, *extra, rank=1)
    _f32(affine, rank=2)
    check(b.shape[0] == w.shape[0], "bias must be f32[Co]")
    check(affine.shape[0] == 3 and affine.shape[1] == x.shape[0], "affine must be f32[3, Ci]")
    check(tile >= STAT_CHUNK and tile % STAT_CHUNK == 0, f"tile must be a positive multiple of {STAT_CHUNK}")
    return shape, (shape[0], ceildiv(shape[1], STAT_CHUNK), 2)


def _fused_attrs(x, w, padding, dilation, tile):
    if tile is None:
        tile = conv_tile(int(x.shape[0]), int(w.shape[2]))
    return dict(padding=_int(padding, "padding"), dilation=_int(dilation, "dilation"), tile=_int(tile, "tile"))


class ConvState:
    """Prepared state of one constant conv weight for the tensor-core kernel: the hi / lo operand pack in the UMMA
    layout plus the host handle passed as `state` (the reference's prepare hook result, kernel.h:56-58)."""

    def __init__(self, handle, wp, shape):
        self.handle, self.wp, self.shape = handle, wp, shape
        self.fmt = "tf32" if _conv_path == "tf32" else "f16"  # operand format of the pack

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().lkc_conv1d_state_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


def conv1d_prepare_f32_cuda(w):
    """Packs a constant conv weight f32[Co, Ci, K] once for the tensor-core path (run at init, like the reference's
    hoisted weight preparation, docs/passes/hoist-init.md). Returns None when the shape is served by the CUDA-core
    kernel instead (Ci % 16 != 0 or K > 64)."""
    _f32(w, rank=3)
    check(w.is_contiguous(), "w must be contiguous")
    co, ci, k = (int(d) for d in w.shape)

    def pack():
        n = int(_lib.lib().lkc_conv1d_tc_pack_floats(co, ci, k))
        if n == 0:
            return None
        wp = torch.empty((n,), dtype=torch.float32, device=w.device)
        _run("conv1d_tc_pack_f32_cuda", [w], [wp])
        handle = _lib.lib().lkc_conv1d_state_create(wp.data_ptr(), co, ci, k)
        if not handle:
            raise _lib.LkcError(_lib.last_error())
        return ConvState(handle, wp, (co, ci, k))

    return _pack_checked(pack)


def conv_transpose1d_prepare_f32_cuda(w, stride, padding):
    """Packs a constant ConvTranspose1d weight f32[Ci, Co, K] once for the tensor-core path of
    conv_transpose1d_poly_f32_cuda. Returns None when the shape is served by the CUDA-core kernel only (the
    tensor-core path takes stride 6 or 10 with K = 2 stride, 2 padding = stride, Ci % 16 == 0)."""
    _f32(w, rank=3)
    s, p = _int(stride, "stride"), _int(padding, "padding")
    check(w.is_contiguous(), "w must be contiguous")
    ci, co, k = (int(d) for d in w.shape)

    def pack():
        n = int(_lib.lib().lkc_convt_tc_pack_floats(ci, co, k, s, p))
        if n == 0:
            return None
        wp = torch.empty((n,), dtype=torch.float32, device=w.device)
        _run("convt_tc_pack_f32_cuda", [w], [wp], attrs_int=[p, s])
        handle = _lib.lib().lkc_convt_state_create(wp.data_ptr(), ci, co, k, s, p)
        if not handle:
            raise _lib.LkcError(_lib.last_error())
        return ConvState(handle, wp, (ci, co, k, s))

    return _pack_checked(pack)


STATUS_F16_ACT, STATUS_F16_WEIGHTS = 0x10000, 0x20000
_conv_path = "auto"


def _pack_checked(pack):
    """Runs a weight pack and, if the f16 split reported a weight beyond the f16 range (status bit 0x20000: the value
    was clamped), packs the weight again in the tf32 format, which has the range of f32. Reads the status word, so it
    synchronises the device: packing is init-time work."""
    with torch.cuda.device(torch.cuda.current_device()):
        st = pack()
        if st is None or _conv_path != "auto":
            return st
        status = conv_tc_status()
        if status & ~STATUS_F16_WEIGHTS:
            raise RuntimeError(f"tensor-core conv kernels reported status {status:#x} before this weight was packed")
        if status & STATUS_F16_WEIGHTS:
            set_conv_path("tf32")
            try:
                st = pack()
            finally:
                set_conv_path("auto")
        return st


def conv_tc_status(reset=True) -> int:
    """Status word of the tensor-core conv kernels on the current device after everything queued on it has finished
    (the call synchronises the device): 0 = ok; low 16 bits = the first bounded wait that gave up; 0x10000 = an
    activation beyond the f16 range overflowed its f16 operand; 0x20000 = a weight beyond the f16 range was clamped in a pack."""
    import ctypes
    v = ctypes.c_int(0)
    if _lib.lib().lkc_conv1d_tc_status(ctypes.byref(v), 1 if reset else 0) != 0:
        raise _lib.LkcError(_lib.last_error())
    return int(v.value)


TC_PROFILE_FIELDS = ("mma_wait_act", "mma_wait_drain", "mma_wait_weights", "mma_wait_lofold", "mma_total",
                     "epi_wait_hi", "epi_wait_lo", "epi_preload", "epi_final", "epi_total",
                     "pro_wait_free", "pro_wait_raw", "pro_transform", "pro_total", "wpro_wait_free", "wpro_total")


def conv_tc_status_async(status_host) -> None:
    """Queues a copy of the status word into `status_host` (a pinned int32 host tensor with one element) behind the
    work already on the current stream; synchronises nothing and clears nothing (see conv_tc_status)."""
    check(status_host.dtype == torch.int32 and status_host.numel() == 1 and status_host.is_pinned(),
          "status_host must be a pinned int32 tensor with one element")
    if _lib.lib().lkc_conv1d_tc_status_async(status_host.data_ptr(), _stream()) != 0:
        raise _lib.LkcError(_lib.last_error())


def conv_tc_profile(enable: bool) -> dict:
    """Turns the tensor-core kernel's role-level cycle counters on / off and returns (then clears) what was recorded:
    cycles summed over CTAs and launches, one representative warp per role. Synchronises the device. Only in a
    library built with LKC_TC_PROF=1 (python -m lokinfer_b200.build --prof); the product build raises."""
    import ctypes
    buf = (ctypes.c_int64 * 16)()
    if _lib.lib().lkc_conv1d_tc_profile(1 if enable else 0, buf) != 0:
        raise _lib.LkcError(_lib.last_error())
    return dict(zip(TC_PROFILE_FIELDS, [int(v) for v in buf]))


def set_conv_path(mode: str) -> None:
    """Convolution path: "auto" = tensor cores when a prepared state is passed and the shape is eligible, operands
    split into f16 hi/lo halves; "tf32" = the same with tf32 hi/lo halves; "simt" = CUDA cores only. The operand
    format is fixed when a state is prepared, so states made under "auto" keep the f16 split after a switch to
    "tf32" and the other way round."""
    global _conv_path
    modes = {"auto": 0, "simt": 1, "tf32": 2}
    check(mode in modes, "mode must be 'auto', 'simt' or 'tf32'")
    if _lib.lib().lkc_set_conv_path(modes[mode]) != 0:
        raise _lib.LkcError(_lib.last_error())
    _conv_path = mode


def set_conv_io(mode: str) -> None:
    """Global-memory route of the tensor-core kernels: "tma" (default) = tiled bulk loads / stores for every tensor
    whose rows are 16-byte aligned, "plain" = 4-byte accesses for all (the A/B partner of the parity tests)."""
    modes = {"tma": 0, "plain": 1}
    check(mode in modes, "mode must be 'tma' or 'plain'")
    if _lib.lib().lkc_set_conv_io(modes[mode]) != 0:
        raise _lib.LkcError(_lib.last_error())


def _state_of(w, state):
    if state is None:
        return None
    check(isinstance(state, ConvState) and state.shape == tuple(int(d) for d in w.shape),
          "state must come from conv1d_prepare_f32_cuda of this weight")
    return state.handle


def conv1d_snake_f32_cuda(x, w, b, affine, alpha, residual=None, padding=0, dilation=1, tile=None, state=None):
    """conv1d(snake((x - mean) * scale + beta, alpha), w) + b [+ residual] -> (out f32[Co, Lo], stats f32[Co, T, 2]).
    affine = f32[3, Ci] rows (mean, scale, beta), e.g. from adain_affine_f32_cuda."""
    at = _fused_attrs(x, w, padding, dilation, tile)
    _f32(alpha, rank=1) if isinstance(alpha, torch.Tensor) else check(False, "alpha must be f32[Ci]")
    check(alpha.shape[0] == x.shape[0], "alpha must be f32[Ci]")
    oshape, sshape = _fused_rule(x, w, b, affine, [alpha], **at)
    out, stats = _new(x, oshape, rows=True), _new(x, sshape)
    ai = [at["dilation"], at["padding"], at["tile"]]
    if residual is None:
        _run("conv1d_snake_f32_cuda", [x, w, b, affine, alpha], [out, stats], attrs_int=ai, state=_state_of(w, state))
    else:
        _f32(residual, rank=2)
        check(tuple(residual.shape) == tuple(oshape), "residual must match the output")
        _run("conv1d_snake_res_f32_cuda", [x, w, b, affine, alpha, residual], [out, stats], attrs_int=ai,
             state=_state_of(w, state))
    return out, stats


def conv1d_leaky_f32_cuda(x, w, b, affine, slope=0.1, residual=None, out_scale=1.0, padding=0, dilation=1,
                          tile=None, state=None):
    """(conv1d(leaky_relu((x - mean) * scale + beta, slope), w) + b [+ residual]) * out_scale -> (out, stats)."""
    at = _fused_attrs(x, w, padding, dilation, tile)
    slope, out_scale = _float(slope, "slope"), _float(out_scale, "out_scale")
    oshape, sshape = _fused_rule(x, w, b, affine, [], **at)
    out, stats = _new(x, oshape, rows=True), _new(x, sshape)
    ai = [at["dilation"], at["padding"], at["tile"]]
    if residual is None:
        check(out_scale == 1.0, "out_scale needs a residual")
        _run("conv1d_leaky_f32_cuda", [x, w, b, affine], [out, stats], attrs_int=ai, attrs_float=[slope],
             state=_state_of(w, state))
    else:
        _f32(residual, rank=2)
        check(tuple(residual.shape) == tuple(oshape), "residual must match the output")
        _run("conv1d_leaky_res_f32_cuda", [x, w, b, affine, residual], [out, stats], attrs_int=ai,
             attrs_float=[out_scale, slope], state=_state_of(w, state))
    return out, stats


def conv1d_affine_f32_cuda(x, w, b, affine, padding=0, dilation=1, tile=None, state=None):
    """conv1d((x - mean) * scale + beta, w) + b -> (out, stats)."""
    at = _fused_attrs(x, w, padding, dilation, tile)
    oshape, sshape = _fused_rule(x, w, b, affine, [], **at)
    out, stats = _new(x, oshape, rows=True), _new(x, sshape)
    _run("conv1d_affine_f32_cuda", [x, w, b, affine], [out, stats],
         attrs_int=[at["dilation"], at["padding"], at["tile"]], state=_state_of(w, state))
    return out, stats


def conv1d_leaky_mean3_f32_cuda(x, x2, x3, w, b, affine, in_scale, slope, padding=0, dilation=1, tile=None,
                                state=None):
    """conv1d_leaky_f32_cuda on ((x + x2) + x3) * in_scale (add3_scale fused into the input window: the generator's
    resblock mean feeding conv_post; the contract of conv1d_leaky_wino_mean3_f32_cpu,
    python/lokinfer/ops/kokoro.py:641-653, as a direct conv) -> (out, stats)."""
    at = _fused_attrs(x, w, padding, dilation, tile)
    _f32(x2, x3, rank=2)
    check(x2.shape == x.shape and x3.shape == x.shape, "x2 / x3 must match x")
    oshape, sshape = _fused_rule(x, w, b, affine, [], **at)
    out, stats = _new(x, oshape), _new(x, sshape)
    _run("conv1d_leaky_mean3_f32_cuda", [x, x2, x3, w, b, affine], [out, stats],
         attrs_int=[at["dilation"], at["padding"], at["tile"]],
         attrs_float=[_float(in_scale, "in_scale"), _float(slope, "slope")], state=_state_of(w, state))
    return out, stats


def channel_stats_f32_cuda(x):
    """Per-(channel, 128-sample chunk) (mean, M2) of x f32[C, L] -> f32[C, ceil(L / 128), 2]."""
    _f32(x, rank=2)
    check(x.shape[1] >= 1, "empty sequence")
    stats = _new(x, (x.shape[0], ceildiv(x.shape[1], STAT_CHUNK), 2))
    _run("channel_stats_f32_cuda", [x], [stats])
    return stats


def adain_affine_f32_cuda(stats, gb, length, eps=1e-5):
    """AdaIN from chunk stats over `length` samples -> affine f32[3, C] = (mean, (1 + g) / std, b)."""
    _f32(stats, rank=3)
    _f32(gb, rank=1)
    length = _int(length, "length")
    c = stats.shape[0]
    check(gb.shape[0] == 2 * c, "gb must be f32[2C]")
    check(stats.shape[1] == ceildiv(length, STAT_CHUNK), "stats chunks don't match length")
    affine = _new(stats, (3, c))
    _run("adain_affine_f32_cuda", [stats, gb], [affine], attrs_int=[length], attrs_float=[_float(eps, "eps")])
    return affine


def registered_kernels():
    """Kernel names in the library registry; every op above resolves its kernel by name through it."""
    return _lib.registered_kernels()
