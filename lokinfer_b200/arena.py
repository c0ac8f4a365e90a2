"""A planned activation arena for the fixed op sequence of a forward: the counterpart, for this path, of the
reference's memory planner (src/compiler/plan_memory.cpp: liveness over the program, offsets into one arena per
device; src/runtime/executable.cpp:732-815: the arena pools the executable allocates once).

The generator's forward is a fixed program for a given input length, so the plan is made once:
  1. trace: one eager forward with a Tracer installed. Every result allocation (ops.allocator) and every kernel call
     (ops._run) is recorded with the stream it ran on and that stream's vector clock; stream joins (wait_stream) merge
     clocks. A tensor's life ends at its last use as an operand.
  2. plan: allocations are placed in program order at the lowest offset where they overlap no tensor that may still be
     in use. "May still be in use" is decided with the vector clocks, not with program order alone: branches on
     different streams run concurrently, so a block is reused only when every use of its previous tenant
     happens-before the new allocation (same stream, or separated by a join).
  3. run: the allocator hands out views of one device buffer at the planned offsets, in the same order.
The buffer is one allocation per device, made when the plan is made; a forward under the plan allocates nothing.
"""
from __future__ import annotations

import torch

ALIGN = 256  # bytes: keeps every tensor's base (and with padded rows every row) 16-byte aligned


class Tracer:
    """Records one forward: allocations, uses and stream joins, with vector clocks."""

    def __init__(self):
        self.allocs = []        # [{bytes, shape, clock (dict stream -> count), stream, uses [(stream, count)], pinned}]
        self.by_storage = {}    # storage data_ptr -> alloc index
        self.clocks = {}        # stream -> {stream: count}
        self._keep = []         # keeps traced tensors alive so that storage pointers stay unique during the trace

    def _clock(self, stream):
        return self.clocks.setdefault(stream, {stream: 0})

    def tick(self, stream):
        c = self._clock(stream)
        c[stream] = c.get(stream, 0) + 1
        return c[stream]

    def on_alloc(self, t, stream):
        self.tick(stream)
        self.by_storage[t.untyped_storage().data_ptr()] = len(self.allocs)
        self.allocs.append({"bytes": t.untyped_storage().nbytes(), "shape": tuple(t.shape), "stream": stream,
                            "clock": dict(self._clock(stream)), "uses": [], "pinned": False})
        self._keep.append(t)

    def on_run(self, tensors, stream):
        n = self.tick(stream)
        for t in tensors:
            i = self.by_storage.get(t.untyped_storage().data_ptr())
            if i is not None:
                self.allocs[i]["uses"].append((stream, n))

    def on_join(self, waiter, waited):
        """`waiter` will not run anything more until everything queued on `waited` so far has finished."""
        cw, cd = self._clock(waiter), self._clock(waited)
        for s, n in cd.items():
            if cw.get(s, 0) < n:
                cw[s] = n

    def pin(self, t):
        i = self.by_storage.get(t.untyped_storage().data_ptr())
        if i is not None:
            self.allocs[i]["pinned"] = True


def happens_before(uses, clock) -> bool:
    """True when every (stream, count) use is ordered before a point whose vector clock is `clock`."""
    return all(clock.get(s, 0) >= n for s, n in uses)


def plan(allocs):
    """Offsets for the traced allocations (same order) and the arena size: the library's planner (lkc_plan_memory,
    csrc/plan.cu). Greedy lowest-offset placement; a tensor blocks its range for every later allocation that it does
    not happen-before (pinned tensors block forever)."""
    import ctypes

    from . import _lib

    n = len(allocs)
    streams = sorted({s for a in allocs for s in list(a["clock"]) + [u[0] for u in a["uses"]] + [a["stream"]]},
                     key=repr)
    col = {s: i for i, s in enumerate(streams)}
    ns = max(1, len(streams))
    size = (ctypes.c_int64 * n)(*[int(a["bytes"]) for a in allocs])
    pinned = (ctypes.c_int32 * n)(*[1 if a["pinned"] else 0 for a in allocs])
    clock = (ctypes.c_int64 * (n * ns))()
    last = (ctypes.c_int64 * (n * ns))()
    for i, a in enumerate(allocs):
        for s, c in a["clock"].items():
            clock[i * ns + col[s]] = int(c)
        for s, c in a["uses"] + [(a["stream"], a["clock"][a["stream"]])]:
            j = i * ns + col[s]
            if last[j] < c:
                last[j] = int(c)
    offsets = (ctypes.c_int64 * n)()
    total = ctypes.c_int64(0)
    fn = _lib.lib().lkc_plan_memory
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_int64, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]
    if fn(n, ns, size, pinned, clock, last, ALIGN, offsets, ctypes.byref(total)) != 0:
        raise _lib.LkcError(_lib.last_error())
    return [int(o) for o in offsets], int(total.value)


class PlannedArena:
    """One device buffer plus the planned offsets; `allocator` replays the traced allocation sequence."""

    def __init__(self, tracer: Tracer, device):
        self.shapes = [a["shape"] for a in tracer.allocs]
        self.sizes = [a["bytes"] for a in tracer.allocs]
        self.offsets, self.nbytes = plan(tracer.allocs)
        self.unplanned_bytes = sum(-(-b // ALIGN) * ALIGN for b in self.sizes)
        self.buffer = torch.empty(max(self.nbytes, ALIGN), dtype=torch.uint8, device=device)
        self.cursor = 0

    def begin(self):
        self.cursor = 0

    def allocator(self, shape, device):
        i = self.cursor
        if i >= len(self.shapes) or tuple(int(d) for d in shape) != self.shapes[i]:
            raise RuntimeError("the forward changed its allocation sequence since the arena was planned")
        self.cursor += 1
        n = self.sizes[i]
        return self.buffer[self.offsets[i]: self.offsets[i] + n].view(torch.float32).view(*self.shapes[i])
