"""One utterance of the Kokoro generator cut along time across the GPUs of one node.

The reference runs one utterance on one device (batch is always 1, docs/impl-notes/research-kokoro.md:67) and has no
multi-GPU path; what has to be preserved is its arithmetic: every conv sees its true neighbourhood (zero padding
applied after the activation, and only at the two ends of the utterance, kernels/cpu/kokoro_conv_fused.cpp:127-135),
and every AdaIN sees the statistics of the whole utterance, combined exactly as on one device
(kokoro_conv_fused.cpp:641-664: chunk grid of 128 columns from t = 0, combine in double).

Partition: rank k owns input frames [bx[k], bx[k+1]) with every inner boundary a multiple of 64 frames. That makes its
stage-0 range [10 bx[k], 10 bx[k+1]) and its stage-1 range [60 bx[k], 60 bx[k+1]) (rank 0 also owns the reflect
column 0 of stage 1, the last rank ends at 60 T + 1) start on multiples of 128 columns, so the chunk statistics a rank
computes over its own columns are exactly the chunks of the unsharded tensor. Every activation tensor lives in a local
buffer [C, MARGIN + longest shard + MARGIN]; the margins hold the neighbours' boundary columns (the receptive-field
halo, at most 25 columns for k = 11, dilation 5).

After each producing kernel comes one exchange (lkc_shard_push + lkc_shard_wait, or both in one launch with
lkc_shard_exchange when every rank has its own GPU; csrc/shard.cu): the boundary columns
go into the neighbours' margins and the rank's slice of the chunk statistics into every rank's copy of the whole
statistics row, by plain stores to peer memory, then a release flag per destination; the consumer waits (bounded) on
its own flags. About 53 exchanges per forward: the sharded forward is bound by their latency, not by bandwidth.

Two fabrics provide the peer pointers: IpcFabric (one process per GPU, torch.distributed for the hand-shake, CUDA IPC
for the mapping) and LocalFabric (all ranks in one process on one GPU, stepped in lock-step: every rank pushes before
any rank waits; this is how the logic is tested on a single GPU).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, ops
from .generator import DILATIONS, RES_KERNELS
from .synth import shapes

MARGIN = 32  # halo columns kept on both sides of a shard (a multiple of 4: rows stay 16-byte aligned)
MAX_FLAGS = 16


class Partition:
    """Time ranges of every rank for an utterance of t input frames."""

    def __init__(self, t: int, world: int):
        ops.check(world >= 1 and t >= 1, "need t >= 1 frames and world >= 1")
        inner = [64 * round(k * t / (64 * world)) for k in range(1, world)]
        self.bx = [0] + inner + [t]
        ops.check(all(b > a for a, b in zip(self.bx, self.bx[1:])),
                  f"an utterance of {t} frames is too short for {world} time shards of at least 64 frames")
        self.t, self.world = t, world
        sh = shapes(t)
        self.l0, self.l1, self.samples = sh["L0"], sh["L1"], sh["S"]
        self.b0 = [10 * b for b in self.bx]
        self.b1 = [0] + [60 * b for b in self.bx[1:-1]] + [self.l1]
        self.bs = [300 * b for b in self.bx]  # output samples

    def rng(self, stage: int, k: int):
        b = (self.b0, self.b1)[stage]
        return b[k], b[k + 1]

    def longest(self, stage: int) -> int:
        b = (self.b0, self.b1)[stage]
        return max(y - x for x, y in zip(b, b[1:]))


class _Raw:
    """A device allocation as a __cuda_array_interface__ object (wrapped zero-copy by torch.as_tensor)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class Arena:
    """One rank's peer-mappable memory: a cudaMalloc'ed block (lkc_peer_alloc) handed out by a bump allocator, so
    that the same sequence of allocations gives the same offsets on every rank."""

    def __init__(self, nbytes: int, device):
        self.device = torch.device(device)
        p = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            if _lib.lib().lkc_peer_alloc(ctypes.c_uint64(nbytes), ctypes.byref(p)) != 0:
                raise _lib.LkcError(_lib.last_error())
        self.base, self.nbytes, self.used = int(p.value), nbytes, 0
        self.bytes = torch.as_tensor(_Raw(self.base, nbytes), device=self.device)

    def alloc(self, shape, dtype=torch.float32):
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = (self.used + 255) // 256 * 256
        ops.check(off + nbytes <= self.nbytes, "time-shard arena exhausted")
        self.used = off + nbytes
        return self.bytes[off: off + nbytes].view(dtype).view(*[int(d) for d in shape])

    def offset(self, t) -> int:
        return t.data_ptr() - self.base

    def close(self):
        if self.base:
            self.bytes = None
            with torch.cuda.device(self.device):
                _lib.lib().lkc_peer_free(ctypes.c_void_p(self.base))
            self.base = 0


class LocalFabric:
    """All ranks in this process (one GPU): a peer's arena is simply that rank's arena. Pushes and waits stay separate
    launches: every rank's push is queued before any rank's wait."""

    fused = False

    def __init__(self, world: int, nbytes: int, device):
        self.world = world
        self.arenas = [Arena(nbytes, device) for _ in range(world)]

    def arena(self, rank):
        return self.arenas[rank]

    def peer_base(self, me, rank):
        return self.arenas[rank].base


class IpcFabric:
    """One process per GPU: the arenas are exchanged as CUDA IPC handles over the process group. An exchange is one
    launch (lkc_shard_exchange: push, then wait for the own flags)."""

    fused = True

    def __init__(self, nbytes: int, device, group=None):
        import torch.distributed as dist

        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self._arena = Arena(nbytes, device)
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self._arena.device):
            if _lib.lib().lkc_peer_handle(ctypes.c_void_p(self._arena.base), handle) != 0:
                raise _lib.LkcError(_lib.last_error())
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=self._arena.device)
        every = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(every, mine, group=group)
        self._bases = []
        for r, h in enumerate(every):
            if r == self.rank:
                self._bases.append(self._arena.base)
                continue
            raw = (ctypes.c_ubyte * 64)(*h.cpu().tolist())
            p = ctypes.c_void_p()
            with torch.cuda.device(self._arena.device):
                if _lib.lib().lkc_peer_open(raw, ctypes.byref(p)) != 0:
                    raise _lib.LkcError(_lib.last_error())
            self._bases.append(int(p.value))

    def arena(self, rank):
        ops.check(rank == self.rank, "only the local arena is addressable as a tensor")
        return self._arena

    def peer_base(self, me, rank):
        return self._bases[rank]


class _Copy(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("src_pitch", ctypes.c_int64),
                ("dst_pitch", ctypes.c_int64), ("rows", ctypes.c_int64), ("cols", ctypes.c_int64)]


class _Push(ctypes.Structure):
    _fields_ = [("copies", _Copy * 16), ("num_copies", ctypes.c_int32), ("flags", ctypes.c_void_p * MAX_FLAGS),
                ("num_flags", ctypes.c_int32), ("epoch", ctypes.c_void_p), ("ticket", ctypes.c_void_p)]


class ShardBuf:
    """One rank's part of a [C, L] activation tensor: `full` f32[C, width] with the rank's n columns at [MARGIN,
    MARGIN + n) and halo columns around them."""

    def __init__(self, full, n, stage):
        self.full, self.n, self.stage = full, n, stage

    @property
    def own(self):
        return self.full[:, MARGIN: MARGIN + self.n]


class TimeShardedGenerator:
    """Rank `rank` of `world` of a time-sharded forward. Weights and prepared conv states come from a Generator of the
    same device (every rank holds all weights: 80 MB)."""

    def __init__(self, gen, t: int, rank: int, world: int, fabric, wait_limit_ns: int = 200_000_000):
        ops.check(world <= MAX_FLAGS - 2, "too many ranks for the flag layout")
        self.gen, self.rank, self.world, self.fabric = gen, rank, world, fabric
        self.part = Partition(t, world)
        self.arena = fabric.arena(rank)
        self.wait_limit_ns = int(wait_limit_ns)
        self.device = gen.device
        a = self.arena
        # control block first (same offsets on every rank): epoch, status, tickets, flags
        self.max_sync = 96
        self.ctl = a.alloc((4,), torch.int32)  # [epoch, status, -, -]
        self.tickets = a.alloc((self.max_sync,), torch.int32)
        self.flags = a.alloc((self.max_sync, MAX_FLAGS), torch.int32)
        self._bufs, self._cursor, self._sync = [], 0, 0
        self._stream, self._keep = None, []
        self.concurrent = True  # independent branches on side streams (as Generator.forward does)
        self._lib = _lib.lib()
        self._lib.lkc_shard_push.argtypes = [ctypes.POINTER(_Push), ctypes.c_void_p]
        self._lib.lkc_shard_wait.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_void_p,
                                             ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
        self._lib.lkc_shard_epoch_bump.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        self._lib.lkc_shard_exchange.argtypes = [ctypes.POINTER(_Push), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]

    @staticmethod
    def arena_bytes(t: int, world: int) -> int:
        """Upper bound of one rank's arena for an utterance of t frames (every intermediate of a forward is kept)."""
        p = Partition(t, world)
        w0, w1 = p.longest(0) + 2 * MARGIN + 4, p.longest(1) + 2 * MARGIN + 4
        act = 4 * (256 * w0 * 30 + 128 * w1 * 30 + 22 * w1 * 2)
        stats = 8 * 60 * (256 * (p.l0 // 128 + 1) + 128 * (p.l1 // 128 + 1))
        return act + stats + (1 << 20)

    # ------------------------------------------------------------------ buffers (same order on every rank and forward)

    def _take(self, shape):
        if self._cursor < len(self._bufs):
            t = self._bufs[self._cursor]
            ops.check(tuple(t.shape) == tuple(int(d) for d in shape), "the sharded forward changed its buffer sequence")
        else:
            t = self.arena.alloc(shape)
            self._bufs.append(t)
        self._cursor += 1
        return t

    def _buf(self, c, stage):
        lo, hi = self.part.rng(stage, self.rank)
        width = -(-(self.part.longest(stage) + 2 * MARGIN) // ops.ROW_ALIGN) * ops.ROW_ALIGN
        return ShardBuf(self._take((c, width)), hi - lo, stage)

    def _stats(self, c, stage):
        """(whole statistics row f32[C, chunks, 2], this rank's slice of it, first chunk, chunks)."""
        lo, hi = self.part.rng(stage, self.rank)
        total = ops.ceildiv((self.part.l0, self.part.l1)[stage], ops.STAT_CHUNK)
        c0, n = lo // ops.STAT_CHUNK, ops.ceildiv(hi - lo, ops.STAT_CHUNK)
        whole = self._take((c, total, 2))
        return whole, whole[:, c0: c0 + n, :], c0, n

    def _peer(self, rank, t) -> int:
        return self.fabric.peer_base(self.rank, rank) + self.arena.offset(t)

    # ------------------------------------------------------------------ exchange

    def _push(self, buf, stats, wait_slots=None):
        """Boundary columns of buf -> the neighbours' margins; this rank's statistics slice -> every rank's row.
        wait_slots: flag slots of this exchange to wait for in the same launch (ranks on different GPUs only)."""
        k, n, sp = self.rank, self.world, self._sync
        ops.check(sp < self.max_sync, "too many exchanges in one forward")
        d = _Push()
        nc = nf = 0

        def flag(rank, slot):
            return self._peer(rank, self.flags[sp, slot])

        if buf is not None:
            stage = buf.stage
            c, pitch = int(buf.full.shape[0]), int(buf.full.stride(0))
            if k > 0:  # my first MARGIN columns -> right margin of the left neighbour
                lo, hi = self.part.rng(stage, k - 1)
                d.copies[nc] = _Copy(buf.full[:, MARGIN:].data_ptr(),
                                     self._peer(k - 1, buf.full) + 4 * (MARGIN + hi - lo), pitch, pitch, c, MARGIN)
                nc += 1
                d.flags[nf] = flag(k - 1, n + 1)
                nf += 1
            if k < n - 1:  # my last MARGIN columns -> left margin of the right neighbour
                d.copies[nc] = _Copy(buf.full[:, buf.n:].data_ptr(), self._peer(k + 1, buf.full), pitch, pitch, c,
                                     MARGIN)
                nc += 1
                d.flags[nf] = flag(k + 1, n)
                nf += 1
        if stats is not None:
            whole, mine, c0, nch = stats
            rows, pitch = int(whole.shape[0]), int(whole.stride(0))
            for r in range(n):
                if r == k:
                    continue
                d.copies[nc] = _Copy(mine.data_ptr(), self._peer(r, whole) + 8 * c0, pitch, pitch, rows, 2 * nch)
                nc += 1
                d.flags[nf] = flag(r, k)
                nf += 1
        d.num_copies, d.num_flags = nc, nf
        d.epoch, d.ticket = self.ctl[0:1].data_ptr(), self.tickets[sp: sp + 1].data_ptr()
        if nf and wait_slots:
            arr = (ctypes.c_void_p * len(wait_slots))(*[self.flags[sp, s].data_ptr() for s in wait_slots])
            if self._lib.lkc_shard_exchange(ctypes.byref(d), arr, len(wait_slots), 0,
                                            ctypes.c_uint64(self.wait_limit_ns),
                                            ctypes.c_void_p(self.ctl[1:2].data_ptr()),
                                            ctypes.c_void_p(ops._stream())) != 0:
                raise _lib.LkcError(_lib.last_error())
            return True
        if nf and self._lib.lkc_shard_push(ctypes.byref(d), ctypes.c_void_p(ops._stream())) != 0:
            raise _lib.LkcError(_lib.last_error())
        return False

    def _slots(self, halo: bool, stats: bool):
        k, n = self.rank, self.world
        slots = []
        if halo and k > 0:
            slots.append(n)
        if halo and k < n - 1:
            slots.append(n + 1)
        if stats:
            slots += [r for r in range(n) if r != k]
        return slots

    def _wait(self, halo: bool, stats: bool, delta=0, slots=None):
        sp = self._sync
        if slots is None:
            slots = self._slots(halo, stats)
        if slots:
            arr = (ctypes.c_void_p * len(slots))(*[self.flags[sp, s].data_ptr() for s in slots])
            if self._lib.lkc_shard_wait(arr, len(slots), ctypes.c_void_p(self.ctl[0:1].data_ptr()), delta,
                                        ctypes.c_uint64(self.wait_limit_ns),
                                        ctypes.c_void_p(self.ctl[1:2].data_ptr()),
                                        ctypes.c_void_p(ops._stream())) != 0:
                raise _lib.LkcError(_lib.last_error())

    def _exchange(self, buf, stats):
        """Generator step: push, then (after every rank has pushed, in the lock-step fabric) wait; one launch for both
        when every rank has its own GPU."""
        fused = getattr(self.fabric, "fused", False)
        waited = self._push(buf, stats, self._slots(buf is not None, stats is not None) if fused else None)
        yield
        torch.cuda.set_stream(self._stream)  # another rank of this process may have switched streams meanwhile
        if not waited:
            self._wait(buf is not None, stats is not None)
        self._sync += 1

    def _use(self, stream):
        """Queues what follows on `stream` (branches that do not depend on each other go to different streams, so that
        the exchange latency of one overlaps the convs of another)."""
        self._stream = stream
        torch.cuda.set_stream(stream)

    # ------------------------------------------------------------------ sharded ops

    def _ends(self):
        return self.rank == 0, self.rank == self.world - 1

    def _conv(self, name, x: ShardBuf, w_key, affine, k, d, stage, alpha=None, residual=None, slope=None):
        """Fused conv over this rank's columns: x is the whole local buffer (halo included), the zero padding applies
        only where the utterance ends."""
        gw = self.gen.w
        w, b = gw[w_key + ".weight"], gw[w_key + ".bias"]
        co = int(w.shape[0])
        out = self._buf(co, stage)
        whole, mine, c0, nch = self._stats(co, stage)
        first, last = self._ends()
        pad = d * (k - 1) // 2
        width = int(x.full.shape[1])
        window = [int(whole.shape[1]), MARGIN, MARGIN if first else 0, MARGIN + x.n if last else width]
        operands = [x.full, w, b, affine]
        if alpha is not None:
            operands.append(gw[alpha])
        if residual is not None:
            operands.append(residual.own)
        st = self.gen.conv_state.get(w_key)
        ops._run(name, operands, [out.own, mine], attrs_int=[d, pad, ops.conv_tile(int(w.shape[1]), k)],
                 attrs_float=[] if slope is None else [slope], state=None if st is None else st.handle, window=window)
        return out, (whole, mine, c0, nch)

    def _channel_stats(self, x: ShardBuf, stage):
        whole, mine, c0, nch = self._stats(int(x.full.shape[0]), stage)
        ops._run("channel_stats_f32_cuda", [x.own], [mine], window=[int(whole.shape[1])])
        return whole, mine, c0, nch

    def _resblock(self, x: ShardBuf, st, gb, prefix, k, stage):
        length = (self.part.l0, self.part.l1)[stage]
        for j, d in enumerate(DILATIONS):
            af = ops.adain_affine_f32_cuda(st[0], gb(f"{prefix}.adain1.{j}.fc"), length=length)
            xt, st1 = self._conv("conv1d_snake_f32_cuda", x, f"{prefix}.convs1.{j}", af, k, d, stage,
                                 alpha=f"{prefix}.alpha1.{j}")
            yield from self._exchange(xt, st1)
            af = ops.adain_affine_f32_cuda(st1[0], gb(f"{prefix}.adain2.{j}.fc"), length=length)
            x, st = self._conv("conv1d_snake_res_f32_cuda", xt, f"{prefix}.convs2.{j}", af, k, 1, stage,
                               alpha=f"{prefix}.alpha2.{j}", residual=x)
            yield from self._exchange(x, st)
        return x, st

    def _add3(self, a, b, c):
        out = ShardBuf(self._take(tuple(a.full.shape)), a.n, a.stage)
        ops._run("add3_scale_f32_cuda", [a.full, b.full, c.full], [out.full], attrs_float=[1.0 / 3.0])
        return out

    # ------------------------------------------------------------------ the forward, as a sequence of steps

    def steps(self, x, har, s):
        """The sharded forward as a Python generator that yields once per exchange, between its push and its wait.
        x f32[512, T], har f32[22, 60 T + 1], s f32[128]: the whole inputs on this rank's device (each rank reads its
        own slices). Ends by storing this rank's samples in self.audio (f32[300 (bx[k+1] - bx[k])])."""
        gen, part, k, n = self.gen, self.part, self.rank, self.world
        gw = gen.w
        first, last = self._ends()
        self._cursor, self._sync, self._keep = 0, 0, []
        cur = torch.cuda.current_stream(self.device)
        side = gen._side_streams() if self.concurrent else [cur] * 4
        try:
            self._use(cur)
            stream = ctypes.c_void_p(cur.cuda_stream)
            # a new epoch; nobody may write into this rank's margins before it has finished reading the last forward
            if self._lib.lkc_shard_epoch_bump(ctypes.c_void_p(self.ctl[0:1].data_ptr()), stream) != 0:
                raise _lib.LkcError(_lib.last_error())
            done_sp = self.max_sync - 1
            self._sync = done_sp
            self._wait(False, True, delta=-1)  # every peer's "done" flag of the previous forward
            self._sync = 0
            gb = gen.style(s)
            noise = [None, None]
            for i, k_noise in enumerate((7, 11)):  # the two noise branches only need `har`: side streams 0 and 1
                side[i].wait_stream(cur)
                self._use(side[i])
                lo, hi = part.rng(i, k)
                xs = self._buf(256 if i == 0 else 128, i)
                if i == 0:
                    s0, s1 = max(0, 6 * lo - 3), min(part.l1, 6 * hi + 3)
                    hs = har[:, s0:s1].contiguous()
                    ops._run("conv1d_f32_cuda", [hs, gw["noise_convs.0.weight"], gw["noise_convs.0.bias"]], [xs.own],
                             attrs_int=[1, 3, 6], window=[6 * lo - s0, 0, s1 - s0])
                else:
                    hs = har[:, lo:hi].contiguous()
                    ops._run("conv1d_f32_cuda", [hs, gw["noise_convs.1.weight"], gw["noise_convs.1.bias"]], [xs.own],
                             attrs_int=[1, 0, 1], window=[0, 0, hi - lo])
                self._keep.append(hs)
                st = self._channel_stats(xs, i)
                yield from self._exchange(xs, st)
                noise[i], _ = yield from self._resblock(xs, st, gb, f"noise_res.{i}", k_noise, i)
            rb = None
            for i, (k_up, u) in enumerate(((20, 10), (12, 6))):
                self._use(cur)
                cur.wait_stream(side[i])
                xi = self._buf(256 if i == 0 else 128, i)
                if i == 0:
                    hl, hr = int(not first), int(not last)
                    xin = x[:, part.bx[k] - hl: part.bx[k + 1] + hr].contiguous()
                    ops._run("conv_transpose1d_poly_f32_cuda",
                             [xin, gen.ups_wp[0], gw["ups.0.bias"], noise[0].own], [xi.own],
                             attrs_int=[0, 5, 10, 2], attrs_float=[0.1], state=gen.ups_state[0].handle,
                             window=[hl, hr])
                else:
                    xm = self._add3(rb[0], rb[1], rb[2])
                    n0 = xm.n
                    if first:
                        # columns 0 (the reflect column) .. 6 n0 of stage 1: one past this rank's range unless it is
                        # also the last rank
                        hr = int(not last)
                        xv = xm.full[:, MARGIN: MARGIN + n0 + hr]
                        cols = 6 * n0 + 1
                        ov, rv = xi.full[:, MARGIN: MARGIN + cols], noise[1].full[:, MARGIN: MARGIN + cols]
                        hl, pl = 0, 1
                    else:
                        # input columns b0 - 1 .. b1: stage-1 columns 6 b0 - 5 .. 6 b1 (unpadded 6 (b0 - 1) .. 6 b1 - 1)
                        hl, hr, pl = 1, int(not last), 0
                        xv = xm.full[:, MARGIN - 2: MARGIN + n0 + hr]
                        cols = 6 * (n0 + 1)
                        ov = xi.full[:, MARGIN - 5: MARGIN - 5 + cols]
                        rv = noise[1].full[:, MARGIN - 5: MARGIN - 5 + cols]
                    ops._run("conv_transpose1d_poly_f32_cuda", [xv, gen.ups_wp[1], gw["ups.1.bias"], rv], [ov],
                             attrs_int=[pl, 3, 6, 2], attrs_float=[0.1], state=gen.ups_state[1].handle,
                             window=[hl, hr])
                st = self._channel_stats(xi, i)
                yield from self._exchange(xi, st)
                side[2].wait_stream(cur)
                side[3].wait_stream(cur)
                new_rb = [None, None, None]
                # the k = 11 block is the longest: it stays on the main stream
                for j, stream_j in ((2, cur), (1, side[2]), (0, side[3])):
                    self._use(stream_j)
                    new_rb[j], _ = yield from self._resblock(xi, st, gb, f"resblocks.{3 * i + j}", RES_KERNELS[j], i)
                self._use(cur)
                cur.wait_stream(side[2])
                cur.wait_stream(side[3])
                rb = new_rb
            xm = self._add3(rb[0], rb[1], rb[2])
            post, _ = self._conv("conv1d_leaky_f32_cuda", xm, "conv_post", gen.ident128, 7, 1, 1, slope=0.01)
            yield from self._exchange(post, None)
            lo, hi = part.rng(1, k)
            hl, hr = (0 if first else 1), (0 if last else 2)
            frames = post.full[:, MARGIN - hl: MARGIN + post.n + hr]
            i0, i1 = part.bs[k], part.bs[k + 1]
            audio = self._take((i1 - i0,))
            ops._run("istft_logits_f32_cuda", [frames], [audio], attrs_int=[5, 20],
                     window=[part.l1, lo - hl, i0])
            self.audio, self.post = audio, post
            # tell every peer that this rank has finished reading its margins
            self._sync = done_sp
            d = _Push()
            nf = 0
            for r in range(n):
                if r != k:
                    d.flags[nf] = self._peer(r, self.flags[done_sp, k])
                    nf += 1
            d.num_copies, d.num_flags = 0, nf
            d.epoch, d.ticket = self.ctl[0:1].data_ptr(), self.tickets[done_sp: done_sp + 1].data_ptr()
            if nf and self._lib.lkc_shard_push(ctypes.byref(d), stream) != 0:
                raise _lib.LkcError(_lib.last_error())
        finally:
            torch.cuda.set_stream(cur)

    def forward(self, x, har, s):
        """One process per GPU: runs the steps back to back (push, then wait). Returns this rank's samples."""
        for _ in self.steps(x, har, s):
            pass
        return self.audio

    def capture(self, x, har, s):
        """Records one sharded forward on the given (static) input tensors into a CUDA graph, after two warm-up
        forwards; every rank has to call this at the same point (the warm-ups exchange halos like any forward).
        Returns the graph: replay() runs one forward, the samples land in self.audio."""
        dev = self.device
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.forward(x, har, s)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.forward(x, har, s)
        return g

    def status(self, reset=True) -> int:
        """Status word of the waits after everything queued has finished (0 = no wait gave up). Synchronises."""
        torch.cuda.synchronize(self.device)
        v = int(self.ctl[1].item())
        if reset and v:
            self.ctl[1] = 0
        return v


def forward_lockstep(ranks, x, har, s):
    """All ranks of a LocalFabric on one GPU: every rank runs up to its next push before any rank goes on to its
    wait, so each flag is already set when its wait starts (kernels that wait on one another must not be queued on
    one GPU in the other order). Returns the concatenated waveform."""
    gens = [r.steps(x, har, s) for r in ranks]
    live = True
    while live:
        live = False
        for g in gens:
            try:
                next(g)
                live = True
            except StopIteration:
                pass
    return torch.cat([r.audio for r in ranks])
