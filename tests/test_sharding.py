"""Utterance sharding (one process per GPU, no data-path collective): the plan is deterministic and balanced, and two
gloo ranks on CPU agree on it and reduce their timings the way bench.py does (max over ranks)."""
import os
import socket
import zlib

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lokinfer_b200 import sharding


def test_assign_is_a_balanced_partition():
    r = np.random.default_rng(0)
    lengths = r.integers(120, 801, 64).tolist()
    for ws in (1, 2, 4, 8):
        plan = sharding.assign(lengths, ws)
        flat = sorted(i for p in plan for i in p)
        assert flat == list(range(64))
        ld = sharding.loads(lengths, plan)
        assert max(ld) - min(ld) <= max(lengths)
        assert max(ld) <= 1.05 * sum(lengths) / ws + max(lengths) / 2
    assert sharding.assign([], 2) == [[], []]
    assert abs(sharding.audio_seconds([2080]) - 26.0) < 1e-12


def _worker(rank, world, port, lengths, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    plan = sharding.assign(lengths, world)
    mine = plan[rank]
    # every rank derives the same plan; check it by exchanging a hash of the whole plan
    h = torch.tensor([zlib.crc32(str(plan).encode())], dtype=torch.int64)
    hs = [torch.zeros_like(h) for _ in range(world)]
    dist.all_gather(hs, h)
    same = all(int(x) == int(h) for x in hs)
    # the benchmark's reduction: time = max over ranks, units = sum over ranks
    t = torch.tensor([float(sum(lengths[i] for i in mine))], dtype=torch.float64)
    units = t.clone()
    dist.barrier()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(units, op=dist.ReduceOp.SUM)
    if rank == 0:
        out.put((same, float(t), float(units), [len(p) for p in plan]))
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_plan():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    lengths = np.random.default_rng(1).integers(120, 801, 16).tolist()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, lengths, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, tmax, units, counts = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same and sum(counts) == 16
    assert units == float(sum(lengths))
    assert tmax == float(max(sharding.loads(lengths, sharding.assign(lengths, 2))))


# ---- time sharding of one utterance: the partition keeps the 128-column chunk grid, so the chunk statistics two ranks
# compute over their own columns are, gathered, exactly the unsharded statistics row, and the AdaIN affine computed from
# the gathered row equals the single-device one bit for bit.

def _stats_worker(rank, world, port, t, out):
    from lokinfer_b200.timeshard import Partition
    from oracle import kokoro_oracle as O

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    part = Partition(t, world)
    g = torch.Generator().manual_seed(5)
    ok = True
    for stage, c in ((0, 8), (1, 4)):
        length = (part.l0, part.l1)[stage]
        x = torch.randn(c, length, generator=g) * 3 + 1  # the same tensor on both ranks (same seed)
        gb = torch.randn(2 * c, generator=g)
        lo, hi = part.rng(stage, rank)
        mine = O.channel_stats(x[:, lo:hi].contiguous())
        total = O.stat_chunks(length)
        sizes = [O.stat_chunks(part.rng(stage, r)[1] - part.rng(stage, r)[0]) for r in range(world)]
        pad = max(sizes)
        buf = torch.zeros(c, pad, 2)
        buf[:, : mine.shape[1]] = mine
        every = [torch.zeros_like(buf) for _ in range(world)]
        dist.all_gather(every, buf)
        row = torch.cat([e[:, :n] for e, n in zip(every, sizes)], dim=1)
        whole = O.channel_stats(x)
        ok = ok and row.shape[1] == total and torch.equal(row, whole)
        ok = ok and torch.equal(O.adain_affine(row, gb, length), O.adain_affine(whole, gb, length))
    if rank == 0:
        out.put(ok)
    dist.destroy_process_group()


def test_two_gloo_ranks_merge_chunk_statistics_exactly():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_stats_worker, args=(r, 2, port, 200, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok


def test_time_shard_partition_covers_the_utterance():
    from lokinfer_b200.timeshard import MARGIN, Partition
    for t, world in ((2080, 8), (2080, 4), (2080, 2), (320, 2), (797, 4), (128, 2)):
        p = Partition(t, world)
        assert p.bx[0] == 0 and p.bx[-1] == t and sorted(p.bx) == p.bx
        assert p.b0[-1] == 10 * t and p.b1[-1] == 60 * t + 1 and p.bs[-1] == 300 * t
        for k in range(1, world):
            assert p.bx[k] % 64 == 0 and p.b0[k] % 128 == 0 and p.b1[k] % 128 == 0
            assert p.b1[k] == 6 * p.b0[k] and p.bs[k] == 5 * p.b1[k]
        assert min(y - x for x, y in zip(p.b0, p.b0[1:])) >= MARGIN
