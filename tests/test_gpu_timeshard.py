"""Time sharding of one utterance (BASELINE config 2's multi-GPU scheme) on ONE GPU: every rank of the partition runs
in this process, in lock-step (all ranks push before any rank waits), with the other ranks' memory reached through
the same peer-pointer arithmetic the multi-process fabric uses. Checks the partition, the halo and statistics
exchange and the windowed kernels against the unsharded forward and the CPU oracle, and that a wait whose flag never
arrives runs out, reports it in the status word and leaves the context usable."""
import numpy as np
import pytest
import torch

from lokinfer_b200 import synth
from oracle import kokoro_oracle as O
from util import WAVE_MAXABS

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gen(cuda):
    from lokinfer_b200 import Generator
    return Generator(synth.generator_weights(0), cuda)


def _ranks(gen, cuda, t, world, limit_ns=200_000_000):
    from lokinfer_b200 import timeshard as ts
    fabric = ts.LocalFabric(world, ts.TimeShardedGenerator.arena_bytes(t, world), cuda)
    return fabric, [ts.TimeShardedGenerator(gen, t, r, world, fabric, wait_limit_ns=limit_ns) for r in range(world)]


@pytest.mark.parametrize("t,world", [(320, 2), (333, 3), (520, 4), (512, 8)])
def test_time_sharded_forward_equals_single_gpu(cuda, gen, t, world):
    from lokinfer_b200 import ops, timeshard as ts
    inp = synth.generator_inputs(t, 70 + t)
    x, har, s = [ops.to_cuda(inp[k], cuda) for k in ("x", "har", "s")]
    single = gen.forward(x, har, s)
    fabric, ranks = _ranks(gen, cuda, t, world)
    try:
        for _ in range(2):  # the second forward runs on the next epoch with the same buffers
            audio = ts.forward_lockstep(ranks, x, har, s)
            assert tuple(audio.shape) == tuple(single.shape)
            assert all(r.status() == 0 for r in ranks) and ops.conv_tc_status() == 0
            assert (audio - single).abs().max().item() <= 1e-6
        if t == 320:
            sd = synth.generator_weights(0)
            ref = O.generator(sd, O.T(inp["x"]), O.T(inp["har"]), O.T(inp["s"]), fused=True).numpy()
            assert np.abs(audio.cpu().numpy() - ref).max() <= WAVE_MAXABS
        # the chunk statistics every rank holds are the unsharded ones: compare rank 0's copy of the last stage-1
        # statistics row it produced with channel_stats of the gathered conv_post input
        posts = torch.cat([r.post.own for r in ranks], dim=1)
        _, post_single = gen.forward(x, har, s, outputs=("audio", "post"))
        assert (posts - post_single).abs().max().item() <= 1e-5 * post_single.abs().max().item()
    finally:
        for a in fabric.arenas:
            a.close()


def test_partition_boundaries():
    from lokinfer_b200.timeshard import Partition
    for t, world in ((2080, 8), (2080, 2), (320, 2), (797, 4)):
        p = Partition(t, world)
        assert p.bx[0] == 0 and p.bx[-1] == t and p.b1[-1] == 60 * t + 1 and p.bs[-1] == 300 * t
        for k in range(1, world):
            assert p.b0[k] % 128 == 0 and p.b1[k] % 128 == 0 and p.b1[k] == 6 * p.b0[k] and p.bs[k] == 5 * p.b1[k]
    with pytest.raises(ValueError):
        Partition(100, 4)


def test_wait_runs_out_and_reports(cuda, gen):
    """Only rank 0 of two runs: the flags its waits need are never set. With a limit of 1 ms every wait gives up,
    records 1 << 24 | flag index in the status word and returns; the forward finishes (on stale halos), nothing hangs,
    and the device keeps working."""
    from lokinfer_b200 import ops, timeshard as ts
    t = 320
    inp = synth.generator_inputs(t, 3)
    x, har, s = [ops.to_cuda(inp[k], cuda) for k in ("x", "har", "s")]
    fabric, ranks = _ranks(gen, cuda, t, 2, limit_ns=1_000_000)
    try:
        audio = ranks[0].forward(x, har, s)
        st = ranks[0].status()
        assert st & (1 << 24)
        assert ranks[0].status() == 0  # cleared
        assert tuple(audio.shape) == (300 * ranks[0].part.bx[1],)
        assert torch.isfinite(gen.forward(x, har, s)).all()
        ops.conv_tc_status()
    finally:
        for a in fabric.arenas:
            a.close()
