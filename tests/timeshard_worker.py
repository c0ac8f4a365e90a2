"""One rank of the multi-process time-sharding test (launched by test_gpu_timeshard_multi.py through
torch.distributed.run, one process per GPU): sharded forward over CUDA IPC peer memory, eager and from a captured
graph, compared with the unsharded forward of the same inputs on the same GPU. Prints one line per rank."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from lokinfer_b200 import Generator, ops, synth, timeshard as ts  # noqa: E402


def main():
    t = int(sys.argv[1]) if len(sys.argv) > 1 else 320
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device(f"cuda:{int(os.environ['LOCAL_RANK'])}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    gen = Generator(synth.generator_weights(0), dev)
    inp = synth.generator_inputs(t, 11)
    x, har, s = [ops.to_cuda(inp[k], dev) for k in ("x", "har", "s")]
    single = gen.forward(x, har, s)
    fabric = ts.IpcFabric(ts.TimeShardedGenerator.arena_bytes(t, world), dev)
    tsg = ts.TimeShardedGenerator(gen, t, rank, world, fabric)
    lo, hi = tsg.part.bs[rank], tsg.part.bs[rank + 1]
    dist.barrier()
    errs = []
    for _ in range(2):
        audio = tsg.forward(x, har, s)
        errs.append((audio - single[lo:hi]).abs().max().item())
    dist.barrier()
    graph = tsg.capture(x, har, s)
    dist.barrier()
    for _ in range(3):
        graph.replay()
    errs.append((tsg.audio - single[lo:hi]).abs().max().item())
    status = tsg.status()
    ok = max(errs) <= 1e-6 and status == 0 and ops.conv_tc_status() == 0
    print(f"rank {rank}/{world} T={t} samples [{lo}, {hi}) max|sharded - single| {max(errs):.3e} status {status} "
          f"{'OK' if ok else 'FAIL'}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
