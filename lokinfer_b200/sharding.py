"""Utterance sharding across the GPUs of one box: one process per GPU, independent utterances, no data-path
collective. Every utterance's AdaIN statistics are its own (instance norm over its own time axis), so ranks never
exchange activations; the only cross-rank step is the timing reduction in the benchmark.

assign() is longest-processing-time-first on the generator input length T (work is proportional to T)."""
from __future__ import annotations

import heapq


def assign(lengths, world_size: int) -> list[list[int]]:
    """Indices of `lengths` per rank: each utterance (longest first, ties by index) goes to the least-loaded rank
    (ties by rank). Deterministic, so every rank computes the same plan without communication."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    heap = [(0, r) for r in range(world_size)]
    plan = [[] for _ in range(world_size)]
    for i in order:
        load, r = heapq.heappop(heap)
        plan[r].append(i)
        heapq.heappush(heap, (load + int(lengths[i]), r))
    return plan


def loads(lengths, plan) -> list[int]:
    return [sum(int(lengths[i]) for i in idx) for idx in plan]


def audio_seconds(lengths, sample_rate: int = 24000) -> float:
    """Seconds of audio a set of utterances produces: 300 samples per unit of T at 24 kHz
    (kernels/cpu/kokoro_signal.cpp:19-20)."""
    return sum(300 * int(t) for t in lengths) / float(sample_rate)
