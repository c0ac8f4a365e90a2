"""The memory planner of the activation arena (lokinfer_b200/arena.py) on synthetic traces: a block is reused only when
every use of its previous tenant happens-before the new allocation (vector clocks over streams and joins), never on
program order alone."""
from lokinfer_b200.arena import ALIGN, Tracer, happens_before, plan


class _T:
    """Stands in for a tensor: the tracer only needs a storage pointer, a size and a shape."""
    n = 0

    def __init__(self, nbytes):
        _T.n += 1
        self._p, self._b, self.shape = 0x1000 * _T.n, nbytes, (nbytes // 4,)

    def untyped_storage(self):
        return self

    def data_ptr(self):
        return self._p

    def nbytes(self):
        return self._b


def test_happens_before():
    assert happens_before([(1, 3)], {1: 3})
    assert not happens_before([(1, 4)], {1: 3})
    assert not happens_before([(1, 1), (2, 1)], {1: 5})
    assert happens_before([], {})


def test_same_stream_chain_reuses_memory():
    tr = Tracer()
    a, b, c, d = (_T(1024) for _ in range(4))
    tr.on_alloc(a, 1); tr.on_run([a], 1)          # a = f()
    tr.on_alloc(b, 1); tr.on_run([a, b], 1)       # b = g(a): last use of a
    tr.on_alloc(c, 1); tr.on_run([b, c], 1)       # c = h(b): a is dead -> c may take a's place
    tr.on_alloc(d, 1); tr.on_run([c, d], 1)       # d = k(c): b is dead
    off, total = plan(tr.allocs)
    assert off[0] == 0 and off[1] == 1024 and off[2] == 0 and off[3] == 1024 and total == 2048


def test_concurrent_streams_do_not_share_until_joined():
    tr = Tracer()
    x, p, q, r, y = (_T(4096) for _ in range(5))
    tr.on_alloc(x, 1); tr.on_run([x], 1)          # stream 1 produces x
    tr.on_join(2, 1)                              # stream 2 forks from stream 1
    tr.on_alloc(p, 2); tr.on_run([x, p], 2)       # branch on stream 2: p = f(x)
    tr.on_alloc(q, 1); tr.on_run([x, q], 1)       # branch on stream 1: q = g(x), last use of x in program order
    tr.on_alloc(r, 1); tr.on_run([q, r], 1)       # r = h(q): x looks dead, but stream 2 may still be reading it
    off, _ = plan(tr.allocs)
    assert off[3] not in (off[0],)                # r does not take x's block (no join of stream 2 yet)
    assert len({off[0], off[1], off[2], off[3]}) == 4
    tr.on_join(1, 2)                              # stream 1 waits for stream 2
    tr.on_alloc(y, 1); tr.on_run([r, p, y], 1)
    off, _ = plan(tr.allocs)
    assert off[4] == off[0]                       # after the join x's block is free for y


def test_pinned_tensors_are_never_reused_and_sizes_are_aligned():
    tr = Tracer()
    a, b, c = _T(100), _T(100), _T(100)
    tr.on_alloc(a, 1); tr.on_run([a], 1)
    tr.pin(a)
    tr.on_alloc(b, 1); tr.on_run([b], 1)
    tr.on_alloc(c, 1); tr.on_run([c], 1)
    off, total = plan(tr.allocs)
    assert off[0] == 0 and off[1] == ALIGN and off[2] == ALIGN and total == 2 * ALIGN


def _plan_python(allocs):
    """The planner restated in Python (greedy lowest offset, happens-before by vector clocks): the check of the
    library's lkc_plan_memory on random traces."""
    placed, offsets, top = [], [], 0
    for a in allocs:
        size = -(-a["bytes"] // ALIGN) * ALIGN
        busy = sorted((o, e) for o, e, p in placed
                      if p["pinned"] or not happens_before(p["uses"] + [(p["stream"], p["clock"][p["stream"]])],
                                                           a["clock"]))
        off = 0
        for o, e in busy:
            if off + size <= o:
                break
            if e > off:
                off = e
        offsets.append(off)
        placed.append((off, off + size, a))
        top = max(top, off + size)
    return offsets, top


def test_native_planner_matches_the_python_restatement_on_random_traces():
    import random
    rng = random.Random(7)
    for trial in range(30):
        tr = Tracer()
        live = []
        streams = [1, 2, 3, 4][: rng.randint(1, 4)]
        for step in range(rng.randint(5, 60)):
            s = rng.choice(streams)
            kind = rng.random()
            if kind < 0.15 and len(streams) > 1:
                w = rng.choice([x for x in streams if x != s])
                tr.on_join(s, w)
                continue
            t = _T(rng.choice([4, 100, 256, 1000, 4096, 70000]))
            tr.on_alloc(t, s)
            ins = rng.sample(live, min(len(live), rng.randint(0, 3)))
            tr.on_run(ins + [t], s)
            live.append(t)
            if rng.random() < 0.1:
                tr.pin(t)
        assert plan(tr.allocs) == _plan_python(tr.allocs)
    assert plan([]) == ([], 0)
