"""Whole-path parity: one AdaINResBlock1, the full generator (fused and basic graphs) against the CPU oracle and the
committed golden fixture, CUDA-graph replay, and size-independent properties at the full 26 s size."""
import numpy as np
import pytest
import torch

from lokinfer_b200 import synth
from oracle import kokoro_oracle as O
from util import REL_L2, WAVE_MAXABS, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gen(cuda):
    from lokinfer_b200 import Generator
    return Generator(synth.generator_weights(0), cuda)


def _inputs(cuda, t, seed=1):
    from lokinfer_b200 import ops
    inp = synth.generator_inputs(t, seed)
    return inp, [ops.to_cuda(inp[k], cuda) for k in ("x", "har", "s")]


@pytest.mark.parametrize("c,l,k", [(16, 300, 7), (128, 1201, 3), (128, 2000, 11), (256, 640, 7)])
def test_resblock(cuda, c, l, k):
    """Config 0 at reduced length: one AdaINResBlock1 (kernel k, dilations 1/3/5) through the fused ops."""
    from lokinfer_b200 import Generator, ops
    sd, x, s = synth.resblock_case(c, l, k, 100 + c + k)
    g = Generator(sd, cuda)
    out, st = g.adain_resblock1_fused(ops.to_cuda(x, cuda), g.style(ops.to_cuda(s, cuda)), "rb", k)
    sd32 = {n: O.T(v) for n, v in sd.items()}
    ref, rst = O.adain_resblock1_fused(O.T(x), O.style_bank(sd32, O.T(s)), sd32, "rb", k)
    sd64 = {n: O.T(v, torch.float64) for n, v in sd.items()}
    ref64, _ = O.adain_resblock1_fused(O.T(x, torch.float64), O.style_bank(sd64, O.T(s, torch.float64)), sd64, "rb", k)
    got = out.cpu().numpy()
    # six chained convs: the per-op bar compounds; the float64 golden is the arbiter
    assert rel_l2(got, ref.numpy()) <= 6 * REL_L2
    assert rel_l2(got, ref64.numpy()) <= 2 * rel_l2(ref.numpy(), ref64.numpy()) + 1e-6
    np.testing.assert_allclose(st.cpu().numpy()[..., 0], rst.numpy()[..., 0], atol=1e-4, rtol=1e-4)


def test_generator_golden(cuda, gen):
    from pathlib import Path
    gold = np.load(Path(__file__).resolve().parent / "golden" / "kokoro_golden.npz")
    _, d = _inputs(cuda, 4)
    post, audio = gen.forward(*d, outputs=("post", "audio"))
    assert tuple(audio.shape) == (1200,) and tuple(post.shape) == (22, 241)
    assert np.abs(audio.cpu().numpy() - gold["gen_audio_f32"]).max() <= WAVE_MAXABS
    assert np.abs(audio.cpu().numpy() - gold["gen_audio_f64"]).max() <= WAVE_MAXABS
    assert rel_l2(post.cpu().numpy(), gold["gen_post_f64"]) <= 1e-4


@pytest.mark.parametrize("t", [1, 7, 16])
@pytest.mark.parametrize("fused", [True, False])
def test_generator_vs_oracle(cuda, gen, t, fused):
    inp, d = _inputs(cuda, t, seed=3 + t)
    audio = gen.forward(*d, fused=fused).cpu().numpy()
    sd = synth.generator_weights(0)
    ref32 = O.generator(sd, O.T(inp["x"]), O.T(inp["har"]), O.T(inp["s"]), fused=fused).numpy()
    dt = torch.float64
    ref64 = O.generator(sd, O.T(inp["x"], dt), O.T(inp["har"], dt), O.T(inp["s"], dt), fused=fused).numpy()
    sh = synth.shapes(t)
    assert audio.shape == (sh["S"],) == ref32.shape
    assert np.abs(audio - ref32).max() <= WAVE_MAXABS
    assert np.abs(audio - ref64).max() <= WAVE_MAXABS


def _oracle_stages(inp, dt, fused=True):
    sd = synth.generator_weights(0)
    return O.generator(sd, O.T(inp["x"], dt), O.T(inp["har"], dt), O.T(inp["s"], dt), fused=fused, stages=True)


@pytest.mark.parametrize("t", [320, 333, 797])
def test_generator_baseline_configs_vs_oracle(cuda, gen, t):
    """BASELINE config 1 (the 4 s sentence case, T = 320) and two utterance lengths of config 3 (T in 120..800, one
    odd: odd T makes every row pitch of stage 0 odd as well) against the CPU oracle in float32 and float64:
    the eager forward with concurrent streams, the same forward on one stream, and the captured-graph path with
    host buffers (Generator.synthesize). Bars: waveform max-abs <= 1e-4, conv_post logits rel-L2, and the GPU's
    error against float64 within 2x the float32 oracle's own."""
    inp, d = _inputs(cuda, t, seed=40 + t)
    post, audio = gen.forward(*d, outputs=("post", "audio"))
    audio_1s = gen.forward(*d, concurrent=False)
    host = [torch.from_numpy(inp[k]).pin_memory() for k in ("x", "har", "s")]
    audio_graph = gen.synthesize(*host).numpy().copy()
    sh = synth.shapes(t)
    assert tuple(audio.shape) == (sh["S"],) and tuple(post.shape) == (22, sh["L1"])
    r32, r64 = _oracle_stages(inp, torch.float32), _oracle_stages(inp, torch.float64)
    a32, a64 = r32["audio"].numpy(), r64["audio"].numpy()
    got = audio.cpu().numpy()
    assert np.abs(got - a32).max() <= WAVE_MAXABS
    assert np.abs(got - a64).max() <= WAVE_MAXABS
    np.testing.assert_array_equal(audio_1s.cpu().numpy(), got)
    np.testing.assert_array_equal(audio_graph, got)
    p = post.cpu().numpy()
    e_gpu, e_cpu = rel_l2(p, r64["post"].numpy()), rel_l2(r32["post"].numpy(), r64["post"].numpy())
    assert rel_l2(p, r32["post"].numpy()) <= 48 * REL_L2  # 48 chained fused convs
    assert e_gpu <= 2 * e_cpu + 1e-6
    assert rel_l2(got, a64) <= 2 * rel_l2(a32, a64) + 1e-6
    from lokinfer_b200 import ops
    assert ops.conv_tc_status() == 0


@pytest.mark.parametrize("k", [3, 7, 11])
@pytest.mark.parametrize("l", [19200, 19201])
def test_resblock_config0_full_length(cuda, k, l):
    """BASELINE config 0 at its full length: one AdaINResBlock1 at C = 128, L = 19200 (and 19201, the generator's
    real stage-1 length for T = 320) for each kernel size, against the float32 and float64 oracle."""
    from lokinfer_b200 import Generator, ops
    sd, x, s = synth.resblock_case(128, l, k, 300 + k)
    g = Generator(sd, cuda)
    with ops.padded_rows():
        out, st = g.adain_resblock1_fused(ops.to_cuda(x, cuda, rows=True), g.style(ops.to_cuda(s, cuda)), "rb", k)
    plain, st_plain = g.adain_resblock1_fused(ops.to_cuda(x, cuda), g.style(ops.to_cuda(s, cuda)), "rb", k)
    assert torch.equal(out, plain) and torch.equal(st, st_plain)  # padded rows (TMA) and contiguous rows agree
    sd32 = {n: O.T(v) for n, v in sd.items()}
    ref, rst = O.adain_resblock1_fused(O.T(x), O.style_bank(sd32, O.T(s)), sd32, "rb", k)
    sd64 = {n: O.T(v, torch.float64) for n, v in sd.items()}
    ref64, _ = O.adain_resblock1_fused(O.T(x, torch.float64), O.style_bank(sd64, O.T(s, torch.float64)), sd64, "rb", k)
    got = out.cpu().numpy()
    assert got.shape == (128, l)
    assert rel_l2(got, ref.numpy()) <= 6 * REL_L2
    assert rel_l2(got, ref64.numpy()) <= 2 * rel_l2(ref.numpy(), ref64.numpy()) + 1e-6
    np.testing.assert_allclose(st.cpu().numpy()[..., 0], rst.numpy()[..., 0], atol=1e-4, rtol=1e-4)
    assert ops.conv_tc_status() == 0


def test_generator_config2_stages_vs_oracle(cuda, gen):
    """BASELINE config 2 (the 26 s paragraph case, T = 2080) against the float32 oracle run once on the CPU: the
    three resblock outputs of each stage, the conv_post logits and the waveform."""
    t = 2080
    inp, d = _inputs(cuda, t, seed=5)
    post, audio, s0, s1 = gen.forward(*d, outputs=("post", "audio", "stage0", "stage1"))
    ref = _oracle_stages(inp, torch.float32)
    for name, got_rb in (("stage0", s0), ("stage1", s1)):
        for j in range(3):
            assert rel_l2(got_rb[j].cpu().numpy(), ref[name][j].numpy()) <= 24 * REL_L2, (name, j)
    assert rel_l2(post.cpu().numpy(), ref["post"].numpy()) <= 48 * REL_L2
    assert np.abs(audio.cpu().numpy() - ref["audio"].numpy()).max() <= WAVE_MAXABS
    from lokinfer_b200 import ops
    assert ops.conv_tc_status() == 0


def test_graph_replay_matches_eager(cuda, gen):
    inp, d = _inputs(cuda, 9, seed=21)
    eager = gen.forward(*d).cpu().numpy()
    host = [torch.from_numpy(inp[k]).pin_memory() for k in ("x", "har", "s")]
    a1 = gen.synthesize(*host).numpy().copy()
    a2 = gen.synthesize(*host).numpy().copy()
    np.testing.assert_array_equal(a1, eager)
    np.testing.assert_array_equal(a1, a2)


def test_planned_arena(cuda):
    """The captured forward lives in a planned arena: identical samples to the eager forward (every intermediate its
    own allocation) and to a capture without the plan, in well under the memory of keeping every intermediate."""
    from lokinfer_b200 import Generator, ops
    t = 416
    inp = synth.generator_inputs(t, 9)
    g1, g2 = Generator(synth.generator_weights(0), cuda), Generator(synth.generator_weights(0), cuda)
    d = [ops.to_cuda(inp[k], cuda) for k in ("x", "har", "s")]
    eager = g1.forward(*d)
    b1, b2 = g1.capture(t), g2.capture(t, planned=False)
    assert "arena" in b1 and "arena" not in b2
    assert b1["arena_bytes"] <= 0.55 * b1["unplanned_bytes"]
    for b in (b1, b2):
        for k, v in zip(("x", "har", "s"), d):
            b[k].copy_(v)
        for _ in range(3):
            b["graph"].replay()
    torch.cuda.synchronize()
    assert torch.equal(b1["audio"], eager) and torch.equal(b2["audio"], eager)
    assert ops.conv_tc_status() == 0


def test_many_captures_keep_their_plans_valid(cuda):
    """One generator captures more lengths than torch's stream pool has streams (32): a stream made for a later
    capture can be the same CUDA stream as one of the generator's side streams. The memory plan must still be made
    for the concurrency the captured graph really has: every replay equals the eager forward."""
    from lokinfer_b200 import Generator, ops
    g = Generator(synth.generator_weights(0), cuda)
    lengths = list(range(40, 40 + 36))
    worst = 0.0
    for i, t in enumerate(lengths):
        inp = synth.generator_inputs(t, 500 + i)
        d = [ops.to_cuda(inp[k], cuda) for k in ("x", "har", "s")]
        eager = g.forward(*d)
        b = g.capture(t)
        for k, v in zip(("x", "har", "s"), d):
            b[k].copy_(v)
        for _ in range(2):
            b["graph"].replay()
        torch.cuda.synchronize()
        assert torch.equal(b["audio"], eager), (i, t)
        worst = max(worst, eager.abs().max().item())
    assert ops.conv_tc_status() == 0 and worst > 0


def test_full_size_properties(cuda, gen):
    """The 26 s case (T = 2080: L0 = 20800, L1 = 124801, 624000 samples), too large for the CPU oracle in a test:
    exact shapes, run-to-run determinism, agreement of the fused graph with the basic-kernel graph (two independent
    kernel sets), and the iSTFT tail against torch.istft on the same logits."""
    t = 2080
    sh = synth.shapes(t)
    _, d = _inputs(cuda, t, seed=5)
    post, audio = gen.forward(*d, outputs=("post", "audio"))
    assert tuple(post.shape) == (22, sh["L1"]) == (22, 124801) and tuple(audio.shape) == (624000,)
    audio2 = gen.forward(*d)
    assert torch.equal(audio, audio2)
    assert torch.isfinite(audio).all()
    basic = gen.forward(*d, fused=False)
    assert (audio - basic).abs().max().item() <= 2 * WAVE_MAXABS
    ref = O.istft_logits_torch(post)  # torch's own CUDA iSTFT
    assert (audio - ref).abs().max().item() <= 1e-5 * ref.abs().max().item()
    from lokinfer_b200 import ops
    assert ops.conv_tc_status() == 0
    # the tensor-core and CUDA-core conv kernels give the same waveform
    ops.set_conv_path("simt")
    try:
        simt = gen.forward(*d)
    finally:
        ops.set_conv_path("auto")
    assert (audio - simt).abs().max().item() <= WAVE_MAXABS


def test_synthesis_pipeline_matches_synthesize(cuda, gen):
    """Generator.pipeline (two utterances in flight, copies overlapping compute) returns, for every utterance of a
    stream of different inputs, exactly what Generator.synthesize returns for it alone."""
    t = 200
    hosts, want = [], []
    for i in range(5):
        inp, _ = _inputs(cuda, t, seed=70 + i)
        h = [torch.from_numpy(inp[k]).pin_memory() for k in ("x", "har", "s")]
        hosts.append(h)
        want.append(gen.synthesize(*h).numpy().copy())
    pipe = gen.pipeline(t, depth=2)
    outs = [torch.empty(want[0].shape, dtype=torch.float32).pin_memory() for _ in hosts]
    tickets = [pipe.submit(*h, o) for h, o in zip(hosts, outs)]
    for k in tickets:
        pipe.wait(k)
    for o, w in zip(outs, want):
        np.testing.assert_array_equal(o.numpy(), w)
    assert not np.array_equal(want[0], want[1])
