"""Parity of every CUDA op (called through the C-ABI via lokinfer_b200.ops) against the CPU oracle on the same seeded
inputs. Bars: rel-L2 <= 1e-5 per op against the float32 oracle; the reference's own float64 tolerances
(tests/kernels/test_kokoro_conv_fused.py:1-7) against the float64 oracle; integer shape logic exact."""
import math

import numpy as np
import pytest
import torch

from lokinfer_b200 import synth
from oracle import kokoro_oracle as O
from util import REL_L2, check_stats, rel_l2, t32, t64

pytestmark = pytest.mark.gpu

GOLD = None


def gold():
    global GOLD
    if GOLD is None:
        from pathlib import Path
        GOLD = np.load(Path(__file__).resolve().parent / "golden" / "kokoro_golden.npz")
    return GOLD


def dev(cuda, *arrs):
    from lokinfer_b200 import ops
    return [ops.to_cuda(a, cuda) for a in arrs]


# (Ci, Co, L, K, dilation): the reference's cases (test_kokoro_conv_fused.py:44-51) + K*d > L, exact chunk multiples,
# Kokoro stage shapes at reduced length.
CONV_CASES = [(8, 8, 50, 3, 1), (16, 12, 700, 7, 3), (12, 16, 97, 11, 5), (128, 128, 5000, 11, 5),
              (64, 64, 3000, 3, 1), (8, 8, 1, 3, 1), (8, 8, 20, 11, 5), (32, 32, 256, 7, 1), (32, 32, 257, 7, 1),
              (128, 128, 1201, 3, 1), (128, 128, 1201, 7, 3), (256, 256, 640, 11, 5), (256, 256, 333, 3, 5),
              (128, 22, 961, 7, 1), (22, 128, 961, 1, 1)]


# Shapes the tensor-core kernel takes (Ci % 16 == 0; Co is padded to a multiple of 128 inside the pack): every Kokoro (C, K, dilation) plus tile edges:
# one partial tile, exact tile / chunk multiples, one column past a tile, many tiles per CTA, L < halo.
TC_CASES = [(128, 128, 1201, 3, 1), (128, 128, 1201, 7, 3), (128, 128, 5000, 11, 5), (256, 256, 640, 11, 5),
            (256, 256, 333, 3, 5), (128, 128, 256, 3, 1), (128, 128, 257, 7, 1), (128, 128, 128, 11, 1),
            (128, 128, 20, 11, 5), (128, 128, 1, 3, 1), (16, 128, 700, 7, 3), (48, 128, 300, 5, 2),
            (256, 128, 900, 3, 3), (128, 256, 900, 7, 5), (128, 128, 45000, 3, 1), (256, 256, 20800, 7, 1),
            (128, 128, 19201, 11, 3), (128, 22, 5000, 7, 1), (32, 200, 700, 3, 1), (16, 129, 300, 5, 1),
            # K beyond the 12-MMA drain bound: one chunk's 13 hi MMAs form the chain (tensor cores); K = 25 has more
            # than the kernel accepts and runs on the CUDA cores although it has a state
            (32, 128, 400, 13, 1), (32, 128, 300, 25, 2)]


@pytest.mark.parametrize("ci,co,l,k,d", CONV_CASES + TC_CASES)
@pytest.mark.parametrize("variant", ["snake", "snake_res", "leaky", "leaky_res", "affine"])
def test_conv1d_fused(cuda, ci, co, l, k, d, variant):
    """Both kernels behind the fused-conv entry points: with a prepared state eligible shapes run on tcgen05, the
    rest (and every shape without a state) on the CUDA-core kernel; each is held to the same bars."""
    from lokinfer_b200 import ops
    if (ci, co, l, k, d) in TC_CASES and l > 6000 and variant not in ("snake", "snake_res"):
        pytest.skip("large shapes: snake variants only (CPU oracle time)")
    x, w, b, affine, alpha, res = synth.conv_case(ci, co, l, k, ci * 31 + l + k)
    pad = d * (k - 1) // 2
    lo = l + 2 * pad - d * (k - 1)
    res = res[:, :lo]
    dx, dw, db, daf, dal, dres = dev(cuda, x, w, b, affine, alpha, np.ascontiguousarray(res))
    state = ops.conv1d_prepare_f32_cuda(dw)
    assert (state is not None) == (ci % 16 == 0)
    kw = dict(padding=pad, dilation=d, state=state)

    okw = dict(padding=pad, dilation=d)

    def oracle(dt):
        a = [O.T(v, dt) for v in (x, w, b, affine, alpha, res)]
        if variant.startswith("snake"):
            return O.conv1d_fused(a[0], a[1], a[2], a[3], "snake", alpha=a[4],
                                  residual=a[5] if variant == "snake_res" else None, **okw)
        if variant.startswith("leaky"):
            rk = dict(residual=a[5], out_scale=0.7071067811865476) if variant == "leaky_res" else {}
            return O.conv1d_fused(a[0], a[1], a[2], a[3], "leaky", slope=0.2, **okw, **rk)
        return O.conv1d_fused(a[0], a[1], a[2], a[3], "none", **okw)

    if variant.startswith("snake"):
        out, stats = ops.conv1d_snake_f32_cuda(dx, dw, db, daf, dal, residual=dres if variant == "snake_res" else None,
                                               **kw)
    elif variant.startswith("leaky"):
        rk = dict(residual=dres, out_scale=0.7071067811865476) if variant == "leaky_res" else {}
        out, stats = ops.conv1d_leaky_f32_cuda(dx, dw, db, daf, slope=0.2, **kw, **rk)
    else:
        out, stats = ops.conv1d_affine_f32_cuda(dx, dw, db, daf, **kw)
    out, stats = out.cpu().numpy(), stats.cpu().numpy()
    ref32, st32 = oracle(torch.float32)
    ref64, _ = oracle(torch.float64)
    assert out.shape == tuple(ref32.shape) == (co, lo) and stats.shape == tuple(st32.shape)
    assert rel_l2(out, ref32.numpy()) <= REL_L2
    np.testing.assert_allclose(out, ref64.numpy(), atol=1e-4, rtol=1e-4)
    # f32 error against the float64 golden stays within 2x the f32 oracle's own error (+ a floor of one ulp-scale)
    e_gpu, e_cpu = rel_l2(out, ref64.numpy()), rel_l2(ref32.numpy(), ref64.numpy())
    assert e_gpu <= 2 * e_cpu + 2e-7
    check_stats(stats, out)
    np.testing.assert_allclose(stats[..., 0], st32.numpy()[..., 0], atol=2e-5, rtol=2e-5)
    assert ops.conv_tc_status() == 0
    if state is not None:  # the CUDA-core kernel on the same operands agrees with the tensor-core one
        ops.set_conv_path("simt")
        try:
            if variant.startswith("snake"):
                o2, s2 = ops.conv1d_snake_f32_cuda(dx, dw, db, daf, dal,
                                                   residual=dres if variant == "snake_res" else None, **kw)
            elif variant.startswith("leaky"):
                rk = dict(residual=dres, out_scale=0.7071067811865476) if variant == "leaky_res" else {}
                o2, s2 = ops.conv1d_leaky_f32_cuda(dx, dw, db, daf, slope=0.2, **kw, **rk)
            else:
                o2, s2 = ops.conv1d_affine_f32_cuda(dx, dw, db, daf, **kw)
        finally:
            ops.set_conv_path("auto")
        assert rel_l2(out, o2.cpu().numpy()) <= REL_L2


# Shapes for the padded-row (TMA) route: partial last tile, exact tile multiples, windows that start before the row
# and end after it, odd lengths (pitch = L rounded up to 4), both stage shapes of the 26 s case, several tiles per CTA.
TMA_CASES = [(128, 128, 1201, 3, 1), (128, 128, 1203, 7, 3), (128, 128, 5000, 11, 5), (256, 256, 641, 11, 5),
             (128, 128, 256, 3, 1), (128, 128, 257, 7, 1), (128, 128, 20, 11, 5), (128, 128, 1, 3, 1),
             (16, 128, 702, 7, 3), (256, 128, 900, 3, 3), (128, 256, 901, 7, 5), (128, 128, 45001, 3, 1),
             (256, 256, 20800, 7, 1), (128, 128, 124801, 11, 5), (128, 22, 5001, 7, 1), (32, 128, 400, 13, 1)]


@pytest.mark.parametrize("ci,co,l,k,d", TMA_CASES)
@pytest.mark.parametrize("variant", ["snake", "snake_res", "leaky_res"])
def test_conv1d_fused_padded_rows(cuda, ci, co, l, k, d, variant):
    """The same op on [C, L] views whose rows are padded to 16 bytes: the tensor-core kernel then loads the raw
    windows and the residual and stores the output with the TMA unit. The arithmetic does not depend on the route:
    results are bit-identical to the contiguous call (4-byte accesses), which the other tests hold to the oracle;
    small cases are also compared with the oracle directly, and the padding columns stay untouched."""
    from lokinfer_b200 import ops
    x, w, b, affine, alpha, res = synth.conv_case(ci, co, l, k, ci * 31 + l + k, big=l < 6000)
    pad = d * (k - 1) // 2
    dx, dw, db, daf, dal, dres = dev(cuda, x, w, b, affine, alpha, res)
    state = ops.conv1d_prepare_f32_cuda(dw)
    assert state is not None

    def call(xx, rr):
        kw = dict(padding=pad, dilation=d, state=state)
        if variant == "snake":
            return ops.conv1d_snake_f32_cuda(xx, dw, db, daf, dal, **kw)
        if variant == "snake_res":
            return ops.conv1d_snake_f32_cuda(xx, dw, db, daf, dal, residual=rr, **kw)
        return ops.conv1d_leaky_f32_cuda(xx, dw, db, daf, slope=0.2, residual=rr, out_scale=0.7071067811865476, **kw)

    ref_out, ref_stats = call(dx, dres)
    with ops.padded_rows():
        px, pres = ops.to_cuda(x, cuda, rows=True), ops.to_cuda(res, cuda, rows=True)
        pitch = -(-l // 4) * 4
        assert px.stride(0) == pitch and pres.stride(0) == pitch
        out, stats = call(px, pres)
    assert out.stride(0) == pitch and tuple(out.shape) == (co, l)
    assert ops.conv_tc_status() == 0
    assert torch.equal(out, ref_out)
    assert torch.equal(stats, ref_stats)
    if l <= 6000:
        a = [O.T(v) for v in (x, w, b, affine, alpha, res)]
        if variant.startswith("snake"):
            ref32 = O.conv1d_fused(a[0], a[1], a[2], a[3], "snake", alpha=a[4],
                                   residual=a[5] if variant == "snake_res" else None, padding=pad, dilation=d)[0]
        else:
            ref32 = O.conv1d_fused(a[0], a[1], a[2], a[3], "leaky", slope=0.2, residual=a[5],
                                   out_scale=0.7071067811865476, padding=pad, dilation=d)[0]
        assert rel_l2(out.cpu().numpy(), ref32.numpy()) <= REL_L2
    # the same padded operands through 4-byte accesses (route switch): still identical
    ops.set_conv_io("plain")
    try:
        with ops.padded_rows():
            out3, stats3 = call(px, pres)
    finally:
        ops.set_conv_io("tma")
    assert torch.equal(out3, out) and torch.equal(stats3, stats)


def test_conv1d_padded_rows_stay_inside_their_buffer(cuda):
    """A bulk tensor store is clipped at the end of the row (at 16-byte granularity: the padding columns of a row may
    be overwritten, they belong to the output buffer): nothing before the first row or after the last one is
    touched, and every valid column is written."""
    from lokinfer_b200 import ops
    ci = co = 128
    l, k, d = 1201, 7, 1
    x, w, b, affine, alpha, res = synth.conv_case(ci, co, l, k, 77)
    dw, db, daf, dal = dev(cuda, w, b, affine, alpha)
    state = ops.conv1d_prepare_f32_cuda(dw)
    guard = torch.full((co + 2, 1204), 123.0, device=cuda)

    def alloc(shape, device):
        return guard[1:co + 1] if tuple(shape) == (co, 1204) else torch.empty(shape, dtype=torch.float32, device=device)

    with ops.padded_rows():
        px = ops.to_cuda(x, cuda, rows=True)
        with ops.use_allocator(alloc):
            out, _ = ops.conv1d_snake_f32_cuda(px, dw, db, daf, dal, padding=3, dilation=1, state=state)
    assert out.data_ptr() == guard[1].data_ptr() and out.stride(0) == 1204
    assert ops.conv_tc_status() == 0
    assert torch.all(guard[0] == 123.0) and torch.all(guard[co + 1] == 123.0)
    assert not torch.any(guard[1:co + 1, :l] == 123.0)


def test_conv1d_weights_beyond_f16_range_fall_back_to_tf32_pack(cuda):
    """A weight beyond the f16 range (65504) cannot go into the f16 hi/lo pack: the pack kernel reports it and the
    prepare step packs the weight in the tf32 format instead, silently correct."""
    from lokinfer_b200 import ops
    ci = co = 128
    l, k, d = 700, 3, 1
    x, w, b, affine, alpha, res = synth.conv_case(ci, co, l, k, 9)
    w = w.copy()
    w[5, 17, 1] = 1.0e5
    dx, dw, db, daf, dal = dev(cuda, x, w, b, affine, alpha)
    st = ops.conv1d_prepare_f32_cuda(dw)
    assert st is not None and st.fmt == "tf32"
    assert ops.conv_tc_status() == 0
    out, _ = ops.conv1d_snake_f32_cuda(dx, dw, db, daf, dal, padding=1, dilation=1, state=st)
    assert ops.conv_tc_status() == 0
    a = [O.T(v) for v in (x, w, b, affine, alpha)]
    ref = O.conv1d_fused(a[0], a[1], a[2], a[3], "snake", alpha=a[4], padding=1, dilation=1)[0].numpy()
    assert rel_l2(out.cpu().numpy(), ref) <= REL_L2
    w2 = w.copy()
    w2[5, 17, 1] = 0.5
    assert ops.conv1d_prepare_f32_cuda(dev(cuda, w2)[0]).fmt == "f16"


TF32_CASES = [(128, 128, 1201, 3, 1), (128, 128, 1201, 7, 3), (256, 256, 640, 11, 5), (128, 128, 257, 7, 1),
              (16, 128, 700, 7, 3), (128, 22, 5000, 7, 1), (128, 128, 19201, 11, 3)]


@pytest.mark.parametrize("ci,co,l,k,d", TF32_CASES)
@pytest.mark.parametrize("variant", ["snake_res", "affine"])
def test_conv1d_tensor_core_tf32_split(cuda, ci, co, l, k, d, variant):
    """The second operand format of the tensor-core kernel (tf32 hi/lo halves, chosen when the state is prepared)
    is held to the same bars as the default f16 hi/lo split."""
    from lokinfer_b200 import ops
    x, w, b, affine, alpha, res = synth.conv_case(ci, co, l, k, ci * 31 + l + k)
    pad = d * (k - 1) // 2
    dx, dw, db, daf, dal, dres = dev(cuda, x, w, b, affine, alpha, res)
    ops.set_conv_path("tf32")
    try:
        state = ops.conv1d_prepare_f32_cuda(dw)
    finally:
        ops.set_conv_path("auto")
    assert state is not None
    if variant == "snake_res":
        out, stats = ops.conv1d_snake_f32_cuda(dx, dw, db, daf, dal, residual=dres, padding=pad, dilation=d,
                                               state=state)
    else:
        out, stats = ops.conv1d_affine_f32_cuda(dx, dw, db, daf, padding=pad, dilation=d, state=state)
    out, stats = out.cpu().numpy(), stats.cpu().numpy()

    def oracle(dt):
        a = [O.T(v, dt) for v in (x, w, b, affine, alpha, res)]
        if variant == "snake_res":
            return O.conv1d_fused(a[0], a[1], a[2], a[3], "snake", alpha=a[4], residual=a[5], padding=pad,
                                  dilation=d)[0].numpy()
        return O.conv1d_fused(a[0], a[1], a[2], a[3], "none", padding=pad, dilation=d)[0].numpy()

    ref32, ref64 = oracle(torch.float32), oracle(torch.float64)
    assert rel_l2(out, ref32) <= REL_L2
    assert rel_l2(out, ref64) <= 2 * rel_l2(ref32, ref64) + 2e-7
    check_stats(stats, out)
    assert ops.conv_tc_status() == 0


def test_conv1d_f16_split_reports_values_beyond_f16_range(cuda):
    """Activations beyond the f16 range (65504) overflow the f16 operand split and are reported in the status
    word (bit 0x10000); the tf32 split and the CUDA-core kernel take the same input without a report."""
    from lokinfer_b200 import ops
    ci = co = 128
    l, k, d = 600, 3, 1
    x, w, b, affine, alpha, res = synth.conv_case(ci, co, l, k, 5)
    x = x.copy()
    x[3, 100] = 3.0e5
    affine = np.stack([np.zeros(ci), np.ones(ci), np.zeros(ci)]).astype(np.float32)  # identity prologue
    dx, dw, db, daf = dev(cuda, x, w, b, affine)
    st = ops.conv1d_prepare_f32_cuda(dw)
    assert ops.conv_tc_status() == 0
    ops.conv1d_affine_f32_cuda(dx, dw, db, daf, padding=1, dilation=1, state=st)
    assert ops.conv_tc_status() == 0x10000      # reads and clears
    assert ops.conv_tc_status() == 0
    ops.set_conv_path("tf32")
    try:
        st32 = ops.conv1d_prepare_f32_cuda(dw)
    finally:
        ops.set_conv_path("auto")
    out, _ = ops.conv1d_affine_f32_cuda(dx, dw, db, daf, padding=1, dilation=1, state=st32)
    assert ops.conv_tc_status() == 0
    a = [O.T(v) for v in (x, w, b, affine)]
    ref = O.conv1d_fused(a[0], a[1], a[2], a[3], "none", padding=1, dilation=1)[0].numpy()
    assert rel_l2(out.cpu().numpy(), ref) <= REL_L2


def test_conv1d_fused_golden(cuda):
    from lokinfer_b200 import ops
    import importlib.util, pathlib
    spec = importlib.util.spec_from_file_location("make_golden", pathlib.Path(__file__).parent / "golden" / "make_golden.py")
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    c = mg.CONV
    x, w, b, affine, alpha, res = synth.conv_case(c["ci"], c["co"], c["l"], c["k"], c["seed"])
    d = dev(cuda, x, w, b, affine, alpha, res)
    out, stats = ops.conv1d_snake_f32_cuda(*d[:5], residual=d[5], padding=c["d"] * (c["k"] - 1) // 2, dilation=c["d"])
    assert rel_l2(out.cpu().numpy(), gold()["conv_out_f32"]) <= REL_L2
    np.testing.assert_allclose(out.cpu().numpy(), gold()["conv_out_f64"], atol=1e-4, rtol=1e-4)
    check_stats(stats.cpu().numpy(), out.cpu().numpy())
    # polyphase convT and iSTFT fixtures
    cx, cw, cb, cres = mg.convt_inputs()
    ct = mg.CONVT
    p = (ct["k"] - ct["s"]) // 2
    dx, dw, db, dres = dev(cuda, cx, cw, cb, cres)
    wp = ops.convt_poly_weights_cuda(dw, ct["s"], p)
    got = ops.conv_transpose1d_poly_f32_cuda(dx, wp, db, dres, stride=ct["s"], padding=p, taps=ct["k"] // ct["s"],
                                             slope=0.1, pad_left=ct["pl"]).cpu().numpy()
    assert rel_l2(got, gold()["convt_f32"]) <= REL_L2
    (dxi,) = dev(cuda, mg.istft_input())
    y = ops.istft_logits_f32_cuda(dxi).cpu().numpy()
    assert np.abs(y - gold()["istft_f64"]).max() <= 1e-5 * np.abs(gold()["istft_f64"]).max()


@pytest.mark.parametrize("c,l", [(4, 1), (16, 700), (128, 5000), (256, 3200), (128, 19201), (3, 128), (3, 129)])
def test_channel_stats_and_adain_affine(cuda, c, l):
    from lokinfer_b200 import ops
    r = np.random.default_rng(c + l)
    x = (r.standard_normal((c, l)) * 3 + 5).astype(np.float32)
    gb = (r.standard_normal(2 * c) * 0.5).astype(np.float32)
    dx, dgb = dev(cuda, x, gb)
    stats = ops.channel_stats_f32_cuda(dx)
    assert tuple(stats.shape) == (c, O.stat_chunks(l), 2)
    check_stats(stats.cpu().numpy(), x)
    af = ops.adain_affine_f32_cuda(stats, dgb, length=l).cpu().numpy()
    ref_af = O.adain_affine(O.channel_stats(t32(x)), t32(gb), l).numpy()
    np.testing.assert_allclose(af, ref_af, atol=2e-5, rtol=2e-5)
    got = (x - af[0][:, None]) * af[1][:, None] + af[2][:, None]
    ref = O.adain1d(t64(x), t64(gb)).numpy()
    np.testing.assert_allclose(got, ref, atol=2e-5 * max(1, np.abs(ref).max()), rtol=1e-4)


CONVT_CASES = [(8, 32, 5, 4, 2, 0), (16, 40, 37, 8, 4, 1), (512, 256, 26, 20, 10, 0), (512, 256, 294, 20, 10, 0),
               (256, 128, 2940, 12, 6, 1), (256, 128, 1, 12, 6, 1), (64, 64, 700, 12, 6, 1), (16, 8, 33, 6, 3, 1),
               (8, 4, 9, 5, 5, 0), (256, 128, 20800, 12, 6, 1), (512, 256, 2080, 20, 10, 0), (32, 7, 257, 20, 10, 1),
               (48, 21, 256, 12, 6, 0)]


@pytest.mark.parametrize("ci,co,l,k,s,pl", CONVT_CASES)
@pytest.mark.parametrize("mean3", [False, True])
def test_conv_transpose1d_poly(cuda, ci, co, l, k, s, pl, mean3):
    from lokinfer_b200 import ops
    r = np.random.default_rng(ci + l + k)
    xs = [(r.standard_normal((ci, l)) * 2).astype(np.float32) for _ in range(3)]
    w = (r.standard_normal((ci, co, k)) / math.sqrt(ci * k / s)).astype(np.float32)
    b = r.standard_normal(co).astype(np.float32)
    p = (k - s) // 2
    if 2 * p != (k // s - 1) * s:
        pytest.skip("not a polyphase shape")
    res = r.standard_normal((co, l * s + pl)).astype(np.float32)
    d = dev(cuda, *xs, w, b, res)
    wp = ops.convt_poly_weights_cuda(d[3], s, p)
    m3 = (d[1], d[2], 1.0 / 3.0) if mean3 else None
    got = ops.conv_transpose1d_poly_f32_cuda(d[0], wp, d[4], d[5], stride=s, padding=p, taps=k // s, slope=0.1,
                                             pad_left=pl, mean3=m3).cpu().numpy()

    def oracle(dt):
        a = [O.T(v, dt) for v in (*xs, w, b, res)]
        return O.conv_transpose1d_poly(a[0], a[3], a[4], a[5], s, p, 0.1, pad_left=pl,
                                       mean3=(a[1], a[2], 1.0 / 3.0) if mean3 else None).numpy()

    assert got.shape == (co, l * s + pl)
    assert rel_l2(got, oracle(torch.float32)) <= REL_L2
    np.testing.assert_allclose(got, oracle(torch.float64), atol=1e-4, rtol=1e-4)
    st = ops.conv_transpose1d_prepare_f32_cuda(d[3], s, p)
    assert (st is not None) == (s in (6, 10) and k == 2 * s and ci % 16 == 0)
    if st is not None and not mean3:  # the tensor-core path on the same operands
        got_tc = ops.conv_transpose1d_poly_f32_cuda(d[0], wp, d[4], d[5], stride=s, padding=p, taps=k // s, slope=0.1,
                                                    pad_left=pl, state=st).cpu().numpy()
        assert ops.conv_tc_status() == 0
        assert rel_l2(got_tc, oracle(torch.float32)) <= REL_L2
        np.testing.assert_allclose(got_tc, oracle(torch.float64), atol=1e-4, rtol=1e-4)
        e_tc, e_cpu = rel_l2(got_tc, oracle(torch.float64)), rel_l2(oracle(torch.float32), oracle(torch.float64))
        assert e_tc <= 2 * e_cpu + 2e-7
        # the same call with padded rows (x, res, out): identical values
        with ops.padded_rows():
            px, pres = ops.to_cuda(xs[0], cuda, rows=True), ops.to_cuda(res, cuda, rows=True)
            got_p = ops.conv_transpose1d_poly_f32_cuda(px, wp, d[4], pres, stride=s, padding=p, taps=k // s,
                                                       slope=0.1, pad_left=pl, state=st)
        assert ops.conv_tc_status() == 0
        np.testing.assert_array_equal(got_p.cpu().numpy(), got_tc)
        if pl == 1 and l * s > 2:
            # left reflect column, reference order (kokoro_conv.cpp:226): out[:, 0] = unpadded[:, 1] + res[:, 0] with
            # the plain conv sum. With a zero residual the column is an exact copy of out[:, 2].
            zres = torch.zeros_like(d[5])
            z = ops.conv_transpose1d_poly_f32_cuda(d[0], wp, d[4], zres, stride=s, padding=p, taps=k // s, slope=0.1,
                                                   pad_left=pl, state=st)
            assert torch.equal(z[:, 0], z[:, 2])
            # and with the residual: out[:, 0] - res[:, 0] and out[:, 2] - res[:, 2] round the same sum
            c0 = z[:, 0] + d[5][:, 0]
            assert torch.equal(torch.from_numpy(got_tc[:, 0]).to(cuda), c0)
    if mean3:  # bit-identical to add3_scale followed by the op (test_kokoro_conv_fused.py:252-264)
        m = ops.add3_scale_f32_cuda(d[0], d[1], d[2], 1.0 / 3.0)
        exp = ops.conv_transpose1d_poly_f32_cuda(m, wp, d[4], d[5], stride=s, padding=p, taps=k // s, slope=0.1,
                                                 pad_left=pl).cpu().numpy()
        np.testing.assert_array_equal(got, exp)


@pytest.mark.parametrize("l", [2, 3, 7, 57, 641, 1201, 19201])
def test_istft_logits(cuda, l):
    from lokinfer_b200 import ops
    x = np.random.default_rng(l).standard_normal((22, l)).astype(np.float32)
    (dx,) = dev(cuda, x)
    y = ops.istft_logits_f32_cuda(dx).cpu().numpy()
    ref64 = O.istft_logits(t64(x)).numpy()
    ref32 = O.istft_logits(t32(x)).numpy()
    assert y.shape == (5 * (l - 1),)
    assert np.abs(y - ref64).max() <= 1e-5 * np.abs(ref64).max()
    assert rel_l2(y, ref32) <= REL_L2


def test_istft_other_sizes(cuda):
    from lokinfer_b200 import ops
    for n_fft, hop, l in ((16, 4, 100), (8, 2, 33), (126, 21, 40)):
        x = (np.random.default_rng(n_fft).standard_normal((n_fft + 2, l)) * 0.5).astype(np.float32)
        (dx,) = dev(cuda, x)
        y = ops.istft_logits_f32_cuda(dx, n_fft=n_fft, hop=hop).cpu().numpy()
        ref = O.istft_logits(t64(x), n_fft, hop).numpy()
        assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("frames", [1, 3, 30, 119, 300, 1040])
def test_harmonic_source(cuda, frames):
    """Reference tolerance for this op: max-abs 2e-6 (tests/kernels/test_kokoro_kernels.py:510-522); the float32
    operation order is part of the contract, so the GPU tracks the oracle far below that."""
    from lokinfer_b200 import ops
    n = 2 * frames
    f0, noise, w, b = synth.source_case(n, frames)
    d = dev(cuda, f0, noise, w, b)
    for _ in range(2):  # second call reuses the per-device phase table
        out = ops.harmonic_source_f32_cuda(*d).cpu().numpy()
    ref = O.harmonic_source(f0, noise, w, b).numpy()
    assert out.shape == ref.shape == (600 * frames,)
    assert np.abs(out - ref).max() <= 2e-6
    assert rel_l2(out, ref) <= REL_L2
    # a shorter call after a longer one (table larger than needed)
    f0s, noises, ws, bs = synth.source_case(2, 99)
    outs = ops.harmonic_source_f32_cuda(*dev(cuda, f0s, noises, ws, bs)).cpu().numpy()
    assert np.abs(outs - O.harmonic_source(f0s, noises, ws, bs).numpy()).max() <= 2e-6


@pytest.mark.parametrize("frames,seed", [(1, 0), (30, 7), (238, 1234), (2080, -5), (1040, (1 << 63) - 1)])
def test_harmonic_source_rng(cuda, frames, seed):
    """The in-kernel noise variant (harmonic_source_rng): same Philox4x32-10 counters and Box-Muller pairing as the
    oracle's restatement of kernels/cpu/kokoro_signal.cpp:66-96, so the output matches harmonic_source fed with the
    oracle's noise within the op's tolerance (2e-6: the noise enters at amplitude 0.003 / 0.033, and logf / sinf /
    cosf differ from numpy's in the last ulp); deterministic per seed."""
    from lokinfer_b200 import ops
    f0, _, w, b = synth.source_case(frames, frames + 3)
    df0, dw, db = dev(cuda, f0, w, b)
    out = ops.harmonic_source_rng_f32_cuda(df0, dw, db, seed).cpu().numpy()
    ref = O.harmonic_source_rng(f0, w, b, seed).numpy()
    assert out.shape == ref.shape == (300 * frames,)
    assert np.abs(out - ref).max() <= 2e-6
    np.testing.assert_array_equal(out, ops.harmonic_source_rng_f32_cuda(df0, dw, db, seed).cpu().numpy())
    other = ops.harmonic_source_rng_f32_cuda(df0, dw, db, seed ^ 1).cpu().numpy()
    assert not np.array_equal(out, other)
    # and against the explicit-noise op with the same draw
    noise = O.source_noise_philox(seed, 300 * frames)
    exp = ops.harmonic_source_f32_cuda(df0, dev(cuda, noise)[0], dw, db).cpu().numpy()
    assert np.abs(out - exp).max() <= 2e-6


@pytest.mark.parametrize("s", [11, 25, 600, 6001, 600 * 300, 624000])
def test_stft_magphase(cuda, s):
    """tests/kernels/test_kokoro_kernels.py:529-542: magnitude within 1e-5 * max, wrapped phase within 1e-4 where
    the bin is significant."""
    from lokinfer_b200 import ops
    r = np.random.default_rng(s)
    t = np.arange(s)
    x = (0.3 * np.sin(t * 0.05) + 0.2 * np.sin(t * 0.9) + 0.05 * r.standard_normal(s)).astype(np.float32)
    x[: s // 7] = 0.0
    out = ops.stft_magphase_f32_cuda(dev(cuda, x)[0]).cpu().numpy()
    ref = O.stft_magphase(torch.from_numpy(x).double()).numpy()
    mag, ph = ref[:11], ref[11:]
    assert out.shape == (22, s // 5 + 1)
    np.testing.assert_allclose(out[:11], mag, atol=1e-5 * mag.max(), rtol=0)
    sig = mag > 1e-3 * mag.max()
    dph = np.angle(np.exp(1j * (out[11:].astype(np.float64) - ph)))
    assert np.abs(dph[sig]).max() < 1e-4
    dc = np.abs(out[11])  # imaginary part exactly 0 at DC: the phase is 0 or pi
    assert np.all((dc == 0) | (dc == np.float32(math.pi)))
    assert rel_l2(out[:11], O.stft_magphase_explicit(torch.from_numpy(x)).numpy()[:11]) <= REL_L2


def test_stft_of_harmonic_source_chain(cuda):
    """har = STFT(harmonic_source(F0)) as the generator's caller computes it, F = 119
    (tests/kernels/test_kokoro_kernels.py:556-575)."""
    from lokinfer_b200 import ops
    n = 238
    f0, noise, w, b = synth.source_case(n, 117)
    d = dev(cuda, f0, noise, w, b)
    out = ops.stft_magphase_f32_cuda(ops.harmonic_source_f32_cuda(*d)).cpu().numpy()
    src = O.harmonic_source(f0, noise, w, b)
    ref = O.stft_magphase(src.double()).numpy()
    mag, ph = ref[:11], ref[11:]
    assert out.shape == (22, 60 * n + 1)
    np.testing.assert_allclose(out[:11], mag, atol=1e-5 * mag.max(), rtol=0)
    sig = mag > 1e-3 * mag.max()
    dph = np.angle(np.exp(1j * (out[11:].astype(np.float64) - ph)))
    assert np.abs(dph[sig]).max() < 1e-3


def test_basic_ops(cuda):
    """The unfused parity layer: conv1d (all strides incl. noise_convs[0]), conv_transpose1d, adain1d (mean-100 trap),
    snake, leaky_relu, add, add3_scale, scale, pad_reflect1d (bit-exact data movement), gemm_bias."""
    from lokinfer_b200 import ops
    r = np.random.default_rng(5)
    # conv1d: (Ci, Co, L, K, s, p, d) from test_kokoro_kernels.py:347-368 style sweep
    for ci, co, l, k, s, p, d in [(22, 32, 1201, 12, 6, 3, 1), (22, 128, 961, 1, 1, 0, 1), (3, 5, 1, 1, 1, 0, 1),
                                  (4, 6, 10, 3, 2, 1, 2), (16, 16, 127, 7, 1, 9, 3), (8, 8, 5, 7, 1, 3, 1)]:
        x = r.standard_normal((ci, l)).astype(np.float32)
        w = (r.standard_normal((co, ci, k)) / math.sqrt(ci * k)).astype(np.float32)
        b = r.standard_normal(co).astype(np.float32)
        dx, dw, db = dev(cuda, x, w, b)
        got = ops.conv1d_f32_cuda(dx, dw, db, stride=s, padding=p, dilation=d).cpu().numpy()
        ref = O.conv1d(t64(x), t64(w), t64(b), stride=s, padding=p, dilation=d).numpy()
        assert got.shape == ref.shape
        np.testing.assert_allclose(got, ref, atol=1e-4, rtol=1e-4)
        assert rel_l2(got, O.conv1d(t32(x), t32(w), t32(b), stride=s, padding=p, dilation=d).numpy()) <= REL_L2
        got = ops.conv1d_nobias_f32_cuda(dx, dw, stride=s, padding=p, dilation=d).cpu().numpy()
        np.testing.assert_allclose(got, ref - b[:, None], atol=1e-4, rtol=1e-4)
    for ci, co, l, k, s, p, op in [(16, 12, 37, 8, 4, 2, 0), (512, 256, 26, 20, 10, 5, 0), (4, 3, 5, 3, 2, 0, 1)]:
        x = r.standard_normal((ci, l)).astype(np.float32)
        w = (r.standard_normal((ci, co, k)) / math.sqrt(ci * k / s)).astype(np.float32)
        b = r.standard_normal(co).astype(np.float32)
        dx, dw, db = dev(cuda, x, w, b)
        got = ops.conv_transpose1d_f32_cuda(dx, dw, db, stride=s, padding=p, output_padding=op).cpu().numpy()
        ref = O.conv_transpose1d(t64(x), t64(w), t64(b), stride=s, padding=p, output_padding=op).numpy()
        assert got.shape == ref.shape
        np.testing.assert_allclose(got, ref, atol=1e-4, rtol=1e-4)
    x = (r.standard_normal((4, 135001)) + 100).astype(np.float32)
    gb = (r.standard_normal(8) * 0.5).astype(np.float32)
    dx, dgb = dev(cuda, x, gb)
    np.testing.assert_allclose(ops.adain1d_f32_cuda(dx, dgb).cpu().numpy(), O.adain1d(t64(x), t64(gb)).numpy(),
                               atol=2e-4, rtol=1e-4)
    x = (r.standard_normal((6, 257)) * 2).astype(np.float32)
    al = r.uniform(0.2, 3.0, 6).astype(np.float32)
    dx, dal = dev(cuda, x, al)
    np.testing.assert_allclose(ops.snake_f32_cuda(dx, dal).cpu().numpy(), O.snake(t64(x), t64(al)).numpy(), atol=1e-6,
                               rtol=1e-6)
    np.testing.assert_array_equal(ops.leaky_relu_f32_cuda(dx, 0.1).cpu().numpy(), O.leaky_relu(t32(x), 0.1).numpy())
    a, b, c = (r.standard_normal((5, 33)).astype(np.float32) for _ in range(3))
    da, dbb, dc = dev(cuda, a, b, c)
    np.testing.assert_array_equal(ops.add_f32_cuda(da, dbb).cpu().numpy(), a + b)
    np.testing.assert_array_equal(ops.add3_scale_f32_cuda(da, dbb, dc, 1 / 3).cpu().numpy(),
                                  ((a + b) + c) * np.float32(1 / 3))
    np.testing.assert_array_equal(ops.scale_f32_cuda(da, 0.5).cpu().numpy(), a * np.float32(0.5))
    for left, right in ((1, 0), (0, 3), (4, 4)):
        np.testing.assert_array_equal(ops.pad_reflect1d_f32_cuda(da, left, right).cpu().numpy(),
                                      O.pad_reflect1d(t32(a), left, right).numpy())
    s = r.standard_normal((1, 128)).astype(np.float32)
    wt = (r.standard_normal((128, 1000)) / math.sqrt(128)).astype(np.float32)
    bb = r.standard_normal(1000).astype(np.float32)
    ds, dwt, dbv = dev(cuda, s, wt, bb)
    np.testing.assert_allclose(ops.gemm_bias_f32_cuda(ds, dwt, dbv).cpu().numpy(), s.astype(np.float64) @ wt + bb,
                               atol=1e-5, rtol=1e-5)


def test_errors_come_back_as_exceptions(cuda):
    """Entry points report failures through their return code and lkc_last_error(); nothing aborts."""
    from lokinfer_b200 import _lib, ops
    x = torch.zeros(22, 8, device=cuda)
    with pytest.raises(_lib.LkcError, match="istft_logits_f32_cuda"):
        out = torch.empty(7, device=cuda)  # wrong out length, bypassing the Python rule
        _lib.run("istft_logits_f32_cuda", [x.data_ptr(), out.data_ptr()], [22, 8, 7, 5, 20], (), None,
                 torch.cuda.current_stream().cuda_stream)
    # the context is still usable
    assert ops.istft_logits_f32_cuda(x).shape == (35,)


@pytest.mark.gpu
@pytest.mark.parametrize("ci,co,l,k,s,p", [(22, 256, 1201, 12, 6, 3), (22, 128, 999, 1, 1, 0), (5, 32, 500, 6, 3, 2),
                                           (22, 256, 124801, 12, 6, 3)])
def test_strided_conv_as_polyphase_conv_on_tensor_cores(cuda, ci, co, l, k, s, p):
    """space_to_depth + the stride-1 tensor-core conv with polyphase weights equals the strided conv (the generator's
    noise_convs, model.py:736-739): against the CUDA-core strided conv of the same library and, at the small sizes,
    against the float64 oracle."""
    from lokinfer_b200 import ops
    rng = np.random.default_rng(ci * 7 + l)
    x = rng.standard_normal((ci, l)).astype(np.float32)
    w = (rng.standard_normal((co, ci, k)) / np.sqrt(ci * k)).astype(np.float32)
    b = (rng.standard_normal(co) * 0.1).astype(np.float32)
    rows = -(-ci * s // 16) * 16
    dx, dw, db = dev(cuda, x, w, b)
    want = ops.conv1d_f32_cuda(dx, dw, db, stride=s, padding=p).cpu().numpy()
    wp = ops.to_cuda(ops.polyphase_conv_weights(w, s, rows), cuda)
    state = ops.conv1d_prepare_f32_cuda(wp)
    assert state is not None
    ident = torch.stack([torch.zeros(rows), torch.ones(rows), torch.zeros(rows)]).to(cuda)
    for padded in (False, True):
        with ops.padded_rows(padded):
            y = ops.space_to_depth_f32_cuda(dx, s, p, k // s, rows)
            got, stats = ops.conv1d_affine_f32_cuda(y, wp, db, ident, state=state)
        assert tuple(y.shape) == (rows, want.shape[1] + k // s - 1) and tuple(got.shape) == want.shape
        got = got.cpu().numpy()
        assert rel_l2(got, want) <= REL_L2
        check_stats(stats.cpu().numpy(), got)
    if l <= 2000:
        ref64 = torch.nn.functional.conv1d(t64(x)[None], t64(w), t64(b), stride=s, padding=p)[0].numpy()
        ref32 = torch.nn.functional.conv1d(t32(x)[None], t32(w), t32(b), stride=s, padding=p)[0].numpy()
        assert rel_l2(got, ref64) <= 2 * rel_l2(ref32, ref64) + 2e-7
    assert ops.conv_tc_status() == 0
