"""Generates tests/golden/kokoro_golden.npz: outputs of the CPU oracle (float32 = reference precision, float64 =
golden) on small seeded cases. Inputs are not stored: lokinfer_b200.synth rebuilds them from the seeds below.

    python tests/golden/make_golden.py

The reference itself cannot run on this host (Apple-only CPU kernels, nanobind extension), so these vectors come
from the oracle after it has been pinned against the reference's test recipes (tests/test_oracle.py)."""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from lokinfer_b200 import synth  # noqa: E402
from oracle import kokoro_oracle as O  # noqa: E402

CONV = dict(ci=16, co=12, l=700, k=7, d=3, seed=101)
RESBLOCK = dict(c=16, l=300, k=7, seed=102)
CONVT = dict(ci=16, co=40, l=37, k=8, s=4, pl=1, seed=103)
ISTFT = dict(l=57, seed=104)
GEN = dict(t=4, wseed=0, iseed=1)


def conv_case(dt):
    c = CONV
    x, w, b, affine, alpha, res = (O.T(a, dt) for a in synth.conv_case(c["ci"], c["co"], c["l"], c["k"], c["seed"]))
    return O.conv1d_fused(x, w, b, affine, "snake", alpha=alpha, residual=res, padding=c["d"] * (c["k"] - 1) // 2,
                          dilation=c["d"])


def resblock_case(dt):
    c = RESBLOCK
    sd, x, s = synth.resblock_case(c["c"], c["l"], c["k"], c["seed"])
    sd = {k: O.T(v, dt) for k, v in sd.items()}
    gbs = O.style_bank(sd, O.T(s, dt))
    return O.adain_resblock1_fused(O.T(x, dt), gbs, sd, "rb", c["k"])[0]


def convt_inputs():
    c = CONVT
    r = np.random.default_rng(c["seed"])
    x = (r.standard_normal((c["ci"], c["l"])) * 2).astype(np.float32)
    w = (r.standard_normal((c["ci"], c["co"], c["k"])) / np.sqrt(c["ci"] * c["k"] / c["s"])).astype(np.float32)
    b = r.standard_normal(c["co"]).astype(np.float32)
    res = r.standard_normal((c["co"], c["l"] * c["s"] + c["pl"])).astype(np.float32)
    return x, w, b, res


def convt_case(dt):
    c = CONVT
    x, w, b, res = (O.T(a, dt) for a in convt_inputs())
    return O.conv_transpose1d_poly(x, w, b, res, c["s"], (c["k"] - c["s"]) // 2, 0.1, pad_left=c["pl"])


def istft_input():
    return np.random.default_rng(ISTFT["seed"]).standard_normal((22, ISTFT["l"])).astype(np.float32)


def gen_case(dt):
    sd = synth.generator_weights(GEN["wseed"])
    inp = synth.generator_inputs(GEN["t"], GEN["iseed"])
    st = O.generator(sd, O.T(inp["x"], dt), O.T(inp["har"], dt), O.T(inp["s"], dt), fused=True, stages=True)
    return st["post"], st["audio"]


def main():
    torch.set_num_threads(1)
    out = {}
    for tag, dt in (("f32", torch.float32), ("f64", torch.float64)):
        y, st = conv_case(dt)
        out[f"conv_out_{tag}"], out[f"conv_stats_{tag}"] = y.numpy(), st.numpy()
        out[f"resblock_{tag}"] = resblock_case(dt).numpy()
        out[f"convt_{tag}"] = convt_case(dt).numpy()
        out[f"istft_{tag}"] = O.istft_logits(O.T(istft_input(), dt)).numpy()
        post, audio = gen_case(dt)
        out[f"gen_post_{tag}"], out[f"gen_audio_{tag}"] = post.numpy(), audio.numpy()
    path = Path(__file__).resolve().parent / "kokoro_golden.npz"
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
