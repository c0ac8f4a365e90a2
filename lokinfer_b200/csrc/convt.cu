// ConvTranspose1d for the generator's two upsamplers.
//
// Polyphase form (the contract of the reference's conv_transpose1d_poly_f32_cpu):
//   out[co, padLeft + j s + r] = sum_c sum_{tt < taps} Wr[r][co][c][tt] * leaky(xin)[c, j + q_r - (taps-1) + tt]
//                                + bias[co] + res[co, padLeft + j s + r]
//   r' = (r + p) mod s, q_r = (r + p) div s, Wr[r][co][c][tt] = w[c, co, r' + (taps-1-tt) s]
// (K = taps s and 2 p = (taps-1) s, so every phase has exactly L outputs and taps is 1 or 2); with padLeft = 1
// the first output column is the reflect pad: out[co, 0] = unpadded[co, 1] + res[co, 0].
// The weight pack is f32[Ci, s, taps, Co] (output channel fastest) so a block's weight slice is read coalesced.
//
// One block = 32 output channels x 64 input columns x all s phases: warp w owns 4 channels, lane owns columns
// j and j + 32, the s phases live in registers, so the staged weights are warp-wide broadcasts and the input
// window reads are conflict-free. The finished tile goes through shared memory so the interleaved output rows
// (and the residual reads) are written as contiguous runs.
#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int BCO = 32, BJ = 64, CIC = 8, NTHREADS = 256;

struct PolyArgs {
  const float *x, *x2, *x3, *wp, *bias, *res;
  float* out;
  int ci, co, s, taps, p, padLeft;
  int64_t l, lo;
  float slope, inScale;
};

template <int S, int TAPS>
__global__ void __launch_bounds__(NTHREADS) convtPolyKernel(const PolyArgs a) {
  constexpr int WIN = BJ + TAPS;  // window slots: input columns j0 - (TAPS-1) .. j0 + BJ
  constexpr int WSZ = CIC * S * TAPS * BCO;
  constexpr int OUTW = BJ * S;
  extern __shared__ float smem[];
  float* xs = smem;              // [CIC][WIN]
  float* ws = smem + CIC * WIN;  // [CIC][S][TAPS][BCO]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t j0 = int64_t(blockIdx.x) * BJ;
  const int co0 = blockIdx.y * BCO;
  float acc[2][4][S];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int r = 0; r < S; ++r) acc[h][i][r] = 0.f;

  for (int c0 = 0; c0 < a.ci; c0 += CIC) {
    __syncthreads();
    for (int idx = tid; idx < CIC * WIN; idx += NTHREADS) {
      const int cc = idx / WIN, q = idx - cc * WIN, c = c0 + cc;
      const int64_t pos = j0 - (TAPS - 1) + q;
      float v = 0.f;
      if (c < a.ci && pos >= 0 && pos < a.l) {
        const int64_t i = int64_t(c) * a.l + pos;
        v = a.x[i];
        if (a.x2) v = __fmul_rn(__fadd_rn(__fadd_rn(v, a.x2[i]), a.x3[i]), a.inScale);
        v = v >= 0.f ? v : v * a.slope;
      }
      xs[idx] = v;
    }
    for (int idx = tid; idx < WSZ; idx += NTHREADS) {
      const int col = idx % BCO, rem = idx / BCO;  // rem = (cc * S + r) * TAPS + tt
      const int cc = rem / (S * TAPS), c = c0 + cc, co = co0 + col;
      ws[idx] = (c < a.ci && co < a.co) ? a.wp[(int64_t(c) * S * TAPS + (rem - cc * S * TAPS)) * a.co + co] : 0.f;
    }
    __syncthreads();
#pragma unroll 2
    for (int cc = 0; cc < CIC; ++cc) {
      float xv[2][TAPS + 1];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int q = 0; q <= TAPS; ++q) xv[h][q] = xs[cc * WIN + lane + 32 * h + q];
      const float* wr = ws + cc * S * TAPS * BCO + warp * 4;
#pragma unroll
      for (int r = 0; r < S; ++r) {
        const int qr = (r + a.p) >= S ? 1 : 0;
#pragma unroll
        for (int tt = 0; tt < TAPS; ++tt) {
          const float4 w4 = *reinterpret_cast<const float4*>(wr + (r * TAPS + tt) * BCO);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float v = qr ? xv[h][tt + 1] : xv[h][tt];
            acc[h][0][r] = fmaf(w4.x, v, acc[h][0][r]);
            acc[h][1][r] = fmaf(w4.y, v, acc[h][1][r]);
            acc[h][2][r] = fmaf(w4.z, v, acc[h][2][r]);
            acc[h][3][r] = fmaf(w4.w, v, acc[h][3][r]);
          }
        }
      }
    }
  }
  // Through shared memory, 8 channels (one per warp) at a time: tile row [BJ * S] in output order.
  __syncthreads();
  float* tile = smem;  // [8][OUTW]
  const int64_t u0 = j0 * S;  // first unpadded output column of the tile
  const int64_t lu = a.l * S;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int r = 0; r < S; ++r) tile[warp * OUTW + (lane + 32 * h) * S + r] = acc[h][i][r];
    __syncwarp();
    const int co = co0 + warp * 4 + i;
    if (co < a.co) {
      const float b = a.bias[co];
      const float* rrow = a.res + int64_t(co) * a.lo + a.padLeft;
      float* orow = a.out + int64_t(co) * a.lo + a.padLeft;
      for (int q = lane; q < OUTW; q += 32) {
        const int64_t u = u0 + q;
        if (u < lu) orow[u] = (tile[warp * OUTW + q] + b) + rrow[u];
      }
      if (a.padLeft && j0 == 0 && lane == 0 && lu > 1)
        a.out[int64_t(co) * a.lo] = (tile[warp * OUTW + 1] + b) + a.res[int64_t(co) * a.lo];
    }
    __syncwarp();
  }
}

// Any stride / taps: one thread per output element (slow; the Kokoro strides use the tiled kernel).
__global__ void convtPolyGenericKernel(const PolyArgs a) {
  const int64_t lu = a.l * a.s, n = int64_t(a.co) * a.lo;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < n; idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t co = idx / a.lo, o = idx - co * a.lo;
    int64_t u = o - a.padLeft;
    if (u < 0) u = 1;  // reflect column
    if (u >= lu) continue;
    const int64_t j = u / a.s;
    const int r = static_cast<int>(u - j * a.s), qr = (r + a.p) / a.s;
    float acc = 0.f;
    for (int c = 0; c < a.ci; ++c)
      for (int tt = 0; tt < a.taps; ++tt) {
        const int64_t pos = j + qr - (a.taps - 1) + tt;
        if (pos < 0 || pos >= a.l) continue;
        const int64_t i = int64_t(c) * a.l + pos;
        float v = a.x[i];
        if (a.x2) v = __fmul_rn(__fadd_rn(__fadd_rn(v, a.x2[i]), a.x3[i]), a.inScale);
        v = v >= 0.f ? v : v * a.slope;
        acc = fmaf(a.wp[((int64_t(c) * a.s + r) * a.taps + tt) * a.co + co], v, acc);
      }
    a.out[idx] = (acc + a.bias[co]) + a.res[idx];
  }
}

__global__ void convtPackKernel(const float* __restrict__ w, float* __restrict__ wp, int ci, int co, int k, int s,
                                int taps, int p) {
  const int64_t n = int64_t(ci) * s * taps * co;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < n; idx += int64_t(gridDim.x) * blockDim.x) {
    const int o = static_cast<int>(idx % co);
    int64_t rem = idx / co;
    const int tt = static_cast<int>(rem % taps);
    rem /= taps;
    const int r = static_cast<int>(rem % s), c = static_cast<int>(rem / s);
    wp[idx] = w[(int64_t(c) * co + o) * k + (r + p) % s + (taps - 1 - tt) * s];
  }
}

// Plain F.conv_transpose1d, one thread per output (the unfused parity layer).
__global__ void convtBasicKernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                 float* __restrict__ out, int ci, int64_t l, int co, int k, int s, int p, int64_t lo) {
  const int64_t n = int64_t(co) * lo;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < n; idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t o = idx / lo, q = idx - o * lo, t = q + p;  // t = j s + kk
    const int64_t jHi = t / s < l - 1 ? t / s : l - 1;
    const int64_t jLo = t - (k - 1) <= 0 ? 0 : (t - (k - 1) + s - 1) / s;
    float acc = 0.f;
    for (int c = 0; c < ci; ++c) {
      const float* xr = x + int64_t(c) * l;
      const float* wr = w + (int64_t(c) * co + o) * k;
      for (int64_t j = jLo; j <= jHi; ++j) acc = fmaf(xr[j], wr[t - j * s], acc);
    }
    out[idx] = acc + (b ? b[o] : 0.f);
  }
}

template <int S, int TAPS>
int launchPoly(const PolyArgs& a, cudaStream_t s) {
  constexpr size_t stage = sizeof(float) * (CIC * (BJ + TAPS) + CIC * S * TAPS * BCO);
  constexpr size_t tile = sizeof(float) * 8 * BJ * S;
  constexpr size_t smem = stage > tile ? stage : tile;
  static_assert(smem <= 48 * 1024, "convt tile must fit the default shared-memory limit");
  dim3 grid(static_cast<unsigned>(ceilDiv(a.l, BJ)), static_cast<unsigned>(ceilDiv(a.co, BCO)));
  convtPolyKernel<S, TAPS><<<grid, NTHREADS, smem, s>>>(a);
  return launched("conv_transpose1d_poly_f32_cuda");
}

int runPoly(const LkcArgs* a, void* stream, bool mean3) {
  const int base = mean3 ? 2 : 0;  // extra operands x2, x3
  LKC_REQUIRE(a && a->numPtrs == uint32_t(5 + base) && a->floats, "conv_transpose1d_poly: bad operand count");
  const int64_t* n = a->ints;
  const int sh = 2 * base;  // extra shape ints
  PolyArgs p;
  p.x = F(a, 0);
  p.x2 = mean3 ? F(a, 1) : nullptr;
  p.x3 = mean3 ? F(a, 2) : nullptr;
  p.wp = F(a, 1 + base);
  p.bias = F(a, 2 + base);
  p.res = F(a, 3 + base);
  p.out = O(a, 4 + base);
  const uint32_t nint = uint32_t(2 + sh + 4 + 1 + 2 + 2 + 4);
  // optional trailing ints (not with mean3): row pitches of x, res, out; served by the tensor-core route only
  // then (window extension, time-sharded tensors) halo_left, halo_right: x holds that many real columns before / after
  // the columns that produce output
  const bool windowed = !mean3 && a->numInts == nint + 5;
  const bool pitched = !mean3 && (a->numInts == nint + 3 || windowed);
  LKC_REQUIRE(a->numInts == nint || pitched, "conv_transpose1d_poly: bad ints count");
  const int64_t haloL = windowed ? n[nint + 3] : 0, haloR = windowed ? n[nint + 4] : 0;
  LKC_REQUIRE(haloL >= 0 && haloL <= 1 && haloR >= 0 && haloR <= 1 && n[1] > haloL + haloR,
              "conv_transpose1d_poly: halos must be 0 or 1 column");
  const int64_t ci = n[0], l = n[1] - haloL - haloR;  // columns that produce output
  if (mean3)
    LKC_REQUIRE(n[2] == ci && n[3] == l && n[4] == ci && n[5] == l, "conv_transpose1d_poly_mean3: x2 / x3 must match x");
  const int64_t* wd = n + 2 + sh;  // wp dims (Ci, s, taps, Co)
  const int64_t co = n[2 + sh + 4];
  const int64_t* at = n + 2 + sh + 4 + 1 + 2 + 2;  // pad_left padding stride taps
  const int64_t padLeft = at[0], pad = at[1], s = at[2], taps = at[3];
  LKC_REQUIRE(s >= 1 && taps >= 1 && 2 * pad == (taps - 1) * s && pad >= 0 && pad < s,
              "conv_transpose1d_poly: needs 2p = (taps-1)*s and 0 <= p < s");
  LKC_REQUIRE(padLeft == 0 || padLeft == 1, "conv_transpose1d_poly: pad_left must be 0 or 1");
  LKC_REQUIRE(wd[0] == ci && wd[1] == s && wd[2] == taps && wd[3] == co,
              "conv_transpose1d_poly: wp must be f32[Ci, stride, taps, Co] from convt_poly_pack_f32_cuda");
  const int64_t lo = l * s + padLeft;
  const int64_t* rd = n + 2 + sh + 4 + 1;
  LKC_REQUIRE(rd[0] == co && rd[1] == lo && rd[2] == co && rd[3] == lo,
              "conv_transpose1d_poly: residual and out must be f32[Co, L*s + pad_left]");
  LKC_REQUIRE(l >= 1 && ci >= 1 && co >= 1, "conv_transpose1d_poly: empty operand");
  LKC_REQUIRE(ci < (1 << 24) && co < (1 << 21) && s <= 4096, "conv_transpose1d_poly: shape out of range");
  p.ci = int(ci), p.co = int(co), p.s = int(s), p.taps = int(taps), p.p = int(pad), p.padLeft = int(padLeft);
  p.l = l, p.lo = lo;
  p.inScale = mean3 ? static_cast<float>(a->floats[0]) : 1.f;
  p.slope = static_cast<float>(a->floats[mean3 ? 1 : 0]);
  cudaStream_t st = S(stream);
  if (a->state && !mean3 && !convPathForcedSimt()) {
    // prepared tensor-core pack of this weight (lkc_convt_state_create): same contract on tcgen05
    const ConvState* cs = static_cast<const ConvState*>(a->state);
    LKC_REQUIRE(cs->wp && cs->stride == s && cs->ci == ci && cs->co == co && cs->k == taps * s,
                "conv_transpose1d_poly: the prepared state does not match the weight shape");
    if (convtTcEligible(ci, co, taps * s, s, pad)) {
      ConvtParams cp{p.x, p.bias, p.res, p.out, ci, l, co, s, padLeft, p.slope};
      if (pitched) {
        cp.xPitch = n[nint], cp.resPitch = n[nint + 1], cp.outPitch = n[nint + 2];
        cp.haloLeft = haloL, cp.haloRight = haloR;
        LKC_REQUIRE(cp.xPitch >= n[1] && cp.resPitch >= lo && cp.outPitch >= lo,
                    "conv_transpose1d_poly: a row pitch is smaller than the row");
      }
      return convtTc(cp, cs->wp, cs->f16, st);
    }
  }
  LKC_REQUIRE(!pitched || (!windowed && n[nint] == l && n[nint + 1] == lo && n[nint + 2] == lo),
              "conv_transpose1d_poly: padded rows need the tensor-core route (a prepared state of an eligible shape)");
  if (taps == 2 && ceilDiv(co, BCO) <= 65535) {
    switch (s) {
      case 2: return launchPoly<2, 2>(p, st);
      case 4: return launchPoly<4, 2>(p, st);
      case 6: return launchPoly<6, 2>(p, st);
      case 10: return launchPoly<10, 2>(p, st);
      default: break;
    }
  }
  const int64_t total = co * lo;
  const int blocks = static_cast<int>(ceilDiv(total, 256) > 148 * 16 ? 148 * 16 : ceilDiv(total, 256));
  convtPolyGenericKernel<<<blocks, 256, 0, st>>>(p);
  return launched("conv_transpose1d_poly_f32_cuda");
}

}  // namespace
}  // namespace lkc

using namespace lkc;

extern "C" LKC_API int lkc_conv_transpose1d_poly_f32_cuda(const LkcArgs* a, void* stream) { return runPoly(a, stream, false); }
extern "C" LKC_API int lkc_conv_transpose1d_poly_mean3_f32_cuda(const LkcArgs* a, void* stream) {
  return runPoly(a, stream, true);
}

extern "C" LKC_API int lkc_convt_poly_pack_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts == 9, "convt_poly_pack_f32_cuda: expected w | wp, padding, stride");
  const int64_t* n = a->ints;
  const int64_t ci = n[0], co = n[1], k = n[2], pad = n[7], s = n[8];
  LKC_REQUIRE(s >= 1 && k % s == 0, "convt_poly_pack_f32_cuda: needs K = taps*s");
  const int64_t taps = k / s;
  LKC_REQUIRE(2 * pad == (taps - 1) * s && pad >= 0 && pad < s, "convt_poly_pack_f32_cuda: needs 2p = (taps-1)*s");
  LKC_REQUIRE(n[3] == ci && n[4] == s && n[5] == taps && n[6] == co,
              "convt_poly_pack_f32_cuda: wp must be f32[Ci, stride, taps, Co]");
  const int64_t total = ci * k * co;
  if (total == 0) return 0;
  LKC_REQUIRE(ci < (1 << 24) && co < (1 << 24) && k < (1 << 16), "convt_poly_pack_f32_cuda: shape out of range");
  const int blocks = static_cast<int>(ceilDiv(total, 256) > 4096 ? 4096 : ceilDiv(total, 256));
  convtPackKernel<<<blocks, 256, 0, S(stream)>>>(F(a, 0), O(a, 1), int(ci), int(co), int(k), int(s), int(taps),
                                                 int(pad));
  return launched("convt_poly_pack_f32_cuda");
}

extern "C" LKC_API int lkc_conv_transpose1d_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 4 && a->numInts == 11, "conv_transpose1d_f32_cuda: expected x, w, b | out + 3 attrs");
  const int64_t* n = a->ints;
  const int64_t ci = n[0], l = n[1], co = n[3], k = n[4], op = n[8], pad = n[9], s = n[10];
  LKC_REQUIRE(n[2] == ci && n[5] == co, "conv_transpose1d_f32_cuda: w must be [Ci, Co, K], b f32[Co]");
  LKC_REQUIRE(s >= 1 && pad >= 0 && op >= 0 && op < s, "conv_transpose1d_f32_cuda: invalid stride/padding/output_padding");
  const int64_t lo = (l - 1) * s - 2 * pad + k + op;
  LKC_REQUIRE(lo >= 1 && n[6] == co && n[7] == lo, "conv_transpose1d_f32_cuda: out must be f32[Co, (L-1)s - 2p + K + op]");
  LKC_REQUIRE(ci < (1 << 24) && co < (1 << 24) && k < (1 << 16) && s < (1 << 16) && pad < (1 << 24),
              "conv_transpose1d_f32_cuda: shape out of range");
  const int64_t total = co * lo;
  const int blocks = static_cast<int>(ceilDiv(total, 256) > 148 * 16 ? 148 * 16 : ceilDiv(total, 256));
  convtBasicKernel<<<blocks, 256, 0, S(stream)>>>(F(a, 0), F(a, 1), F(a, 2), O(a, 3), int(ci), l, int(co), int(k),
                                                  int(s), int(pad), lo);
  return launched("conv_transpose1d_f32_cuda");
}
