// CUDA-core implicit-GEMM conv1d for any shape: the fused family
//   out = (conv1d(act((xin - mean) * scale + beta), w) + b [+ res]) [* oscale],  xin = x or ((x + x2) + x3) * s
// with the output's per-(channel, 128-sample chunk) (mean, M2), and the plain strided conv1d.
// This is the generic path (any Ci / Co / K / dilation / padding / stride); shapes the tensor-core kernel
// accepts are routed there by the entry points.
//
// One block = 64 output channels x 128 output columns (exactly one stats chunk), 256 threads, each thread a
// 4 (channels) x 8 (columns tx + 16 j) register tile. Per 8-input-channel step the block stages the transformed
// input window (activation applied once per element, zeros outside [0, L) written after the activation, as the
// reference does) and the weight slice in shared memory.
#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int BCO = 64, BT = 128, CIC = 8, NTHREADS = 256;

struct SimtArgs {
  const float *x, *x2, *x3, *w, *bias, *affine, *alpha, *residual;
  float *out, *stats;
  int ci, co, k, dilation, padding, stride;
  int64_t l, lo, nchunks;
  int64_t xPitch, resPitch, outPitch;  // row pitches in floats
  int64_t validLo, validHi;            // x columns outside [validLo, validHi) are zero padding (after the activation)
  float slope, outScale, inScale;
  int win;  // staged window length per input channel
};

template <int ACT, bool MEAN3>
__device__ __forceinline__ float loadTransformed(const SimtArgs& p, int c, int64_t pos, float mean, float scale,
                                                 float beta, float alpha, float inv) {
  const int64_t i = int64_t(c) * p.xPitch + pos;
  float v = p.x[i];
  if (MEAN3) v = __fmul_rn(__fadd_rn(__fadd_rn(v, p.x2[i]), p.x3[i]), p.inScale);
  v = (v - mean) * scale + beta;
  if (ACT == 1) {
    const float s = sinf(alpha * v);
    v = v + inv * (s * s);
  } else if (ACT == 2) {
    v = v >= 0.f ? v : v * p.slope;
  }
  return v;
}

template <int ACT, bool MEAN3>
__global__ void __launch_bounds__(NTHREADS) convSimtKernel(const SimtArgs p) {
  extern __shared__ float smem[];
  float* xs = smem;                 // [CIC][win]
  float* ws = smem + CIC * p.win;   // [CIC][k][BCO]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t t0 = int64_t(blockIdx.x) * BT;
  const int co0 = blockIdx.y * BCO;
  const int64_t p0 = t0 * p.stride - p.padding;  // input position of window slot 0
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  for (int c0 = 0; c0 < p.ci; c0 += CIC) {
    __syncthreads();
    for (int idx = tid; idx < CIC * p.win; idx += NTHREADS) {
      const int cc = idx / p.win, q = idx - cc * p.win, c = c0 + cc;
      const int64_t pos = p0 + q;
      float v = 0.f;
      if (c < p.ci && pos >= p.validLo && pos < p.validHi) {
        float mean = 0.f, scale = 1.f, beta = 0.f, alpha = 0.f, inv = 0.f;
        if (p.affine) mean = p.affine[c], scale = p.affine[p.ci + c], beta = p.affine[2 * p.ci + c];
        if (ACT == 1) alpha = p.alpha[c], inv = 1.f / alpha;
        v = loadTransformed<ACT, MEAN3>(p, c, pos, mean, scale, beta, alpha, inv);
      }
      xs[idx] = v;
    }
    for (int idx = tid; idx < CIC * p.k * BCO; idx += NTHREADS) {
      const int col = idx % BCO, rem = idx / BCO;  // rem = cc * k + kk
      const int cc = rem / p.k, kk = rem - cc * p.k, c = c0 + cc, co = co0 + col;
      ws[idx] = (c < p.ci && co < p.co) ? p.w[(int64_t(co) * p.ci + c) * p.k + kk] : 0.f;
    }
    __syncthreads();
    for (int cc = 0; cc < CIC; ++cc) {
      const float* xr = xs + cc * p.win + tx * p.stride;
      const float* wr = ws + cc * p.k * BCO + ty * 4;
      for (int kk = 0; kk < p.k; ++kk) {
        const float4 w4 = *reinterpret_cast<const float4*>(wr + kk * BCO);
        const float* xk = xr + kk * p.dilation;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xv = xk[16 * j * p.stride];
          acc[0][j] = fmaf(w4.x, xv, acc[0][j]);
          acc[1][j] = fmaf(w4.y, xv, acc[1][j]);
          acc[2][j] = fmaf(w4.z, xv, acc[2][j]);
          acc[3][j] = fmaf(w4.w, xv, acc[3][j]);
        }
      }
    }
  }

  const int64_t nrem = p.lo - t0;
  const int n = static_cast<int>(nrem < BT ? nrem : BT);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int co = co0 + ty * 4 + i;
    const bool cok = co < p.co;
    const float b = (cok && p.bias) ? p.bias[co] : 0.f;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int tl = tx + 16 * j;
      float v = acc[i][j] + b;
      if (cok && tl < n) {
        const int64_t o = int64_t(co) * p.outPitch + t0 + tl;
        if (p.residual) {
          v += p.residual[int64_t(co) * p.resPitch + t0 + tl];
          if (p.outScale != 1.f) v *= p.outScale;
        }
        p.out[o] = v;
      } else {
        v = 0.f;
      }
      acc[i][j] = v;
      sum += v;
    }
    if (p.stats) {
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      const float mean = sum / static_cast<float>(n);
      float q = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = (tx + 16 * j) < n ? acc[i][j] - mean : 0.f;
        q = fmaf(d, d, q);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
      if (tx == 0 && cok) {
        float* st = p.stats + (int64_t(co) * p.nchunks + blockIdx.x) * 2;
        st[0] = mean;
        st[1] = q;
      }
    }
  }
}

template <int ACT, bool MEAN3>
int launch(const SimtArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
  static bool configured[64] = {};  // per instantiation and device; the attribute is sticky for the context
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(convSimtKernel<ACT, MEAN3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024);
    if (e != cudaSuccess) return failCuda("conv (CUDA-core): cudaFuncSetAttribute", e);
    configured[dev] = true;
  }
  convSimtKernel<ACT, MEAN3><<<grid, NTHREADS, smem, s>>>(a);
  return launched("conv (CUDA-core)");
}

}  // namespace

int convSimt(const ConvFusedParams& p, int64_t stride, cudaStream_t s) {
  SimtArgs a;
  a.x = p.x, a.x2 = p.x2, a.x3 = p.x3, a.w = p.w, a.bias = p.bias, a.affine = p.affine, a.alpha = p.alpha;
  a.residual = p.residual, a.out = p.out, a.stats = p.stats;
  LKC_REQUIRE(p.ci <= (1 << 20) && p.co <= (1 << 20) && p.k <= 4096 && p.dilation <= 4096 && p.padding <= (1 << 24) &&
                  stride <= 4096 && p.xOrigin >= 0 && p.xOrigin <= (1 << 24),
              "conv: shape out of range");
  a.ci = int(p.ci), a.co = int(p.co), a.k = int(p.k), a.dilation = int(p.dilation), a.padding = int(p.padding);
  a.stride = int(stride);
  a.l = p.l, a.lo = p.lo, a.nchunks = p.statsStride ? p.statsStride : statChunks(p.lo);
  a.padding = int(p.padding - p.xOrigin);  // window slot 0 of output column t is x column t * stride - padding + xOrigin
  a.validLo = p.validLo < 0 ? 0 : p.validLo, a.validHi = (p.validHi < 0 || p.validHi > p.l) ? p.l : p.validHi;
  a.xPitch = p.xPitch ? p.xPitch : p.l, a.resPitch = p.resPitch ? p.resPitch : p.lo;
  a.outPitch = p.outPitch ? p.outPitch : p.lo;
  a.slope = p.slope, a.outScale = p.outScale, a.inScale = p.inScale;
  a.win = (BT - 1) * a.stride + (a.k - 1) * a.dilation + 1;
  const size_t smem = sizeof(float) * (size_t(CIC) * a.win + size_t(CIC) * a.k * BCO);
  LKC_REQUIRE(smem <= 200 * 1024, "conv: kernel window too large for the generic kernel (K * dilation or stride)");
  const int64_t tiles = ceilDiv(p.lo, BT), cotiles = ceilDiv(p.co, BCO);
  LKC_REQUIRE(tiles <= 0x7fffffff && cotiles <= 65535, "conv: grid too large");
  dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(cotiles));
  const bool m3 = p.x2 != nullptr;
  switch (p.act) {
    case Act::None:
      return m3 ? launch<0, true>(a, grid, smem, s) : launch<0, false>(a, grid, smem, s);
    case Act::Snake:
      return m3 ? launch<1, true>(a, grid, smem, s) : launch<1, false>(a, grid, smem, s);
    case Act::Leaky:
      return m3 ? launch<2, true>(a, grid, smem, s) : launch<2, false>(a, grid, smem, s);
  }
  return fail("conv: bad activation");
}

}  // namespace lkc
