// Basic (unfused) layer and the HBM-bound statistics kernels of the Kokoro generator path:
// snake / leaky_relu / add / add3_scale / scale / pad_reflect1d / adain1d, channel_stats, adain_affine and the
// style-bank GEMV. Each is a streaming kernel: one pass over its operands, coalesced along time, grids sized
// from the element count.
#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int kThreads = 256;

inline int gridFor(int64_t n, int perThread = 1) {
  int64_t b = ceilDiv(n, int64_t(kThreads) * perThread);
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 32 ? 148 * 32 : b));
}

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warpSumD(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void snakeKernel(const float* __restrict__ x, const float* __restrict__ alpha, float* __restrict__ out,
                            int64_t c, int64_t l) {
  const int64_t n = c * l;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const float a = alpha[i / l], v = x[i];
    const float s = sinf(a * v);
    out[i] = v + (1.f / a) * (s * s);
  }
}

__global__ void leakyKernel(const float* __restrict__ x, float* __restrict__ out, int64_t n, float slope) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const float v = x[i];
    out[i] = v > 0.f ? v : v * slope;
  }
}

__global__ void addKernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                          int64_t n) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    out[i] = a[i] + b[i];
}

__global__ void add3ScaleKernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ c,
                                float* __restrict__ out, int64_t n, float s) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    out[i] = __fmul_rn(__fadd_rn(__fadd_rn(a[i], b[i]), c[i]), s);
}

__global__ void scaleKernel(const float* __restrict__ x, float* __restrict__ out, int64_t n, float s) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    out[i] = x[i] * s;
}

__global__ void padReflectKernel(const float* __restrict__ x, float* __restrict__ out, int64_t c, int64_t l,
                                 int64_t left, int64_t right) {
  const int64_t lo = left + l + right, n = c * lo;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t ch = i / lo, j = i - ch * lo;
    int64_t src = j - left;
    if (src < 0) src = -src;
    if (src >= l) src = 2 * (l - 1) - src;
    out[i] = x[ch * l + src];
  }
}

// One block per channel: two-pass mean / biased variance, then (x - mean) * a + b.
__global__ void adain1dKernel(const float* __restrict__ x, const float* __restrict__ gb, float* __restrict__ out,
                              int64_t c, int64_t l, float eps) {
  __shared__ double red[kThreads / 32];
  __shared__ float bc[2];
  const int64_t ch = blockIdx.x;
  const float* xr = x + ch * l;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  double s = 0.0;
  for (int64_t i = threadIdx.x; i < l; i += blockDim.x) s += xr[i];
  s = warpSumD(s);
  if (lane == 0) red[wid] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) t += red[w];
    bc[0] = static_cast<float>(t / static_cast<double>(l));
  }
  __syncthreads();
  const float mean = bc[0];
  double q = 0.0;
  for (int64_t i = threadIdx.x; i < l; i += blockDim.x) {
    const float d = xr[i] - mean;
    q += d * d;
  }
  q = warpSumD(q);
  __syncthreads();
  if (lane == 0) red[wid] = q;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) t += red[w];
    const float var = static_cast<float>(t / static_cast<double>(l));
    bc[1] = (1.f + gb[ch]) * (1.0f / sqrtf(var + eps));
  }
  __syncthreads();
  const float a = bc[1], b = gb[c + ch];
  float* o = out + ch * l;
  for (int64_t i = threadIdx.x; i < l; i += blockDim.x) o[i] = (xr[i] - mean) * a + b;
}

// One warp per (channel, 128-sample chunk): mean, then M2 = sum (v - mean)^2 from registers.
__global__ void channelStatsKernel(const float* __restrict__ x, float* __restrict__ stats, int64_t l,
                                   int64_t nchunks, int64_t pitch, int64_t statsStride) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t chunk = blockIdx.x * int64_t(blockDim.x >> 5) + wid, ch = blockIdx.y;
  if (chunk >= nchunks) return;
  const int64_t t0 = chunk * kStatChunk;
  const int n = static_cast<int>(l - t0 < kStatChunk ? l - t0 : kStatChunk);
  const float* xr = x + ch * pitch + t0;
  float v[4];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    v[j] = i < n ? xr[i] : 0.f;
    s += v[j];
  }
  s = warpSum(s);
  const float mean = s / static_cast<float>(n);
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float d = (lane + 32 * j) < n ? v[j] - mean : 0.f;
    q = fmaf(d, d, q);
  }
  q = warpSum(q);
  if (lane == 0) {
    float* st = stats + (ch * statsStride + chunk) * 2;
    st[0] = mean;
    st[1] = q;
  }
}

// One 128-thread block per channel: exact combine of the (count, mean, M2) partials in double, two passes. The
// chunk partials of a channel are read once into registers (up to 8 per thread; longer rows loop), so both passes
// cost one round of memory latency.
constexpr int kAffineThreads = 128;
__global__ void __launch_bounds__(kAffineThreads) adainAffineKernel(const float* __restrict__ stats,
                                                                    const float* __restrict__ gb,
                                                                    float* __restrict__ affine, int64_t c, int64_t l,
                                                                    int64_t nchunks, float eps) {
  __shared__ double red[kAffineThreads / 32];
  __shared__ double bc;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t ch = blockIdx.x;
  const float2* sc = reinterpret_cast<const float2*>(stats) + ch * nchunks;  // (mean, M2) pairs, 8-byte aligned
  const double nT = static_cast<double>(kStatChunk), nLast = static_cast<double>(l - (nchunks - 1) * kStatChunk);
  constexpr int R = 8;
  float2 v[R];
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int64_t t = threadIdx.x + int64_t(j) * kAffineThreads;
    v[j] = t < nchunks ? sc[t] : make_float2(0.f, 0.f);
  }
  double sum = 0.0;
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int64_t t = threadIdx.x + int64_t(j) * kAffineThreads;
    if (t < nchunks) sum += static_cast<double>(v[j].x) * (t + 1 < nchunks ? nT : nLast);
  }
  for (int64_t t = threadIdx.x + int64_t(R) * kAffineThreads; t < nchunks; t += kAffineThreads)
    sum += static_cast<double>(sc[t].x) * (t + 1 < nchunks ? nT : nLast);
  sum = warpSumD(sum);
  if (lane == 0) red[wid] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kAffineThreads / 32; ++w) t += red[w];
    bc = t / static_cast<double>(l);
  }
  __syncthreads();
  const double mean = bc;
  double m2 = 0.0;
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int64_t t = threadIdx.x + int64_t(j) * kAffineThreads;
    if (t < nchunks) {
      const double dm = static_cast<double>(v[j].x) - mean;
      m2 += static_cast<double>(v[j].y) + (t + 1 < nchunks ? nT : nLast) * dm * dm;
    }
  }
  for (int64_t t = threadIdx.x + int64_t(R) * kAffineThreads; t < nchunks; t += kAffineThreads) {
    const double dm = static_cast<double>(sc[t].x) - mean;
    m2 += static_cast<double>(sc[t].y) + (t + 1 < nchunks ? nT : nLast) * dm * dm;
  }
  m2 = warpSumD(m2);
  __syncthreads();
  if (lane == 0) red[wid] = m2;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < kAffineThreads / 32; ++w) t += red[w];
    const float m = static_cast<float>(mean), var = static_cast<float>(t / static_cast<double>(l));
    affine[ch] = m;
    affine[c + ch] = (1.f + gb[ch]) * (1.0f / sqrtf(var + eps));
    affine[2 * c + ch] = gb[c + ch];
  }
}

// out[m, n] = sum_k x[m, k] wt[k, n] + b[n]; one thread per output column, coalesced over n. Meant for the
// style bank (M = 1, K = 128).
__global__ void gemmBiasKernel(const float* __restrict__ x, const float* __restrict__ wt, const float* __restrict__ b,
                               float* __restrict__ out, int64_t m, int64_t k, int64_t n) {
  extern __shared__ float xs[];
  const int64_t row = blockIdx.y;
  for (int64_t i = threadIdx.x; i < k; i += blockDim.x) xs[i] = x[row * k + i];
  __syncthreads();
  const int64_t col = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  if (col >= n) return;
  float acc = 0.f;
  for (int64_t i = 0; i < k; ++i) acc = fmaf(xs[i], wt[i * n + col], acc);
  out[row * n + col] = acc + b[col];
}

int64_t numel(const int64_t* dims, int rank) {
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) n *= dims[i];
  return n;
}

// Rank of the operands of an elementwise op with `nOperands` operands and one out, all of the same rank.
int rankOf(const LkcArgs* a, int nOperands) { return static_cast<int>(a->numInts) / (nOperands + 1); }

}  // namespace
}  // namespace lkc

using namespace lkc;

extern "C" LKC_API int lkc_snake_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 3 && a->numInts >= 5, "snake_f32_cuda: expected x, alpha | out");
  const int64_t c = a->ints[0], l = a->ints[1];
  LKC_REQUIRE(a->ints[2] == c, "snake_f32_cuda: alpha must be f32[C]");
  if (c * l == 0) return 0;
  snakeKernel<<<gridFor(c * l), kThreads, 0, S(stream)>>>(F(a, 0), F(a, 1), O(a, 2), c, l);
  return launched("snake_f32_cuda");
}

extern "C" LKC_API int lkc_leaky_relu_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->floats, "leaky_relu_f32_cuda: expected x | out and slope");
  const int64_t n = numel(a->ints, rankOf(a, 1));
  if (n == 0) return 0;
  leakyKernel<<<gridFor(n), kThreads, 0, S(stream)>>>(F(a, 0), O(a, 1), n, static_cast<float>(a->floats[0]));
  return launched("leaky_relu_f32_cuda");
}

extern "C" LKC_API int lkc_add_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 3, "add_f32_cuda: expected a, b | out");
  const int64_t n = numel(a->ints, rankOf(a, 2));
  if (n == 0) return 0;
  addKernel<<<gridFor(n), kThreads, 0, S(stream)>>>(F(a, 0), F(a, 1), O(a, 2), n);
  return launched("add_f32_cuda");
}

extern "C" LKC_API int lkc_add3_scale_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 4 && a->floats, "add3_scale_f32_cuda: expected a, b, c | out and scale");
  const int64_t n = numel(a->ints, rankOf(a, 3));
  if (n == 0) return 0;
  add3ScaleKernel<<<gridFor(n), kThreads, 0, S(stream)>>>(F(a, 0), F(a, 1), F(a, 2), O(a, 3), n,
                                                          static_cast<float>(a->floats[0]));
  return launched("add3_scale_f32_cuda");
}

extern "C" LKC_API int lkc_scale_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->floats, "scale_f32_cuda: expected x | out and scale");
  const int64_t n = numel(a->ints, rankOf(a, 1));
  if (n == 0) return 0;
  scaleKernel<<<gridFor(n), kThreads, 0, S(stream)>>>(F(a, 0), O(a, 1), n, static_cast<float>(a->floats[0]));
  return launched("scale_f32_cuda");
}

extern "C" LKC_API int lkc_pad_reflect1d_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts == 6, "pad_reflect1d_f32_cuda: expected x | out, left, right");
  const int64_t c = a->ints[0], l = a->ints[1], left = a->ints[4], right = a->ints[5];
  LKC_REQUIRE(left >= 0 && right >= 0 && left < l && right < l, "pad_reflect1d_f32_cuda: reflect padding must be < L");
  LKC_REQUIRE(a->ints[3] == l + left + right, "pad_reflect1d_f32_cuda: out must be f32[C, left + L + right]");
  const int64_t n = c * (l + left + right);
  if (n == 0) return 0;
  padReflectKernel<<<gridFor(n), kThreads, 0, S(stream)>>>(F(a, 0), O(a, 1), c, l, left, right);
  return launched("pad_reflect1d_f32_cuda");
}

// Polyphase view of a strided conv's input: y[ci * s + r, t] = x[ci, s t + r - pad] (zero outside [0, L)); rows from
// Ci * s on are zero (channel padding up to the row count of y). A conv with stride s, K = taps * s and padding pad
// over x equals a stride-1 conv with `taps` taps over y with the weights w'[co, ci * s + r, j] = w[co, ci, s j + r],
// which is a shape the tensor-core conv takes. No counterpart in the reference (its strided conv is direct,
// kernels/cpu/kokoro_conv.cpp:32-69).
__global__ void spaceToDepthKernel(const float* __restrict__ x, float* __restrict__ y, int64_t ci, int64_t l,
                                   int64_t rows, int64_t ly, int64_t xPitch, int64_t yPitch, int s, int64_t pad) {
  const int64_t total = rows * ly;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t row = idx / ly, t = idx - row * ly;
    const int64_t c = row / s, r = row - c * s;
    const int64_t pos = int64_t(s) * t + r - pad;
    y[row * yPitch + t] = (c < ci && pos >= 0 && pos < l) ? x[c * xPitch + pos] : 0.f;
  }
}

// ints: x(Ci, L) y(rows, Ly) pad stride [x_pitch y_pitch]
extern "C" LKC_API int lkc_space_to_depth_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && (a->numInts == 6 || a->numInts == 8), "space_to_depth_f32_cuda: expected x | y, pad, stride");
  const int64_t ci = a->ints[0], l = a->ints[1], rows = a->ints[2], ly = a->ints[3], pad = a->ints[4], s = a->ints[5];
  const int64_t xPitch = a->numInts == 8 ? a->ints[6] : l, yPitch = a->numInts == 8 ? a->ints[7] : ly;
  LKC_REQUIRE(s >= 1 && s <= 64 && pad >= 0 && ci >= 1 && l >= 1, "space_to_depth_f32_cuda: invalid stride / padding");
  LKC_REQUIRE(rows >= ci * s && ly >= 1 && yPitch >= ly && xPitch >= l,
              "space_to_depth_f32_cuda: y must be f32[rows >= Ci * stride, Ly]");
  spaceToDepthKernel<<<gridFor(rows * ly, 4), kThreads, 0, S(stream)>>>(F(a, 0), O(a, 1), ci, l, rows, ly, xPitch, yPitch,
                                                                        int(s), pad);
  return launched("space_to_depth_f32_cuda");
}

extern "C" LKC_API int lkc_adain1d_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 3 && a->numInts == 5 && a->floats, "adain1d_f32_cuda: expected x, gb | out and eps");
  const int64_t c = a->ints[0], l = a->ints[1];
  LKC_REQUIRE(a->ints[2] == 2 * c, "adain1d_f32_cuda: gb must be f32[2C]");
  LKC_REQUIRE(l >= 1, "adain1d_f32_cuda: empty sequence");
  if (c == 0) return 0;
  adain1dKernel<<<static_cast<int>(c), kThreads, 0, S(stream)>>>(F(a, 0), F(a, 1), O(a, 2), c, l,
                                                                 static_cast<float>(a->floats[0]));
  return launched("adain1d_f32_cuda");
}

extern "C" LKC_API int lkc_channel_stats_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts >= 5 && a->numInts <= 7, "channel_stats_f32_cuda: expected x | stats");
  const int64_t c = a->ints[0], l = a->ints[1], nchunks = statChunks(l);
  const int64_t pitch = a->numInts >= 6 ? a->ints[5] : l;  // optional trailing ints: row pitch of x, row stride of stats in chunks
  const int64_t statsStride = a->numInts == 7 ? a->ints[6] : nchunks;
  LKC_REQUIRE(pitch >= l && statsStride >= nchunks, "channel_stats_f32_cuda: a row pitch is smaller than the row");
  LKC_REQUIRE(l >= 1, "channel_stats_f32_cuda: empty sequence");
  LKC_REQUIRE(a->ints[2] == c && a->ints[3] == nchunks && a->ints[4] == 2,
              "channel_stats_f32_cuda: stats must be f32[C, ceil(L/128), 2]");
  LKC_REQUIRE(c <= 65535, "channel_stats_f32_cuda: too many channels");
  if (c == 0) return 0;
  dim3 grid(static_cast<unsigned>(ceilDiv(nchunks, kThreads / 32)), static_cast<unsigned>(c));
  channelStatsKernel<<<grid, kThreads, 0, S(stream)>>>(F(a, 0), O(a, 1), l, nchunks, pitch, statsStride);
  return launched("channel_stats_f32_cuda");
}

extern "C" LKC_API int lkc_adain_affine_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 3 && a->numInts == 7 && a->floats,
              "adain_affine_f32_cuda: expected stats, gb | affine, length and eps");
  const int64_t c = a->ints[0], nchunks = a->ints[1], l = a->ints[6];
  LKC_REQUIRE(l >= 1 && nchunks == statChunks(l), "adain_affine_f32_cuda: stats chunks don't match length");
  LKC_REQUIRE(a->ints[3] == 2 * c, "adain_affine_f32_cuda: gb must be f32[2C]");
  LKC_REQUIRE(a->ints[4] == 3 && a->ints[5] == c, "adain_affine_f32_cuda: affine must be f32[3, C]");
  if (c == 0) return 0;
  LKC_REQUIRE(c <= 0x7fffffff, "adain_affine_f32_cuda: too many channels");
  LKC_REQUIRE((reinterpret_cast<uintptr_t>(a->ptrs[0]) & 7) == 0, "adain_affine_f32_cuda: stats must be 8-byte aligned");
  adainAffineKernel<<<static_cast<unsigned>(c), kAffineThreads, 0, S(stream)>>>(F(a, 0), F(a, 1), O(a, 2), c, l, nchunks,
                                                                               static_cast<float>(a->floats[0]));
  return launched("adain_affine_f32_cuda");
}

extern "C" LKC_API int lkc_gemm_bias_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 4 && a->numInts == 7, "gemm_bias_f32_cuda: expected x, wt, b | out");
  const int64_t m = a->ints[0], k = a->ints[1], n = a->ints[3];
  LKC_REQUIRE(a->ints[2] == k && a->ints[4] == n && a->ints[5] == m && a->ints[6] == n,
              "gemm_bias_f32_cuda: shapes must be x[M,K] wt[K,N] b[N] out[M,N]");
  LKC_REQUIRE(k * 4 <= 48 * 1024 && m <= 65535, "gemm_bias_f32_cuda: K or M too large for this kernel");
  if (m * n == 0) return 0;
  dim3 grid(static_cast<unsigned>(ceilDiv(n, kThreads)), static_cast<unsigned>(m));
  gemmBiasKernel<<<grid, kThreads, static_cast<size_t>(k) * 4, S(stream)>>>(F(a, 0), F(a, 1), F(a, 2), O(a, 3), m, k,
                                                                           n);
  return launched("gemm_bias_f32_cuda");
}
