// The three small ops the decoder's AdainResBlk1d stack needs besides the fused conv family (the producer of the
// generator's input x [512, 2F], models/kokoro/model.py:158-221, 704-717): depthwise ConvTranspose1d (the "pool" of the
// upsampling block), nearest-neighbour upsampling of the shortcut, and the row concatenation that builds the block
// inputs. All three are memory-bound data movement with lanes along time.
#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int kThreads = 256;

inline int gridFor(int64_t n) {
  const int64_t b = ceilDiv(n, kThreads);
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 32 ? 148 * 32 : b));
}

// out[c, q] = bias[c] + sum_j x[c, j] w[c, q + p - j s], j ascending over the taps that exist: the gather form of the
// reference (kernels/cpu/kokoro_conv.cpp:97-117), same accumulation order.
__global__ void convtDwKernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                              float* __restrict__ out, int64_t c, int64_t l, int64_t lo, int k, int stride, int padding) {
  const int64_t total = c * lo;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t ch = idx / lo, q = idx - ch * lo;
    const int64_t t = q + padding;
    int64_t jHi = t / stride;
    if (jHi > l - 1) jHi = l - 1;
    const int64_t jLo = t - (k - 1) <= 0 ? 0 : (t - (k - 1) + stride - 1) / stride;
    const float* xr = x + ch * l;
    const float* wr = w + ch * k;
    float v = bias ? bias[ch] : 0.f;
    for (int64_t j = jLo; j <= jHi; ++j) v = fmaf(xr[j], wr[t - j * stride], v);
    out[idx] = v;
  }
}

__global__ void upsampleNearestKernel(const float* __restrict__ x, float* __restrict__ out, int64_t c, int64_t l,
                                      int64_t scale) {
  const int64_t lo = l * scale, total = c * lo;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
    const int64_t ch = idx / lo, q = idx - ch * lo;
    out[idx] = x[ch * l + q / scale];
  }
}

struct ConcatArgs {
  const float* xs[8];
  int64_t start[9];  // first output element of each operand, then the total
  int n;
};

__global__ void concatRowsKernel(const ConcatArgs a, float* __restrict__ out) {
  const int64_t total = a.start[a.n];
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
    int i = 0;
    while (i + 1 < a.n && idx >= a.start[i + 1]) ++i;
    out[idx] = a.xs[i][idx - a.start[i]];
  }
}

}  // namespace
}  // namespace lkc

using namespace lkc;

// ints: x(C, L) w(C, 1, K) b(C) out(C, Lo) output_padding padding stride
extern "C" LKC_API int lkc_conv_transpose1d_dw_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 4 && a->numInts == 11, "conv_transpose1d_dw_f32_cuda: expected x w b | out");
  const int64_t* n = a->ints;
  const int64_t c = n[0], l = n[1], k = n[4], op = n[8], p = n[9], s = n[10];
  LKC_REQUIRE(n[2] == c && n[3] == 1 && n[5] == c, "conv_transpose1d_dw_f32_cuda: w must be [C, 1, K], bias f32[C]");
  LKC_REQUIRE(s >= 1 && p >= 0 && op >= 0 && op < s && k >= 1 && k <= 4096 && s <= 4096,
              "conv_transpose1d_dw_f32_cuda: invalid stride/padding/output_padding");
  const int64_t lo = (l - 1) * s - 2 * p + k + op;
  LKC_REQUIRE(l >= 1 && lo >= 1, "conv_transpose1d_dw_f32_cuda: empty conv_transpose output");
  LKC_REQUIRE(n[6] == c && n[7] == lo, "conv_transpose1d_dw_f32_cuda: out must be f32[C, Lo]");
  if (c == 0) return 0;
  convtDwKernel<<<gridFor(c * lo), kThreads, 0, S(stream)>>>(F(a, 0), F(a, 1), F(a, 2), O(a, 3), c, l, lo, int(k), int(s),
                                                             int(p));
  return launched("conv_transpose1d_dw_f32_cuda");
}

// ints: x(C, L) out(C, L * scale) scale
extern "C" LKC_API int lkc_upsample_nearest1d_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts == 5, "upsample_nearest1d_f32_cuda: expected x | out, scale");
  const int64_t c = a->ints[0], l = a->ints[1], scale = a->ints[4];
  LKC_REQUIRE(scale >= 1, "upsample_nearest1d_f32_cuda: scale must be >= 1");
  LKC_REQUIRE(a->ints[2] == c && a->ints[3] == l * scale, "upsample_nearest1d_f32_cuda: out must be f32[C, L * scale]");
  if (c * l == 0) return 0;
  upsampleNearestKernel<<<gridFor(c * l * scale), kThreads, 0, S(stream)>>>(F(a, 0), O(a, 1), c, l, scale);
  return launched("upsample_nearest1d_f32_cuda");
}

// ints: x_i(R_i, C) for each input, out(sum R, C)
extern "C" LKC_API int lkc_concat_rows_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs >= 3 && a->numPtrs <= 9 && a->numInts == 2 * a->numPtrs,
              "concat_rows_f32_cuda: concat takes 2..8 operands");
  const int nin = int(a->numPtrs) - 1;
  const int64_t cols = a->ints[1];
  ConcatArgs ca;
  int64_t rows = 0;
  for (int i = 0; i < nin; ++i) {
    LKC_REQUIRE(a->ints[2 * i + 1] == cols && a->ints[2 * i] >= 0, "concat_rows_f32_cuda: column counts differ");
    ca.xs[i] = F(a, i);
    ca.start[i] = rows * cols;
    rows += a->ints[2 * i];
  }
  ca.start[nin] = rows * cols, ca.n = nin;
  LKC_REQUIRE(a->ints[2 * nin] == rows && a->ints[2 * nin + 1] == cols, "concat_rows_f32_cuda: out must be f32[sum R, C]");
  if (rows * cols == 0) return 0;
  concatRowsKernel<<<gridFor(rows * cols), kThreads, 0, S(stream)>>>(ca, O(a, nin));
  return launched("concat_rows_f32_cuda");
}
