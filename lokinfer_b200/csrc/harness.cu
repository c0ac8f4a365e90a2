// Test-harness kernels of the reference's RUN2 message (include/lokinfer/remote/server.h:30-47): inputs generated on the
// device from a seed, and outputs compared on the device, so that only a few numbers leave the GPU.
//
//   generate: element i of a tensor uses the splitmix64 values of seed + (2 i + 1) * golden and seed + (2 i + 2) * golden
//             (src/remote/server.cpp:739-782): u = (mix >> 11) * 2^-53; dist 0 normal(a, b) = a + b sqrt(-2 log(1 - u1))
//             cos(2 pi u2), dist 1 uniform [a, b) = a + (b - a) u1, dist 2 integers in [floor a, floor b) = floor(a) +
//             floor(u1 (floor(b) - floor(a))); all in double, then converted to f32 / i32 / i64. Uniform and integer
//             draws are bit-exact against the reference's generator; normals can differ by an ulp of f32 where the
//             device's double log / cos round differently from the host's libm (the reference says the same of its own
//             two implementations, python/lokinfer/remote.py:103-105).
//   compare:  count, nonfinite, mismatches (|got - ref| > atol + rtol |ref|), worst index (largest excess, first on a
//             tie), max |err|, max |ref|, sum of squared errors, sum of squared refs (src/remote/server.cpp:686-736), all
//             in double. A non-finite `got` counts as nonfinite, and as a mismatch unless both are NaN or both the same
//             infinity, and takes no part in the other figures. The sums are taken in a fixed tree order (per thread,
//             per block, then over the blocks), so they are reproducible but not the sequential sums of the reference.
#include <cmath>
#include <cstring>

#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int kBlocks = 296, kThreads = 256;  // two blocks per SM of a B200; any grid gives the same result layout

__device__ __forceinline__ uint64_t splitmix(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) generateKernel(T* out, int64_t n, uint64_t seed, int dist, double a, double b) {
  constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const uint64_t ui = static_cast<uint64_t>(i);
    const double u1 = static_cast<double>(splitmix(seed + (2 * ui + 1) * kGolden) >> 11) * 0x1.0p-53;
    double x;
    if (dist == 0) {
      const double u2 = static_cast<double>(splitmix(seed + (2 * ui + 2) * kGolden) >> 11) * 0x1.0p-53;
      x = a + b * sqrt(-2.0 * log(1.0 - u1)) * cos(6.283185307179586 * u2);
    } else if (dist == 1) {
      x = a + (b - a) * u1;
    } else {
      x = floor(a) + floor(u1 * (floor(b) - floor(a)));
    }
    out[i] = static_cast<T>(x);
  }
}

struct Partial {
  unsigned long long nonfinite, mismatches;
  long long worst;
  double worstExcess, maxErr, maxRef, sse, ssr;
};

__device__ __forceinline__ void merge(Partial& p, const Partial& q) {
  p.nonfinite += q.nonfinite, p.mismatches += q.mismatches;
  // the largest excess wins; on a tie the smaller index (the reference scans upwards and keeps the first)
  if (q.worst >= 0 && (p.worst < 0 || q.worstExcess > p.worstExcess || (q.worstExcess == p.worstExcess && q.worst < p.worst)))
    p.worst = q.worst, p.worstExcess = q.worstExcess;
  p.maxErr = fmax(p.maxErr, q.maxErr), p.maxRef = fmax(p.maxRef, q.maxRef);
  p.sse += q.sse, p.ssr += q.ssr;
}

__device__ __forceinline__ Partial emptyPartial() { return Partial{0, 0, -1, -HUGE_VAL, 0, 0, 0, 0}; }

// Block-level tree merge through shared memory; the result is valid in thread 0.
__device__ Partial blockMerge(Partial p) {
  __shared__ Partial sh[kThreads];
  sh[threadIdx.x] = p;
  __syncthreads();
  for (int step = kThreads / 2; step > 0; step >>= 1) {
    if (int(threadIdx.x) < step) merge(sh[threadIdx.x], sh[threadIdx.x + step]);
    __syncthreads();
  }
  return sh[0];
}

template <typename T>
__global__ void __launch_bounds__(kThreads) comparePartialKernel(const T* got, const T* ref, int64_t n, double rtol,
                                                                double atol, Partial* partials) {
  Partial p = emptyPartial();
  // grid-stride (coalesced): a thread sees its indices in increasing order, and merge() breaks ties by index
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const double g = static_cast<double>(got[i]), r = static_cast<double>(ref[i]);
    if (!isfinite(g)) {
      ++p.nonfinite;
      if (!(isnan(g) && isnan(r)) && g != r) ++p.mismatches;
      continue;
    }
    const double e = fabs(g - r);
    p.maxErr = fmax(p.maxErr, e), p.maxRef = fmax(p.maxRef, fabs(r));
    p.sse += e * e, p.ssr += r * r;
    const double excess = e - (atol + rtol * fabs(r));
    if (excess > 0) ++p.mismatches;
    if (excess > p.worstExcess) p.worstExcess = excess, p.worst = i;
  }
  const Partial b = blockMerge(p);
  if (threadIdx.x == 0) partials[blockIdx.x] = b;
}

// stats: 8 slots of 8 bytes = i64 count, nonfinite, mismatches, worst | f64 max_abs_err, max_abs_ref, sum_sq_err, sum_sq_ref
__global__ void __launch_bounds__(kThreads) compareFinalKernel(const Partial* partials, int numPartials, int64_t n,
                                                              void* stats) {
  Partial p = emptyPartial();
  for (int i = threadIdx.x; i < numPartials; i += kThreads) merge(p, partials[i]);
  const Partial total = blockMerge(p);
  if (threadIdx.x == 0) {
    long long* si = static_cast<long long*>(stats);
    double* sd = reinterpret_cast<double*>(si + 4);
    si[0] = n, si[1] = static_cast<long long>(total.nonfinite), si[2] = static_cast<long long>(total.mismatches);
    si[3] = total.worst;
    sd[0] = total.maxErr, sd[1] = total.maxRef, sd[2] = total.sse, sd[3] = total.ssr;
  }
}

}  // namespace
}  // namespace lkc

using namespace lkc;

// ptrs seed | out: ptrs[0] points at an 8-byte HOST slot with the u64 seed (the reference's packing of scalar
// operands); ints out(1) dtype (0 f32, 1 i32, 2 i64) dist (0 normal, 1 uniform, 2 integers); floats a b.
extern "C" LKC_API int lkc_generate_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts == 3 && a->ptrs[0] && a->floats, "generate_cuda: expected seed | out, dtype, dist, a, b");
  const int64_t n = a->ints[0], dtype = a->ints[1], dist = a->ints[2];
  const double lo = a->floats[0], hi = a->floats[1];
  LKC_REQUIRE(n >= 0 && n <= (int64_t(1) << 28), "generate_cuda: at most 2^28 elements (1 GiB of f32, the reference's limit)");
  LKC_REQUIRE(dtype >= 0 && dtype <= 2, "generate_cuda: generated tensors are f32, i32 or i64");
  LKC_REQUIRE(dist >= 0 && dist <= 2 && std::isfinite(lo) && std::isfinite(hi), "generate_cuda: bad generated distribution");
  LKC_REQUIRE(dist != 2 || (hi > lo && hi - lo < 9.0e15), "generate_cuda: bad generated integer range");
  if (n == 0) return 0;
  uint64_t seed;
  std::memcpy(&seed, a->ptrs[0], sizeof seed);
  const int blocks = int(ceilDiv(n, kThreads) < kBlocks ? ceilDiv(n, kThreads) : kBlocks);
  void* out = const_cast<void*>(a->ptrs[1]);
  if (dtype == 0) generateKernel<float><<<blocks, kThreads, 0, S(stream)>>>(static_cast<float*>(out), n, seed, int(dist), lo, hi);
  else if (dtype == 1) generateKernel<int32_t><<<blocks, kThreads, 0, S(stream)>>>(static_cast<int32_t*>(out), n, seed, int(dist), lo, hi);
  else generateKernel<long long><<<blocks, kThreads, 0, S(stream)>>>(static_cast<long long*>(out), n, seed, int(dist), lo, hi);
  return launched("generate_cuda");
}

// ptrs got ref | stats (64 bytes) workspace (LKC_COMPARE_WORKSPACE_BYTES): ints n dtype (0 f32, 1 i32, 2 i64); floats
// rtol atol.
extern "C" LKC_API int lkc_compare_stats_cuda(const LkcArgs* a, void* stream) {
  static_assert(sizeof(Partial) * kBlocks <= LKC_COMPARE_WORKSPACE_BYTES, "workspace size in the header");
  LKC_REQUIRE(a && a->numPtrs == 4 && a->numInts == 2 && a->floats, "compare_stats_cuda: expected got ref | stats workspace, n, dtype, rtol, atol");
  const int64_t n = a->ints[0], dtype = a->ints[1];
  const double rtol = a->floats[0], atol = a->floats[1];
  LKC_REQUIRE(n >= 0 && dtype >= 0 && dtype <= 2, "compare_stats_cuda: f32, i32 or i64 tensors");
  LKC_REQUIRE(rtol >= 0 && atol >= 0, "compare_stats_cuda: bad tolerance");
  LKC_REQUIRE((n == 0 || (a->ptrs[0] && a->ptrs[1])) && a->ptrs[2] && a->ptrs[3], "compare_stats_cuda: null pointer");
  Partial* ws = static_cast<Partial*>(const_cast<void*>(a->ptrs[3]));
  int blocks = int(ceilDiv(n, kThreads) < kBlocks ? ceilDiv(n, kThreads) : kBlocks);
  if (blocks < 1) blocks = 1;
  if (dtype == 0)
    comparePartialKernel<float><<<blocks, kThreads, 0, S(stream)>>>(static_cast<const float*>(a->ptrs[0]), static_cast<const float*>(a->ptrs[1]), n, rtol, atol, ws);
  else if (dtype == 1)
    comparePartialKernel<int32_t><<<blocks, kThreads, 0, S(stream)>>>(static_cast<const int32_t*>(a->ptrs[0]), static_cast<const int32_t*>(a->ptrs[1]), n, rtol, atol, ws);
  else
    comparePartialKernel<long long><<<blocks, kThreads, 0, S(stream)>>>(static_cast<const long long*>(a->ptrs[0]), static_cast<const long long*>(a->ptrs[1]), n, rtol, atol, ws);
  if (int rc = launched("compare_stats_cuda")) return rc;
  compareFinalKernel<<<1, kThreads, 0, S(stream)>>>(ws, blocks, n, const_cast<void*>(a->ptrs[2]));
  return launched("compare_stats_cuda");
}
