// Producer of the generator's `har` input: Kokoro's harmonic source (SourceModuleHnNSF: sine generator with 9
// harmonics, x300 upsampling, Linear 9 -> 1, tanh) and the STFT that follows it. Contracts of the reference's
// harmonic_source_f32_cpu and stft_magphase_f32_cpu (kernels/cpu/kokoro_signal.cpp:97-272).
//
// harmonic source, f0 f32[n] (one value per 80 Hz frame), noise f32[300 n, 9], w f32[9], b f32[1] -> f32[300 n]:
//   rad[j, h]  = remainder(f0[j] (h + 1) / 24000, 1)                                   (float32)
//   p300[j, h] = ((float32(sum_{j' <= j} rad[j', h]) * 2) * pi) * 300                  (running sum in float64)
//   sample i:  real = max(fma(1/300, i + 0.5, -0.5), 0), i0 = min(floor(real), n - 1), l1 = clamp(real - i0, 0, 1),
//              phase_h = fma(p300[i0, h], 1 - l1, p300[i1, h] * l1), i1 = i0 + (i0 < n - 1)
//              v_h = sin(phase_h) * 0.1 * uv + amp * noise[i, h],  uv = f0[i / 300] > 10, amp = uv ? 0.003 : 0.1 / 3
//              out[i] = tanh(sum_h v_h w[h] + b)                                       (accumulated in harmonic order)
// The phase reaches ~1e6 rad, where one float32 ulp is 0.06 rad: the float32 operation sequence above IS the
// contract, so every rounding is spelled out (__fmul_rn / __fadd_rn / fmaf keep the compiler from re-associating or
// contracting), and the running sum is the reference's sequential float64 loop, one thread per harmonic (a parallel
// scan would round differently in rare cases and move a sample's phase by a whole ulp).
//
// The phase table p300 is scratch memory (n x 9 floats) between the two kernels of the op; the entry point keeps one
// grow-only buffer per device for it.
//
// STFT, x f32[S] -> f32[n_fft + 2, S / hop + 1]: reflect-padded frames times a windowed DFT basis (periodic Hann,
// built in double), re / im accumulated over m = 0..n_fft-1 in order with separate multiply and add, imaginary part
// exactly 0 at DC and Nyquist, rows [0, bins) = sqrt(re^2 + im^2), rows [bins, 2 bins) = atan2(im, re).
// Both are small HBM / latency-bound kernels (one thread per output sample or frame, coalesced along time).
#include <cstring>

#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int kHarmonics = 9;
constexpr int kUp = 300;
constexpr float kSampleRate = 24000.f, kVoicedThreshold = 10.f, kSineAmp = 0.1f, kNoiseStd = 0.003f;

__device__ __forceinline__ float torchRemainder(float a, float b) {
  float m = fmodf(a, b);
  if (m != 0.f && ((b < 0.f) != (m < 0.f))) m += b;
  return m;
}

// One block. Phase 1 (all threads): rad[j, h] into the table. Phase 2 (threads 0..8): the running sum per harmonic.
__global__ void __launch_bounds__(288) harmonicPhaseKernel(const float* __restrict__ f0, float* __restrict__ p300,
                                                           int64_t n) {
  for (int64_t idx = threadIdx.x; idx < n * kHarmonics; idx += blockDim.x) {
    const int64_t j = idx / kHarmonics;
    const int h = int(idx - j * kHarmonics);
    const float fn = __fmul_rn(f0[j], float(h + 1));
    p300[idx] = torchRemainder(__fdiv_rn(fn, kSampleRate), 1.f);
  }
  __syncthreads();
  if (threadIdx.x < kHarmonics) {
    const int h = threadIdx.x;
    double acc = 0.0;
#pragma unroll 8
    for (int64_t j = 0; j < n; ++j) {
      acc += double(p300[j * kHarmonics + h]);
      const float phase = __fmul_rn(__fmul_rn(float(acc), 2.f), 3.14159265358979323846f);
      p300[j * kHarmonics + h] = __fmul_rn(phase, float(kUp));
    }
  }
}

// Counter-based Philox4x32-10 (Salmon et al. 2011), the generator of the reference's in-kernel noise
// (kernels/cpu/kokoro_signal.cpp:42-96): sample i uses counters (i_lo, i_hi, blk, 0x6C6B6E7A) for blk = 0..2 under
// the key (seed_lo, seed_hi); Box-Muller on the word pairs (c0, c1) and (c2, c3) of each block gives its normals
// u1 = (float(c_even) + 0.5) * 2^-32, u2 = float(c_odd) * 2^-32, r = sqrt(-2 ln u1), (r cos(2 pi u2), r sin(2 pi u2));
// the 9 harmonics take the first 9 of the 12. Stateless: the noise depends only on (seed, sample index).
__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t lo0 = c[0] * 0xD2511F53u, hi0 = __umulhi(c[0], 0xD2511F53u);
    const uint32_t lo1 = c[2] * 0xCD9E8D57u, hi1 = __umulhi(c[2], 0xCD9E8D57u);
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0, c[1] = lo1, c[2] = n2, c[3] = lo0;
    k0 += 0x9E3779B9u, k1 += 0xBB67AE85u;
  }
}

__device__ __forceinline__ void philoxNormals(uint64_t seed, int64_t i, float* nz /* kHarmonics */) {
  const uint32_t k0 = uint32_t(seed), k1 = uint32_t(seed >> 32);
#pragma unroll
  for (int blk = 0; blk * 4 < 10; ++blk) {  // kHarmonics + 1 = 10: three blocks
    uint32_t c[4] = {uint32_t(uint64_t(i)), uint32_t(uint64_t(i) >> 32), uint32_t(blk), 0x6C6B6E7Au};
    philox4x32_10(c, k0, k1);
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int id = blk * 4 + 2 * q;
      if (id >= 9) break;
      const float u1 = __fmul_rn(__fadd_rn(__uint2float_rn(c[2 * q]), 0.5f), 2.3283064e-10f);
      const float u2 = __fmul_rn(__uint2float_rn(c[2 * q + 1]), 2.3283064e-10f);
      const float r = sqrtf(__fmul_rn(-2.f, logf(u1)));
      const float t = __fmul_rn(6.2831853f, u2);
      nz[id] = __fmul_rn(r, cosf(t));
      if (id + 1 < 9) nz[id + 1] = __fmul_rn(r, sinf(t));
    }
  }
}

// RNG = false: the noise is the operand `noise` f32[300 n, 9]; RNG = true: it is drawn in the kernel from `seed`.
template <bool RNG>
__global__ void __launch_bounds__(256) harmonicSourceKernel(const float* __restrict__ f0, const float* __restrict__ noise,
                                                            uint64_t seed, const float* __restrict__ w,
                                                            const float* __restrict__ b,
                                                            const float* __restrict__ p300, float* __restrict__ out,
                                                            int64_t n) {
  const int64_t s = n * kUp;
  const float scale = float(1.0 / double(kUp));
  const float ampV = kNoiseStd, ampU = __fdiv_rn(__fmul_rn(1.f, kSineAmp), 3.f);
  float wr[kHarmonics];
#pragma unroll
  for (int h = 0; h < kHarmonics; ++h) wr[h] = w[h];
  const float bias = b[0];
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < s; i += int64_t(gridDim.x) * blockDim.x) {
    float real = fmaf(scale, __fadd_rn(float(i), 0.5f), -0.5f);
    real = fmaxf(real, 0.f);
    int64_t i0 = int64_t(floorf(real));
    if (i0 > n - 1) i0 = n - 1;
    const float l1 = fminf(fmaxf(__fsub_rn(real, float(i0)), 0.f), 1.f);
    const float l0 = __fsub_rn(1.f, l1);
    const int64_t i1 = i0 + (i0 < n - 1 ? 1 : 0);
    const bool voiced = f0[i / kUp] > kVoicedThreshold;
    const float uv = voiced ? 1.f : 0.f, amp = voiced ? ampV : ampU;
    const float* r0 = p300 + i0 * kHarmonics;
    const float* r1 = p300 + i1 * kHarmonics;
    float nzr[kHarmonics];
    const float* nz = nzr;
    if constexpr (RNG) philoxNormals(seed, i, nzr);
    else nz = noise + i * kHarmonics;
    float y = 0.f;
#pragma unroll
    for (int h = 0; h < kHarmonics; ++h) {
      const float phase = fmaf(r0[h], l0, __fmul_rn(r1[h], l1));
      const float sine = __fmul_rn(sinf(phase), kSineAmp);
      const float v = __fadd_rn(__fmul_rn(sine, uv), __fmul_rn(amp, nz[h]));
      y = __fadd_rn(y, __fmul_rn(v, wr[h]));
    }
    out[i] = tanhf(__fadd_rn(y, bias));
  }
}

constexpr int kMaxFft = 64;  // the windowed basis (2 x bins x n_fft floats) lives in shared memory

__global__ void __launch_bounds__(256) stftMagphaseKernel(const float* __restrict__ x, float* __restrict__ out, int64_t s,
                                                          int nfft, int hop, int64_t frames) {
  extern __shared__ float tab[];  // [bins][nfft] re, then [bins][nfft] im
  const int bins = nfft / 2 + 1;
  for (int idx = threadIdx.x; idx < bins * nfft; idx += blockDim.x) {
    const int k = idx / nfft, m = idx - k * nfft;
    const float win = float(0.5 - 0.5 * cos(2.0 * 3.14159265358979323846 * double(m) / double(nfft)));
    const double ang = 2.0 * 3.14159265358979323846 * double((k * m) % nfft) / double(nfft);
    tab[idx] = float(double(win) * cos(ang));
    tab[bins * nfft + idx] = float(-double(win) * sin(ang));
  }
  __syncthreads();
  const int64_t pad = nfft / 2;
  float* mag = out;
  float* ph = out + int64_t(bins) * frames;
  for (int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; t < frames; t += int64_t(gridDim.x) * blockDim.x) {
    float fr[kMaxFft];
#pragma unroll 4
    for (int m = 0; m < nfft; ++m) {
      int64_t q = t * hop + m - pad;  // reflect pad
      if (q < 0) q = -q;
      if (q >= s) q = 2 * (s - 1) - q;
      fr[m] = x[q];
    }
    for (int k = 0; k < bins; ++k) {
      const float* cr = tab + k * nfft;
      const float* ci = cr + bins * nfft;
      float re = 0.f, im = 0.f;
      for (int m = 0; m < nfft; ++m) {
        re = __fadd_rn(re, __fmul_rn(fr[m], cr[m]));
        im = __fadd_rn(im, __fmul_rn(fr[m], ci[m]));
      }
      if (k == 0 || 2 * k == nfft) im = 0.f;  // real input: exactly +0 at DC / Nyquist
      mag[k * frames + t] = sqrtf(fmaf(im, im, __fmul_rn(re, re)));
      ph[k * frames + t] = atan2f(im, re);
    }
  }
}

// Grow-only phase-table scratch, one buffer per device (allocated on first use and whenever n grows: that call must
// not be inside a stream capture; calls on one device that overlap in time would share the table and race).
float* phaseScratch(int64_t floats) {
  static float* buf[64] = {};
  static int64_t cap[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cap[dev] < floats) {
    if (buf[dev]) cudaFree(buf[dev]);
    buf[dev] = nullptr, cap[dev] = 0;
    int64_t want = floats < 4096 ? 4096 : floats;
    float* p = nullptr;
    if (cudaMalloc(&p, size_t(want) * sizeof(float)) != cudaSuccess) return nullptr;
    buf[dev] = p, cap[dev] = want;
  }
  return buf[dev];
}

}  // namespace

// noise != null: the noise operand; noise == null: drawn in the kernel from seed.
int harmonicSourceLaunch(const float* f0, const float* noise, uint64_t seed, const float* w, const float* b, float* p300,
                         float* out, int64_t n, cudaStream_t s) {
  harmonicPhaseKernel<<<1, 288, 0, s>>>(f0, p300, n);
  const int64_t samples = n * kUp;
  const int blocks = int(ceilDiv(samples, 256) > 148 * 16 ? 148 * 16 : ceilDiv(samples, 256));
  if (noise) harmonicSourceKernel<false><<<blocks, 256, 0, s>>>(f0, noise, 0, w, b, p300, out, n);
  else harmonicSourceKernel<true><<<blocks, 256, 0, s>>>(f0, nullptr, seed, w, b, p300, out, n);
  return launched("harmonic_source_f32_cuda");
}

}  // namespace lkc

using namespace lkc;

extern "C" LKC_API int lkc_harmonic_source_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 5 && a->numInts == 6, "harmonic_source_f32_cuda: expected f0 noise w b | out");
  const int64_t n = a->ints[0];
  LKC_REQUIRE(n >= 1 && n <= (int64_t(1) << 23) / kUp, "harmonic_source_f32_cuda: f0 must be f32[n], 1 <= n <= 27962");
  LKC_REQUIRE(a->ints[1] == n * kUp && a->ints[2] == kHarmonics, "harmonic_source_f32_cuda: noise must be f32[300n, 9]");
  LKC_REQUIRE(a->ints[3] == kHarmonics && a->ints[4] == 1, "harmonic_source_f32_cuda: w must be f32[9], b f32[1]");
  LKC_REQUIRE(a->ints[5] == n * kUp, "harmonic_source_f32_cuda: out must be f32[300n]");
  float* p300 = phaseScratch(n * kHarmonics);
  LKC_REQUIRE(p300 != nullptr, "harmonic_source_f32_cuda: cannot allocate the phase table");
  return harmonicSourceLaunch(F(a, 0), F(a, 1), 0, F(a, 2), F(a, 3), p300, O(a, 4), n, S(stream));
}

// operands f0(n), w(9), b(1), seed (an i64 scalar: ptrs[3] points at an 8-byte HOST slot, as the reference packs
// scalars); out(300 n). ints: f0, w, b, out shapes (kernels/cpu/kokoro_signal.cpp:375-380).
extern "C" LKC_API int lkc_harmonic_source_rng_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 5 && a->numInts == 4 && a->ptrs[3], "harmonic_source_rng_f32_cuda: expected f0 w b seed | out");
  const int64_t n = a->ints[0];
  LKC_REQUIRE(n >= 1 && n <= (int64_t(1) << 23) / kUp, "harmonic_source_rng_f32_cuda: f0 must be f32[n], 1 <= n <= 27962");
  LKC_REQUIRE(a->ints[1] == kHarmonics && a->ints[2] == 1, "harmonic_source_rng_f32_cuda: w must be f32[9], b f32[1]");
  LKC_REQUIRE(a->ints[3] == n * kUp, "harmonic_source_rng_f32_cuda: out must be f32[300n]");
  int64_t seed;
  std::memcpy(&seed, a->ptrs[3], sizeof seed);
  float* p300 = phaseScratch(n * kHarmonics);
  LKC_REQUIRE(p300 != nullptr, "harmonic_source_rng_f32_cuda: cannot allocate the phase table");
  return harmonicSourceLaunch(F(a, 0), nullptr, static_cast<uint64_t>(seed), F(a, 1), F(a, 2), p300, O(a, 4), n,
                              S(stream));
}

extern "C" LKC_API int lkc_stft_magphase_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts == 5, "stft_magphase_f32_cuda: expected x | out, hop, n_fft");
  const int64_t s = a->ints[0], rows = a->ints[1], frames = a->ints[2], hop = a->ints[3], nfft = a->ints[4];
  LKC_REQUIRE(nfft >= 2 && nfft % 2 == 0 && hop >= 1, "stft_magphase_f32_cuda: n_fft must be even, hop >= 1");
  LKC_REQUIRE(nfft <= kMaxFft, "stft_magphase_f32_cuda: n_fft too large (at most 64)");
  LKC_REQUIRE(s >= nfft / 2 + 1, "stft_magphase_f32_cuda: signal must be longer than n_fft/2 (reflect pad)");
  LKC_REQUIRE(rows == nfft + 2 && frames == s / hop + 1, "stft_magphase_f32_cuda: out must be f32[n_fft+2, S/hop+1]");
  const int bins = int(nfft / 2 + 1);
  const size_t smem = sizeof(float) * size_t(2) * bins * nfft;
  const int blocks = int(ceilDiv(frames, 256) > 148 * 8 ? 148 * 8 : ceilDiv(frames, 256));
  stftMagphaseKernel<<<blocks, 256, smem, S(stream)>>>(F(a, 0), O(a, 1), s, int(nfft), int(hop), frames);
  return launched("stft_magphase_f32_cuda");
}

// ---- the same op for callers that must not allocate --------------------------------------------------------------
// lkc_harmonic_source_noalloc_f32_cuda runs the two kernels above with the phase table in a fixed array of this
// module instead of the grow-only cudaMalloc buffer: no cudaMalloc / cudaFree / allocating library call on any path.
// Limit: kNoAllocMaxFrames frames (51 s of audio at 80 frames/s; the table is 144 KB of device memory that exists
// whether or not the entry point is used). Larger inputs are rejected. Nothing has to start at zero: the first kernel
// writes every table element the second one reads. The first call on a device looks the array's address up
// (cudaGetSymbolAddress) and should come before any stream capture; calls on one device share the array, so two
// calls that overlap in time (different streams) race on it.
namespace lkc {
namespace {
constexpr int64_t kNoAllocMaxFrames = 4096;
static __device__ __align__(256) float gPhaseTable[kNoAllocMaxFrames * kHarmonics];
}  // namespace
}  // namespace lkc

extern "C" LKC_API int lkc_harmonic_source_noalloc_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 5 && a->numInts == 6, "harmonic_source_noalloc_f32_cuda: expected f0 noise w b | out");
  const int64_t n = a->ints[0];
  LKC_REQUIRE(n >= 1 && n <= kNoAllocMaxFrames, "harmonic_source_noalloc_f32_cuda: f0 must be f32[n], 1 <= n <= 4096");
  LKC_REQUIRE(a->ints[1] == n * kUp && a->ints[2] == kHarmonics,
              "harmonic_source_noalloc_f32_cuda: noise must be f32[300n, 9]");
  LKC_REQUIRE(a->ints[3] == kHarmonics && a->ints[4] == 1, "harmonic_source_noalloc_f32_cuda: w must be f32[9], b f32[1]");
  LKC_REQUIRE(a->ints[5] == n * kUp, "harmonic_source_noalloc_f32_cuda: out must be f32[300n]");
  static float* table[64] = {};  // per device, looked up once
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return failCuda("harmonic_source_noalloc_f32_cuda: cudaGetDevice", e);
  LKC_REQUIRE(dev >= 0 && dev < 64, "harmonic_source_noalloc_f32_cuda: device index out of range");
  if (!table[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), gPhaseTable);
    if (e != cudaSuccess) return failCuda("harmonic_source_noalloc_f32_cuda: cudaGetSymbolAddress", e);
    table[dev] = ptr;
  }
  return harmonicSourceLaunch(F(a, 0), F(a, 1), 0, F(a, 2), F(a, 3), table[dev], O(a, 4), n, S(stream));
}
