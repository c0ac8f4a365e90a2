// iSTFT tail of the generator: logits [n_fft + 2, L] -> waveform [hop (L - 1)], the contract of the reference's
// istft_logits_f32_cpu:
//   X_k = exp(x[k]) * e^{i sin(x[K + k])}, K = n_fft/2 + 1 bins,
//   frame synthesis y_t[m] = (w[m]/N)(Re X_0 + Re X_{N/2}(-1)^m + 2 sum_{0<k<N/2}(Re X_k cos - Im X_k sin)(2 pi k m/N))
//   out[i] = sum_{t = tLo..tHi} y_t[p - t hop] / sum_t w^2[p - t hop],  p = n_fft/2 + i,
//   tHi = min(L - 1, p / hop), tLo = p >= n_fft ? (p - n_fft)/hop + 1 : 0, frames added in ascending order.
// The window is the periodic Hann window and the synthesis table is built in double, like the reference.
//
// HBM-bound: each block owns FB * hop consecutive output samples, reads the logits of the FB + n_fft/hop frames
// that touch them once (coalesced along time), keeps spectrum, frames and the overlap-add in shared memory and
// writes the samples once.
#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int FB = 128, NTHREADS = 256;

struct IstftArgs {
  const float* x;
  float* out;
  int64_t l, len, pitch;
  int64_t frame0, i0;  // shard: x column 0 is frame frame0 of the l frames, out[0] is sample i0 (len samples from there)
  int nfft, hop, bins, nfMax;
};

__global__ void __launch_bounds__(NTHREADS) istftKernel(const IstftArgs a) {
  extern __shared__ float smem[];
  const int nfft = a.nfft, hop = a.hop, bins = a.bins, nfMax = a.nfMax;
  float* tabRe = smem;                   // [bins][nfft]
  float* tabIm = tabRe + bins * nfft;    // [bins][nfft]
  float* win = tabIm + bins * nfft;      // [nfft]
  float* re = win + nfft;                // [bins][nfMax]
  float* im = re + bins * nfMax;         // [bins][nfMax]
  float* fr = im + bins * nfMax;         // [nfft][nfMax]
  const int tid = threadIdx.x;
  const int64_t iEnd = a.i0 + a.len;
  const int64_t i0 = a.i0 + int64_t(blockIdx.x) * FB * hop;
  const int64_t i1 = (i0 + int64_t(FB) * hop < iEnd) ? i0 + int64_t(FB) * hop : iEnd;
  const int64_t pad = nfft / 2;
  const int64_t pMin = pad + i0, pMax = pad + i1 - 1;
  const int64_t fLo = pMin >= nfft ? (pMin - nfft) / hop + 1 : 0;
  const int64_t fHiRaw = pMax / hop, fHi = fHiRaw < a.l - 1 ? fHiRaw : a.l - 1;
  const int nf = static_cast<int>(fHi - fLo + 1);  // <= nfMax

  const double kPi = 3.14159265358979323846;
  for (int m = tid; m < nfft; m += NTHREADS)
    win[m] = static_cast<float>(0.5 - 0.5 * cos(2.0 * kPi * static_cast<double>(m) / static_cast<double>(nfft)));
  __syncthreads();
  for (int idx = tid; idx < bins * nfft; idx += NTHREADS) {
    const int k = idx / nfft, m = idx - k * nfft;
    const bool edge = k == 0 || 2 * k == nfft;
    const double ang = 2.0 * kPi * static_cast<double>((int64_t(k) * m) % nfft) / static_cast<double>(nfft);
    const double c = (edge ? 1.0 : 2.0) * static_cast<double>(win[m]) / static_cast<double>(nfft);
    tabRe[idx] = static_cast<float>(c * cos(ang));
    tabIm[idx] = edge ? 0.f : static_cast<float>(-c * sin(ang));
  }
  for (int idx = tid; idx < bins * nf; idx += NTHREADS) {
    const int k = idx / nf, f = idx - k * nf;
    const int64_t col = fLo + f - a.frame0;
    const float lm = a.x[int64_t(k) * a.pitch + col], lp = a.x[int64_t(bins + k) * a.pitch + col];
    const float mag = expf(lm), ph = sinf(lp);
    float sn, cs;
    sincosf(ph, &sn, &cs);
    re[k * nfMax + f] = mag * cs;
    im[k * nfMax + f] = mag * sn;
  }
  __syncthreads();
  for (int idx = tid; idx < nfft * nf; idx += NTHREADS) {
    const int m = idx / nf, f = idx - m * nf;
    float v = 0.f;
    for (int k = 0; k < bins; ++k)
      v += re[k * nfMax + f] * tabRe[k * nfft + m] + im[k * nfMax + f] * tabIm[k * nfft + m];
    fr[m * nfMax + f] = v;
  }
  __syncthreads();
  for (int64_t i = i0 + tid; i < i1; i += NTHREADS) {
    const int64_t p = pad + i;
    const int64_t tHiRaw = p / hop, tHi = tHiRaw < a.l - 1 ? tHiRaw : a.l - 1;
    const int64_t tLo = p >= nfft ? (p - nfft) / hop + 1 : 0;
    float y = 0.f, env = 0.f;
    for (int64_t t = tLo; t <= tHi; ++t) {
      const int m = static_cast<int>(p - t * hop);
      y += fr[m * nfMax + static_cast<int>(t - fLo)];
      env += win[m] * win[m];
    }
    a.out[i - a.i0] = y / env;
  }
}

}  // namespace
}  // namespace lkc

using namespace lkc;

extern "C" LKC_API int lkc_istft_logits_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && (a->numInts == 5 || a->numInts == 6 || a->numInts == 9),
              "istft_logits_f32_cuda: expected x | out, hop, n_fft");
  const int64_t rows = a->ints[0], len = a->ints[2], hop = a->ints[3], nfft = a->ints[4];
  // shard extension (ints [x_pitch, frames, frame0, i0]): x holds some of the `frames` frames of the signal, from frame
  // frame0 on, and out receives samples i0 .. i0 + len; the caller provides every frame those samples overlap
  const bool shard = a->numInts == 9;
  const int64_t lx = a->ints[1], l = shard ? a->ints[6] : lx;
  const int64_t frame0 = shard ? a->ints[7] : 0, i0 = shard ? a->ints[8] : 0;
  LKC_REQUIRE(nfft >= 2 && nfft % 2 == 0 && hop >= 1, "istft_logits_f32_cuda: n_fft must be even, hop >= 1");
  LKC_REQUIRE(nfft / 2 + 1 <= 64, "istft_logits_f32_cuda: n_fft too large (at most 126)");
  LKC_REQUIRE(rows == nfft + 2, "istft_logits_f32_cuda: x must be f32[n_fft+2, L]");
  if (!shard) LKC_REQUIRE(l >= 2 && len == hop * (l - 1), "istft_logits_f32_cuda: out must be f32[hop*(L-1)], L >= 2");
  if (shard) {
    LKC_REQUIRE(l >= 2 && len >= 1 && i0 >= 0 && i0 + len <= hop * (l - 1) && frame0 >= 0 && frame0 + lx <= l,
                "istft_logits_f32_cuda: shard out of range");
    const int64_t pFirst = nfft / 2 + i0, pLast = nfft / 2 + i0 + len - 1;
    const int64_t fFirst = pFirst >= nfft ? (pFirst - nfft) / hop + 1 : 0;
    const int64_t fLast = pLast / hop < l - 1 ? pLast / hop : l - 1;
    LKC_REQUIRE(fFirst >= frame0 && fLast < frame0 + lx, "istft_logits_f32_cuda: x does not hold every frame the samples overlap");
  }
  LKC_REQUIRE(hop <= 4096, "istft_logits_f32_cuda: hop out of range");
  IstftArgs p;
  p.x = F(a, 0), p.out = O(a, 1), p.l = l, p.len = len;
  p.pitch = a->numInts >= 6 ? a->ints[5] : lx;  // optional trailing int: row pitch of x
  p.frame0 = frame0, p.i0 = i0;
  LKC_REQUIRE(p.pitch >= lx, "istft_logits_f32_cuda: the row pitch is smaller than the row");
  p.nfft = int(nfft), p.hop = int(hop), p.bins = int(nfft / 2 + 1);
  p.nfMax = int(FB + (nfft + hop - 1) / hop + 2);
  const size_t smem = sizeof(float) * (size_t(2) * p.bins * p.nfft + p.nfft + size_t(2) * p.bins * p.nfMax +
                                       size_t(p.nfft) * p.nfMax);
  LKC_REQUIRE(smem <= 200 * 1024, "istft_logits_f32_cuda: n_fft / hop too large for one block's shared memory");
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(istftKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return failCuda("istft_logits_f32_cuda: cudaFuncSetAttribute", e);
    configured[dev] = true;
  }
  const int64_t blocks = ceilDiv(len, int64_t(FB) * hop);
  LKC_REQUIRE(blocks <= 0x7fffffff, "istft_logits_f32_cuda: grid too large");
  istftKernel<<<static_cast<unsigned>(blocks), NTHREADS, smem, S(stream)>>>(p);
  return launched("istft_logits_f32_cuda");
}
