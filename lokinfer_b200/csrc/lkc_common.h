// Internal helpers shared by the lkc kernel sources: error reporting and argument decoding.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "lkc.h"

namespace lkc {

// Records a failure message for lkc_last_error() and returns 1.
int fail(const char* msg);
int failCuda(const char* what, cudaError_t e);

inline const float* F(const LkcArgs* a, int i) { return static_cast<const float*>(a->ptrs[i]); }
inline float* O(const LkcArgs* a, int i) { return static_cast<float*>(a->ptrs[i]); }
inline cudaStream_t S(void* stream) { return static_cast<cudaStream_t>(stream); }

// Checks the launch that was just issued (no synchronisation).
inline int launched(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return failCuda(what, e);
  }
  return 0;
}

#define LKC_REQUIRE(cond, msg) \
  do {                         \
    if (!(cond)) return ::lkc::fail(msg); \
  } while (0)

constexpr int64_t kStatChunk = 128;
inline int64_t statChunks(int64_t l) { return (l + kStatChunk - 1) / kStatChunk; }
inline int64_t ceilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

enum class Act : int { None = 0, Snake = 1, Leaky = 2 };

// Operands of the fused conv family (one struct for the CUDA-core and the tensor-core kernels).
struct ConvFusedParams {
  const float* x = nullptr;
  const float* x2 = nullptr;  // mean3 prologue: input = ((x + x2) + x3) * inScale
  const float* x3 = nullptr;
  const float* w = nullptr;  // [co, ci, k]
  const float* bias = nullptr;
  const float* affine = nullptr;  // [3, ci] rows mean, scale, beta; null = identity
  const float* alpha = nullptr;
  const float* residual = nullptr;
  float* out = nullptr;
  float* stats = nullptr;  // may be null
  int64_t ci = 0, l = 0, co = 0, k = 0, dilation = 1, padding = 0, lo = 0;
  // Row pitches in floats of the [C, L] tensors x (x2, x3 share it), residual and out; 0 = contiguous rows.
  int64_t xPitch = 0, resPitch = 0, outPitch = 0;
  // Window extension (time-sharded tensors): output column t reads x columns xOrigin + t * stride - padding + kk *
  // dilation; x columns outside [validLo, validHi) count as zero padding (applied after the activation). A regular
  // call has xOrigin = 0 and the valid range [0, l) (validHi < 0 = not set). statsStride = row stride of `stats` in
  // chunks (0 = ceil(lo / 128)): the chunk statistics can be written into a slice of a longer row.
  int64_t xOrigin = 0, validLo = 0, validHi = -1, statsStride = 0;
  Act act = Act::None;
  float slope = 0.f, outScale = 1.f, inScale = 1.f;
  const void* state = nullptr;
};

// One fused conv, routed to the tensor-core kernel when the shape qualifies, else to the CUDA-core kernel (api.cu).
int convFused(const ConvFusedParams& p, cudaStream_t s);
// CUDA-core implicit-GEMM conv for any shape (conv_simt.cu). stride > 1 only for the plain conv1d.
int convSimt(const ConvFusedParams& p, int64_t stride, cudaStream_t s);

// Tensor-core (tcgen05, split operands) fused conv (conv_tc.cu). `state` of ConvFusedParams is an LkcConvState.
struct ConvState {
  const float* wp;  // packed weights (convTcPack / convtTcPack)
  int64_t co, ci, k;
  int64_t stride;  // 0 = conv1d pack; otherwise the ConvTranspose1d stride the pack was made for
  bool f16;        // operand format of the pack: f16 hi/lo split (true) or tf32 hi/lo split (false)
};
// Operands of the polyphase ConvTranspose1d (convt.cu decodes them, conv_tc.cu can run them).
struct ConvtParams {
  const float *x, *bias, *res;
  float* out;
  int64_t ci, l, co, stride, padLeft;
  float slope;
  int64_t xPitch = 0, resPitch = 0, outPitch = 0;  // row pitches in floats; 0 = contiguous rows
  // Window extension: x holds haloLeft / haloRight real columns before / after the l columns that produce output
  // (time-sharded tensors; the zero padding of the transposed conv then applies only where a halo is absent).
  int64_t haloLeft = 0, haloRight = 0;
};
bool convtTcEligible(int64_t ci, int64_t co, int64_t k, int64_t stride, int64_t padding);
int64_t convtTcPackFloats(int64_t ci, int64_t co, int64_t stride, bool f16);
int convtTcPack(const float* w, float* wp, int64_t ci, int64_t co, int64_t k, int64_t stride, int64_t padding, bool f16,
                cudaStream_t s);
int convtTc(const ConvtParams& p, const float* wp, bool f16, cudaStream_t s);
bool convPathForcedSimt();
bool convPackF16();  // operand format new packs are made in (lkc_set_conv_path)
bool convTcEligible(const ConvFusedParams& p, bool f16);
int64_t convTcPackFloats(int64_t co, int64_t ci, int64_t k, bool f16);
int convTcPack(const float* w, float* wp, int64_t co, int64_t ci, int64_t k, bool f16, cudaStream_t s);
int convTc(const ConvFusedParams& p, const float* wp, bool f16, cudaStream_t s);
int convTcStatus(int* out, bool reset);
int convTcStatusAsync(int* hostOut, cudaStream_t s);
int convTcSetIo(int mode);
int convTcProfile(int enable, long long* out16);

}  // namespace lkc
