// C-ABI entry points of the conv family, the kernel registry and error reporting.
#include <algorithm>
#include <cstring>
#include <new>

#include "lkc_common.h"

namespace lkc {

namespace {
thread_local char gError[512] = "";
}

int fail(const char* msg) {
  std::snprintf(gError, sizeof gError, "%s", msg);
  return 1;
}

int failCuda(const char* what, cudaError_t e) {
  std::snprintf(gError, sizeof gError, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return 2;
}

namespace {

// conv1d_{act}[_res]_f32_cuda(x, w, b, affine, [alpha,] [res]) outs(out, stats): the reference adapter's packing
// (runConvFused): ints x(Ci, L) w(Co, Ci, K) b(Co) affine(3, Ci) [alpha(Ci)] [res(Co, Lo)] out(Co, Lo)
// stats(Co, S, 2) dilation padding tile; floats [oscale] [slope].
int runConvFused(const LkcArgs* a, void* stream, Act act, bool res, const char* name) {
  const bool hasAlpha = act == Act::Snake;
  const uint32_t nptr = 4 + (hasAlpha ? 1 : 0) + (res ? 1 : 0) + 2;
  const uint32_t nint = 8 + (hasAlpha ? 1 : 0) + (res ? 2 : 0) + 2 + 3 + 3;
  // optional trailing ints: row pitches of x, [res,] out; then the window extension stats_chunks, x_origin, valid_lo,
  // valid_hi (see lkc.h)
  const uint32_t npitch = res ? 3 : 2, nwin = 4;
  if (!a || a->numPtrs != nptr ||
      (a->numInts != nint && a->numInts != nint + npitch && a->numInts != nint + npitch + nwin)) {
    std::snprintf(gError, sizeof gError, "%s: expected %u pointers and %u ints (+ %u row pitches (+ %u window ints))",
                  name, nptr, nint, npitch, nwin);
    return 1;
  }
  const int64_t* n = a->ints;
  ConvFusedParams p;
  p.x = F(a, 0), p.w = F(a, 1), p.bias = F(a, 2), p.affine = F(a, 3);
  int pi = 4, ni = 8;
  if (hasAlpha) {
    p.alpha = F(a, pi++);
    LKC_REQUIRE(n[ni] == n[0], "conv1d fused: alpha must be f32[Ci]");
    ni += 1;
  }
  const int64_t* resDims = nullptr;
  if (res) {
    p.residual = F(a, pi++);
    resDims = n + ni;
    ni += 2;
  }
  p.out = O(a, pi++);
  p.stats = O(a, pi++);
  p.ci = n[0], p.l = n[1], p.co = n[2], p.k = n[4];
  const int64_t* outDims = n + ni;
  const int64_t* stDims = n + ni + 2;
  p.dilation = n[ni + 5], p.padding = n[ni + 6];  // n[ni + 7] = tile: accepted, unused
  p.act = act;
  LKC_REQUIRE(n[3] == p.ci, "conv1d fused: w must be [Co, Ci, K]");
  LKC_REQUIRE(n[5] == p.co, "conv1d fused: bias must be f32[Co]");
  LKC_REQUIRE(n[6] == 3 && n[7] == p.ci, "conv1d fused: affine must be f32[3, Ci]");
  LKC_REQUIRE(p.dilation >= 1 && p.padding >= 0 && p.k >= 1, "conv1d fused: invalid padding/dilation");
  const bool window = a->numInts == nint + npitch + nwin;
  if (window) {
    // x is a window into a longer row: the output length is given by `out`, x columns outside [valid_lo, valid_hi)
    // are the zero padding
    const int64_t* wn = n + nint + npitch;
    p.statsStride = wn[0], p.xOrigin = wn[1], p.validLo = wn[2], p.validHi = wn[3];
    p.lo = outDims[1];
    LKC_REQUIRE(p.xOrigin >= 0 && p.xOrigin <= p.l && p.validLo >= 0 && p.validHi <= p.l && p.validLo <= p.validHi,
                "conv1d fused: window out of range");
    LKC_REQUIRE(p.statsStride >= statChunks(p.lo), "conv1d fused: stats row stride is smaller than the row");
  } else {
    p.lo = p.l + 2 * p.padding - p.dilation * (p.k - 1);
  }
  LKC_REQUIRE(p.lo >= 1, "conv1d fused: empty conv output");
  LKC_REQUIRE(outDims[0] == p.co && outDims[1] == p.lo, "conv1d fused: out must be f32[Co, Lo]");
  LKC_REQUIRE(stDims[0] == p.co && stDims[1] == statChunks(p.lo) && stDims[2] == 2,
              "conv1d fused: stats must be f32[Co, ceil(Lo/128), 2]");
  if (res) LKC_REQUIRE(resDims[0] == p.co && resDims[1] == p.lo, "conv1d fused: residual must match the output");
  if (a->numInts >= nint + npitch) {
    const int64_t* pt = n + nint;
    p.xPitch = pt[0], p.resPitch = res ? pt[1] : 0, p.outPitch = pt[npitch - 1];
    LKC_REQUIRE(p.xPitch >= p.l && p.outPitch >= p.lo && (!res || p.resPitch >= p.lo),
                "conv1d fused: a row pitch is smaller than the row");
  }
  int fi = 0;
  if (act == Act::Leaky) LKC_REQUIRE(a->floats, "conv1d fused: missing float attributes");
  if (res && act == Act::Leaky) p.outScale = static_cast<float>(a->floats[fi++]);
  if (act == Act::Leaky) p.slope = static_cast<float>(a->floats[fi++]);
  p.state = a->state;
  return convFused(p, S(stream));
}

int runConv1d(const LkcArgs* a, void* stream, bool bias) {
  const uint32_t nptr = bias ? 4 : 3, nint = bias ? 11 : 10;
  LKC_REQUIRE(a && a->numPtrs == nptr && (a->numInts == nint || a->numInts == nint + 2 || a->numInts == nint + 5),
              "conv1d_f32_cuda: bad operand count");
  const int64_t* n = a->ints;
  ConvFusedParams p;
  p.x = F(a, 0), p.w = F(a, 1);
  p.bias = bias ? F(a, 2) : nullptr;
  p.out = O(a, bias ? 3 : 2);
  p.ci = n[0], p.l = n[1], p.co = n[2], p.k = n[4];
  const int at = bias ? 8 : 7;
  p.dilation = n[at], p.padding = n[at + 1];
  const int64_t stride = n[at + 2];
  LKC_REQUIRE(n[3] == p.ci, "conv1d_f32_cuda: w must be [Co, Ci, K]");
  if (bias) LKC_REQUIRE(n[5] == p.co, "conv1d_f32_cuda: bias must be f32[Co]");
  LKC_REQUIRE(stride >= 1 && p.dilation >= 1 && p.padding >= 0 && p.k >= 1,
              "conv1d_f32_cuda: invalid stride/padding/dilation");
  if (a->numInts == nint + 5) {  // window extension: x_origin, valid_lo, valid_hi; the output length is given by `out`
    p.xOrigin = n[nint + 2], p.validLo = n[nint + 3], p.validHi = n[nint + 4];
    p.lo = n[at - 1];
    LKC_REQUIRE(p.xOrigin >= 0 && p.validLo >= 0 && p.validHi <= p.l && p.validLo <= p.validHi && p.lo >= 1,
                "conv1d_f32_cuda: window out of range");
  } else {
    const int64_t span = p.l + 2 * p.padding - p.dilation * (p.k - 1) - 1;
    LKC_REQUIRE(span >= 0, "conv1d_f32_cuda: empty conv output");
    p.lo = span / stride + 1;
  }
  LKC_REQUIRE(n[at - 2] == p.co && n[at - 1] == p.lo, "conv1d_f32_cuda: out must be f32[Co, Lo]");
  if (a->numInts >= nint + 2) {  // optional trailing ints: row pitches of x and out
    p.xPitch = n[nint], p.outPitch = n[nint + 1];
    LKC_REQUIRE(p.xPitch >= p.l && p.outPitch >= p.lo, "conv1d_f32_cuda: a row pitch is smaller than the row");
  }
  return convSimt(p, stride, S(stream));
}

struct Entry {
  const char* name;
  LkcRunFn fn;
};

}  // namespace

// Routes one fused conv to the tensor-core kernel when the shape qualifies, else to the CUDA-core kernel.
namespace {
int gConvPath = 0;  // 0 = tensor cores, f16 split packs; 1 = CUDA-core kernel only; 2 = tensor cores, tf32 split packs
}

bool convPathForcedSimt() { return gConvPath == 1; }
bool convPackF16() { return gConvPath != 2; }

int convFused(const ConvFusedParams& p, cudaStream_t s) {
  if (gConvPath != 1 && p.state != nullptr) {
    const ConvState* st = static_cast<const ConvState*>(p.state);
    LKC_REQUIRE(st->wp && st->stride == 0 && st->co == p.co && st->ci == p.ci && st->k == p.k,
                "conv1d fused: the prepared state does not match the weight shape");
    if (convTcEligible(p, st->f16)) return convTc(p, st->wp, st->f16, s);
  }
  return convSimt(p, 1, s);
}

}  // namespace lkc

using namespace lkc;

extern "C" LKC_API int lkc_conv1d_snake_f32_cuda(const LkcArgs* a, void* s) {
  return runConvFused(a, s, Act::Snake, false, "conv1d_snake_f32_cuda");
}
extern "C" LKC_API int lkc_conv1d_snake_res_f32_cuda(const LkcArgs* a, void* s) {
  return runConvFused(a, s, Act::Snake, true, "conv1d_snake_res_f32_cuda");
}
extern "C" LKC_API int lkc_conv1d_leaky_f32_cuda(const LkcArgs* a, void* s) {
  return runConvFused(a, s, Act::Leaky, false, "conv1d_leaky_f32_cuda");
}
extern "C" LKC_API int lkc_conv1d_leaky_res_f32_cuda(const LkcArgs* a, void* s) {
  return runConvFused(a, s, Act::Leaky, true, "conv1d_leaky_res_f32_cuda");
}
extern "C" LKC_API int lkc_conv1d_affine_f32_cuda(const LkcArgs* a, void* s) {
  return runConvFused(a, s, Act::None, false, "conv1d_affine_f32_cuda");
}

// ints: x(2) x2(2) x3(2) w(3) b(1) affine(2) out(2) stats(3) dilation padding tile; floats in_scale slope.
extern "C" LKC_API int lkc_conv1d_leaky_mean3_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 8 && a->numInts == 20 && a->floats, "conv1d_leaky_mean3_f32_cuda: bad operand count");
  const int64_t* n = a->ints;
  ConvFusedParams p;
  p.x = F(a, 0), p.x2 = F(a, 1), p.x3 = F(a, 2), p.w = F(a, 3), p.bias = F(a, 4), p.affine = F(a, 5);
  p.out = O(a, 6), p.stats = O(a, 7);
  p.ci = n[0], p.l = n[1], p.co = n[6], p.k = n[8];
  LKC_REQUIRE(n[2] == p.ci && n[3] == p.l && n[4] == p.ci && n[5] == p.l,
              "conv1d_leaky_mean3_f32_cuda: x2 / x3 must match x");
  LKC_REQUIRE(n[7] == p.ci && n[9] == p.co && n[10] == 3 && n[11] == p.ci,
              "conv1d_leaky_mean3_f32_cuda: w must be [Co, Ci, K], b f32[Co], affine f32[3, Ci]");
  p.dilation = n[17], p.padding = n[18];
  LKC_REQUIRE(p.dilation >= 1 && p.padding >= 0 && p.k >= 1, "conv1d_leaky_mean3_f32_cuda: invalid padding/dilation");
  p.lo = p.l + 2 * p.padding - p.dilation * (p.k - 1);
  LKC_REQUIRE(p.lo >= 1, "conv1d_leaky_mean3_f32_cuda: empty conv output");
  LKC_REQUIRE(n[12] == p.co && n[13] == p.lo && n[14] == p.co && n[15] == statChunks(p.lo) && n[16] == 2,
              "conv1d_leaky_mean3_f32_cuda: out must be f32[Co, Lo], stats f32[Co, ceil(Lo/128), 2]");
  p.act = Act::Leaky;
  p.inScale = static_cast<float>(a->floats[0]);
  p.slope = static_cast<float>(a->floats[1]);
  p.state = a->state;
  return convFused(p, S(stream));
}

extern "C" LKC_API int lkc_conv1d_f32_cuda(const LkcArgs* a, void* s) { return runConv1d(a, s, true); }
extern "C" LKC_API int lkc_conv1d_nobias_f32_cuda(const LkcArgs* a, void* s) { return runConv1d(a, s, false); }

// ints: w(Co, Ci, K) wp(n)
extern "C" LKC_API int lkc_conv1d_tc_pack_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts == 4, "conv1d_tc_pack_f32_cuda: expected w | wp");
  const int64_t co = a->ints[0], ci = a->ints[1], k = a->ints[2];
  LKC_REQUIRE(co > 0 && ci > 0 && ci % 16 == 0 && k >= 1 && k <= 64,
              "conv1d_tc_pack_f32_cuda: needs Ci % 16 == 0, 1 <= K <= 64");
  LKC_REQUIRE(a->ints[3] == convTcPackFloats(co, ci, k, convPackF16()),
              "conv1d_tc_pack_f32_cuda: wp must hold lkc_conv1d_tc_pack_floats (of the current operand format)");
  return convTcPack(F(a, 0), O(a, 1), co, ci, k, convPackF16(), S(stream));
}

extern "C" LKC_API int64_t lkc_conv1d_tc_pack_floats(int64_t co, int64_t ci, int64_t k) {
  if (co <= 0 || ci <= 0 || ci % 16 != 0 || k < 1 || k > 64) return 0;
  return convTcPackFloats(co, ci, k, convPackF16());
}

extern "C" LKC_API LkcConvState* lkc_conv1d_state_create(const void* wp, int64_t co, int64_t ci, int64_t k) {
  if (!wp || lkc_conv1d_tc_pack_floats(co, ci, k) == 0) {
    fail("conv1d_state_create: shape not eligible for the tensor-core path or null pack");
    return nullptr;
  }
  ConvState* st = new (std::nothrow) ConvState{static_cast<const float*>(wp), co, ci, k, 0, convPackF16()};
  if (!st) fail("conv1d_state_create: out of host memory");
  return reinterpret_cast<LkcConvState*>(st);
}

extern "C" LKC_API void lkc_conv1d_state_destroy(LkcConvState* st) { delete reinterpret_cast<ConvState*>(st); }

// ints: w(Ci, Co, K) wp(n) padding stride
extern "C" LKC_API int lkc_convt_tc_pack_f32_cuda(const LkcArgs* a, void* stream) {
  LKC_REQUIRE(a && a->numPtrs == 2 && a->numInts == 6, "convt_tc_pack_f32_cuda: expected w | wp, padding, stride");
  const int64_t ci = a->ints[0], co = a->ints[1], k = a->ints[2], pad = a->ints[4], s = a->ints[5];
  LKC_REQUIRE(convtTcEligible(ci, co, k, s, pad),
              "convt_tc_pack_f32_cuda: needs stride 6 or 10, K = 2 stride, 2 padding = stride, Ci % 16 == 0");
  LKC_REQUIRE(a->ints[3] == convtTcPackFloats(ci, co, s, convPackF16()),
              "convt_tc_pack_f32_cuda: wp must hold lkc_convt_tc_pack_floats (of the current operand format)");
  return convtTcPack(F(a, 0), O(a, 1), ci, co, k, s, pad, convPackF16(), S(stream));
}

extern "C" LKC_API int64_t lkc_convt_tc_pack_floats(int64_t ci, int64_t co, int64_t k, int64_t stride, int64_t padding) {
  return convtTcEligible(ci, co, k, stride, padding) ? convtTcPackFloats(ci, co, stride, convPackF16()) : 0;
}

extern "C" LKC_API LkcConvState* lkc_convt_state_create(const void* wp, int64_t ci, int64_t co, int64_t k,
                                                        int64_t stride, int64_t padding) {
  if (!wp || !convtTcEligible(ci, co, k, stride, padding)) {
    fail("convt_state_create: shape not eligible for the tensor-core path or null pack");
    return nullptr;
  }
  ConvState* st = new (std::nothrow) ConvState{static_cast<const float*>(wp), co, ci, k, stride, convPackF16()};
  if (!st) fail("convt_state_create: out of host memory");
  return reinterpret_cast<LkcConvState*>(st);
}

extern "C" LKC_API int lkc_conv1d_tc_status(int* status, int reset) {
  LKC_REQUIRE(status, "conv1d_tc_status: null out pointer");
  return convTcStatus(status, reset != 0);
}

extern "C" LKC_API int lkc_conv1d_tc_status_async(int* status_host, void* stream) {
  LKC_REQUIRE(status_host, "conv1d_tc_status_async: null out pointer");
  return convTcStatusAsync(status_host, S(stream));
}

extern "C" LKC_API int lkc_conv1d_tc_profile(int enable, int64_t* counters16) {
  return convTcProfile(enable, reinterpret_cast<long long*>(counters16));
}

extern "C" LKC_API int lkc_set_conv_io(int mode) { return convTcSetIo(mode); }

extern "C" LKC_API int lkc_set_conv_path(int mode) {
  LKC_REQUIRE(mode >= 0 && mode <= 2, "set_conv_path: mode must be 0 (f16 split), 1 (CUDA cores only) or 2 (tf32 split)");
  gConvPath = mode;
  return 0;
}

namespace {
// Sorted by name.
const Entry kEntries[] = {
    {"adain1d_f32_cuda", lkc_adain1d_f32_cuda},
    {"adain_affine_f32_cuda", lkc_adain_affine_f32_cuda},
    {"add3_scale_f32_cuda", lkc_add3_scale_f32_cuda},
    {"add_f32_cuda", lkc_add_f32_cuda},
    {"channel_stats_f32_cuda", lkc_channel_stats_f32_cuda},
    {"concat_rows_f32_cuda", lkc_concat_rows_f32_cuda},
    {"conv1d_affine_f32_cuda", lkc_conv1d_affine_f32_cuda},
    {"conv1d_f32_cuda", lkc_conv1d_f32_cuda},
    {"conv1d_leaky_f32_cuda", lkc_conv1d_leaky_f32_cuda},
    {"conv1d_leaky_mean3_f32_cuda", lkc_conv1d_leaky_mean3_f32_cuda},
    {"conv1d_leaky_res_f32_cuda", lkc_conv1d_leaky_res_f32_cuda},
    {"conv1d_nobias_f32_cuda", lkc_conv1d_nobias_f32_cuda},
    {"conv1d_snake_f32_cuda", lkc_conv1d_snake_f32_cuda},
    {"conv1d_snake_res_f32_cuda", lkc_conv1d_snake_res_f32_cuda},
    {"conv1d_tc_pack_f32_cuda", lkc_conv1d_tc_pack_f32_cuda},
    {"conv_transpose1d_dw_f32_cuda", lkc_conv_transpose1d_dw_f32_cuda},
    {"conv_transpose1d_f32_cuda", lkc_conv_transpose1d_f32_cuda},
    {"conv_transpose1d_poly_f32_cuda", lkc_conv_transpose1d_poly_f32_cuda},
    {"conv_transpose1d_poly_mean3_f32_cuda", lkc_conv_transpose1d_poly_mean3_f32_cuda},
    {"convt_poly_pack_f32_cuda", lkc_convt_poly_pack_f32_cuda},
    {"convt_tc_pack_f32_cuda", lkc_convt_tc_pack_f32_cuda},
    {"gemm_bias_f32_cuda", lkc_gemm_bias_f32_cuda},
    {"harmonic_source_f32_cuda", lkc_harmonic_source_f32_cuda},
    {"harmonic_source_rng_f32_cuda", lkc_harmonic_source_rng_f32_cuda},
    {"istft_logits_f32_cuda", lkc_istft_logits_f32_cuda},
    {"leaky_relu_f32_cuda", lkc_leaky_relu_f32_cuda},
    {"pad_reflect1d_f32_cuda", lkc_pad_reflect1d_f32_cuda},
    {"scale_f32_cuda", lkc_scale_f32_cuda},
    {"snake_f32_cuda", lkc_snake_f32_cuda},
    {"space_to_depth_f32_cuda", lkc_space_to_depth_f32_cuda},
    {"stft_magphase_f32_cuda", lkc_stft_magphase_f32_cuda},
    {"upsample_nearest1d_f32_cuda", lkc_upsample_nearest1d_f32_cuda},
};
constexpr int kNumEntries = static_cast<int>(sizeof(kEntries) / sizeof(kEntries[0]));
}  // namespace

extern "C" LKC_API int lkc_kernel_count(void) { return kNumEntries; }
extern "C" LKC_API const char* lkc_kernel_name(int i) { return (i >= 0 && i < kNumEntries) ? kEntries[i].name : nullptr; }
extern "C" LKC_API LkcRunFn lkc_find_kernel(const char* name) {
  if (!name) return nullptr;
  for (int i = 0; i < kNumEntries; ++i)
    if (std::strcmp(kEntries[i].name, name) == 0) return kEntries[i].fn;
  return nullptr;
}
extern "C" LKC_API const char* lkc_last_error(void) { return gError; }
extern "C" LKC_API const char* lkc_build_info(void) { return "lkc sm_100a: tcgen05 split-operand fused conv / convT with TMA tile I/O + cuda-core conv/convT/stats/source/stft/istft"; }
