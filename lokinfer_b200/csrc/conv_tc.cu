// Tensor-core fused conv1d for sm_100a: implicit GEMM on tcgen05 with TMEM accumulators and split operands.
//
//   out[co, t] = sum_{ci, kk} W[co, ci, kk] * A[ci, t + kk d - pad],  A = act((x - mean) * scale + beta), zero outside
//   [0, L); epilogue + bias [+ residual] [* oscale] and the per-(channel, 128-column chunk) (mean, M2).
//
// GEMM view: D[128 co, 256 t] += Wtap[128 co, 16 ci] * Ashift[16 ci, 256 t] for every 16-channel chunk and tap.
// f32 accuracy comes from splitting both operands, v = hi + lo with an 11-bit hi and an 11-bit lo:
// out = sum Whi Ahi + (sum Wlo Ahi + Whi Alo); the lo*lo term, 2^-22 relative, is dropped. Two operand formats
// (see Fmt below): f16 halves (default; 3 kind::f16 K16 MMAs per tap and 16 channels) or tf32 halves (6 kind::tf32
// K8 MMAs).
//
// The tensor core adds into its f32 accumulator with truncation, so a long accumulation chain drifts towards zero by
// about 1.5e-8 of the result per MMA (measured: the error grows linearly with the chain length). Two accumulators
// keep that out of the result: Dhi (TMEM columns 0-255) takes only the hi*hi products of a short run of MMAs (a drain
// group: as many whole 16-channel chunks as fit in 24 chained MMAs, at least one chunk), is then drained by the
// epilogue warps into f32 registers (round-to-nearest adds on the CUDA cores) and restarted; Dlo (columns 256-511)
// takes every lo product of the tile, where the same drift is scaled by 2^-11.
//
// Global memory traffic goes through the TMA unit whenever the rows of a tensor are 16-byte aligned (base pointer and
// row pitch; the entry points take a row pitch for every [C, L] activation tensor, so a caller that owns its
// intermediates can pad the rows): the raw input window of a 16-channel chunk is one pair of tiled bulk loads, the
// residual arrives as 32 x 32 boxes in the 128-byte swizzle, and the output leaves as 32 x 32 boxes of the same
// swizzle (bulk tensor stores). Tensors whose rows are not aligned (the reference's contiguous [C, L] with an odd L)
// take 4-byte cp.async loads and transposed 4-byte stores instead; the arithmetic is the same on both routes.
// No copy uses cluster multicast, and every tensor map covers memory of this GPU only.
//
// One persistent CTA per SM, 20 warps in 5 warpgroups, warp-specialised (registers rebalanced with setmaxnreg). A warp
// is issued by scheduler (warp id % 4) of the SM. The MMA issuer's instructions between two MMAs are what keeps the
// tensor pipe fed, so its scheduler (1) hosts no activation producer, only the other two light control warps and the
// two epilogue warps that TMEM's lane rule puts there (measured: the issuer's own time outside waits fell by 15-19 %
// against a layout with two producers on its scheduler):
//   warps 0-7   accumulate + epilogue: 128 running sums per thread, started from the bias; the residual is added one
//               32-column batch at a time (fetched into the warp's tile behind a Dhi drain); per drain group += Dhi
//               (tcgen05.ld); per tile += Dlo (folded in before the tile's last drain: Dlo is complete one run of hi
//               MMAs before Dhi is), oscale, chunk statistics and the store
//   (launches that are bound by the producers, few MMAs per chunk, use the plain layout instead: producers 8-15,
//   two per scheduler, control warps 16-18)
//   warps 8, 10, 11, 12, 14, 15, 16, 18
//               activation producers: affine -> Snake / leaky -> hi / lo split of the current chunk's raw window into
//               shared memory in the K-major no-swizzle UMMA layout [16-byte K chunk][time row][4 f32 or 8 f16
//               channels]: a tap shift of kk*d time steps is a +16*kk*d byte offset of the descriptor start address,
//               so one staged window serves all taps (on the unaligned route they also issue the cp.async of the next
//               chunk's raw window)
//   warp 9      weight producer: one cp.async.bulk per tap group (up to 6 taps; hi | lo of [128 co x 16 ci] per tap,
//               pre-packed in the UMMA layout, L2-resident) into a ring of shared-memory slots
//   warp 13     MMA issuer (one lane): per tap group one wait, the group's MMAs back to back, one release
//   warp 17     raw-window loader of the aligned route (one lane): two tiled TMA loads per chunk, one chunk ahead
//   warp 19     idle (completes the fifth warpgroup)
// All hand-offs are mbarriers. Every wait is bounded: on a timeout the kernel records a status word, drains its
// copies in flight and returns (TMEM is freed on every path).
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "lkc_common.h"

#ifndef LKC_TC_PROF
#define LKC_TC_PROF 0  // 1: role-level cycle counters (lkc_conv1d_tc_profile); a build option, off in the product
#endif

namespace lkc {
namespace {

constexpr bool kProf = LKC_TC_PROF != 0;
constexpr int NT = 256;         // time columns per tile (= UMMA N)
constexpr int MT = 128;         // output channels per tile (= UMMA M)
constexpr int KC = 16;          // input channels per staged chunk (one weight stage, two K8 steps)
constexpr int MAX_NB = 4;       // most activation (hi / lo) buffers
constexpr int NRAW = 2;         // raw-input staging buffers, filled one chunk ahead
constexpr int EPI_WARPS = 8, PRO_WARPS = 8;
constexpr int IDLE_WARP = 19;
constexpr int NWARPS = EPI_WARPS + PRO_WARPS + 4;
constexpr int NTHREADS = NWARPS * 32;  // 640
// warpgroups 2-4 mix producers and control warps, and setmaxnreg takes one value per warpgroup
constexpr int LAUNCH_REGS = 96, EPI_REGS = 152, PRO_REGS = 56, CTL_REGS = PRO_REGS;
static_assert(NTHREADS * LAUNCH_REGS <= 65536, "launch register budget");
// setmaxnreg moves registers inside the CTA's own launch allocation (NTHREADS * LAUNCH_REGS); an increase beyond what
// the decreases release would block forever.
static_assert(EPI_WARPS * 32 * EPI_REGS + (NWARPS - EPI_WARPS) * 32 * PRO_REGS <= NTHREADS * LAUNCH_REGS,
              "register pool");
// Operand formats (template parameter F16 of the kernel):
//   tf32 split (F16 = false): hi = tf32(v), lo = v - hi, both stored as f32; per tap and 16 channels 6 MMAs of
//     kind::tf32 (K8): 2 x hi*hi into Dhi, 2 x (lo*hi + hi*lo) into Dlo.
//   f16 split (F16 = true): hi = f16(v), lo = f16((v - hi) * 2^11), both with the same 11-bit significand as tf32;
//     per tap and 16 channels 3 MMAs of kind::f16 (K16): hi*hi into Dhi, lo*hi + hi*lo into Dlo, which is folded in
//     with the factor 2^-11. Products are exact and accumulate in f32 as before, so the accuracy is that of the
//     tf32 split at half the tensor time, half the staged bytes and half the weight traffic. Values beyond the f16
//     range (|v| > 65504) are flagged in the status word: an activation becomes an infinite f16 operand (the output
//     of that launch is then not finite; kStatusF16Range), a weight is clamped at pack time (kStatusF16Weights).
constexpr float kLoScale = 2048.f;  // 2^11
constexpr int kStatusF16Range = 0x10000, kStatusF16Weights = 0x20000, kStatusWaitMask = 0xffff;
template <bool F16>
struct Fmt {
  static constexpr int W_STAGE_BYTES = F16 ? 2 * MT * KC * 2 : 2 * MT * KC * 4;  // hi + lo of [128 co x 16 ci]
  static constexpr int W_STAGE_FLOATS = W_STAGE_BYTES / 4;
  static constexpr int NB = F16 ? 3 : 2;  // activation (hi / lo) buffers; the f16 ones are half the size
  static constexpr int ACT_BYTES_PER_ROW = F16 ? 2 * KC * 2 : 2 * KC * 4;  // hi + lo of one time row, 16 channels
};
constexpr int STAGE_PITCH = 33;  // floats per row of an epilogue transpose tile (unaligned route)
constexpr int STAGE_FLOATS = 32 * STAGE_PITCH;
constexpr int BOX = 32, BOX_BYTES = BOX * BOX * 4;  // residual / output boxes of the aligned route: 32 co x 32 t
static_assert(BOX_BYTES <= STAGE_FLOATS * 4, "a swizzled box fits in a warp's tile");
constexpr int MAX_HALO = 50;     // (K - 1) * dilation of the widest Kokoro conv (K 11, dilation 5)
constexpr int MAX_W_STAGES = 4, MIN_W_STAGES = 2, PREF_W_STAGES = 2;  // weight ring slots
constexpr int TAP_GROUP = 6;  // most taps per weight slot: one bulk copy, one wait, MMAs back to back, one release
constexpr int MAX_CHAIN = 24;  // most chained hi MMAs between two drains of Dhi
constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr uint32_t SLEEP_EPI_NS = 256, SLEEP_PRO_NS = 128, SLEEP_W_NS = 64, SLEEP_MMA_NS = 32;
constexpr uint64_t WAIT_LIMIT_NS = 200ull * 1000 * 1000;  // 0.2 s: a healthy wait is tens of microseconds
constexpr int kMaxSmem = 232448;  // 227 KB per CTA on sm_100

// Shared-memory carve-up of one CTA (byte offsets from the 1024-byte aligned base). The epilogue tiles come first:
// the 128-byte swizzle of the aligned route needs each warp's 4 KB box on a 1024-byte boundary.
struct SmemLayout {
  uint32_t act, raw, w, par, bar, total;
};
__host__ __device__ inline SmemLayout smemLayout(int ci, int rows, int half, int nb, int wStages, int wG, int actRowBytes,
                                                 int wStageBytes) {
  SmemLayout s;
  s.act = EPI_WARPS * STAGE_FLOATS * 4;  // tiles: [0, act)
  s.raw = (s.act + uint32_t(nb) * actRowBytes * rows + 127u) & ~127u;
  s.w = s.raw + uint32_t(NRAW) * 2 * KC * half * 4;  // a multiple of 128
  s.par = s.w + uint32_t(wStages) * wG * wStageBytes;
  s.bar = s.par + uint32_t(4) * ci * 4;
  s.total = s.bar + 512;
  return s;
}

struct TcArgs {
  const float *x, *wp, *bias, *affine, *alpha, *residual;
  float *out, *stats;
  int ci, co, k, dilation, padding;
  int64_t l, lo, nchunks;
  int64_t validLo, validHi;            // x columns outside [validLo, validHi) are zero padding (after the activation)
  int64_t xPitch, resPitch, outPitch;  // row pitches in floats
  int padLeft;       // ConvTranspose: 1 = one-sample left reflect pad
  float slope, outScale;
  int rows;        // staged time rows per buffer = NT + (k-1)*dilation
  int half;        // raw staging: every channel's window is kept as two runs of `half` floats (two TMA boxes)
  int wStages;     // weight ring depth (slots)
  int nb;          // activation buffers
  int wG;          // taps per weight slot: the k taps of a chunk go in ceil(k / wG) groups of near-equal size
  int drainN;      // 16-channel chunks accumulated in Dhi between two drains into the running sums
  int balanced;    // warp-role layout (see the kernel)
  int tmaIn;       // 1: x rows are 16-byte aligned, the raw windows come by tiled TMA loads
  int tmaOut;      // 1: out (and residual) rows are 16-byte aligned, boxes go by TMA
  int numTTiles, numCoBlk;
  int* status;
  long long* prof;  // null, or 16 cycle counters summed over CTAs (see convTcProfile)
};

__device__ int gTcStatus = 0;       // 0 = ok; low 16 bits (role << 8 | code) of the first bounded wait that gave up; flag bits above
__device__ long long gTcProf[16];   // wait / phase cycle sums of one representative warp per role (profiling build)

// ---------------------------------------------------------------------------------------------- PTX helpers

__device__ __forceinline__ uint32_t smemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void mbarArriveExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
// One poll. Without a suspend-time hint the hardware parks the thread only briefly, which keeps the wake-up latency of
// the hand-offs low (a 1 ms hint measured 3-7 % slower end to end).
__device__ __forceinline__ bool mbarTryWait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up (false) after SPIN_LIMIT polls or WAIT_LIMIT_NS of wall time, whichever comes first, or as
// soon as another role has aborted. Between polls the warp sleeps `sleepNs`: the warp scheduler issues greedily from
// a ready warp, so a tight spin loop starves the producer warps that share its scheduler (measured: the producers
// ran at a tenth of their instruction rate next to spinning epilogue warps). Latency-critical waiters pass 0.
__device__ __forceinline__ bool mbarWait(uint64_t* bar, uint32_t parity, volatile int* abortFlag, uint32_t sleepNs) {
  if (mbarTryWait(bar, parity)) return true;
  const uint64_t t0 = globalTimerNs();
  for (uint32_t spins = 0; !mbarTryWait(bar, parity); ++spins) {
    if (sleepNs) __nanosleep(sleepNs);
    if (*abortFlag || spins >= SPIN_LIMIT) return false;
    if ((spins & 63) == 63 && globalTimerNs() - t0 > WAIT_LIMIT_NS) return false;
  }
  return true;
}
// Wait without the abort check, for draining copies in flight after an abort (bounded all the same).
__device__ __forceinline__ void mbarWaitQuiet(uint64_t* bar, uint32_t parity) {
  const uint64_t t0 = globalTimerNs();
  uint32_t spins = 0;
  while (!mbarTryWait(bar, parity) && ++spins < SPIN_LIMIT && globalTimerNs() - t0 < WAIT_LIMIT_NS) {
  }
}
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fenceBarrierInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void bulkCopyG2S(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smemAddr(dst)),
               "l"(src), "r"(bytes), "r"(smemAddr(bar))
               : "memory");
}
// Tiled TMA copies of a rank-2 tensor (coordinates: x = innermost = time, y = channel). x * 4 bytes must be a
// multiple of 16; a load may start outside the tensor (the missing part is filled with zeros), a store is clipped.
__device__ __forceinline__ void tmaLoad2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smemAddr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smemAddr(bar))
      : "memory");
}
__device__ __forceinline__ void tmaStore2d(const CUtensorMap* map, int x, int y, const void* src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(smemAddr(src))
               : "memory");
}
__device__ __forceinline__ void bulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until the bulk stores of this thread have read their shared-memory source / have completed.
__device__ __forceinline__ void bulkWaitRead() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void cpAsync4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smemAddr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void tmemAlloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(slot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], kind::tf32, issued by one thread.
__device__ __forceinline__ void mmaTf32(uint32_t dTmem, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(dTmem),
      "l"(descA), "l"(descB), "r"(idesc), "r"(accum)
      : "memory");
}
// kind::f16 with the descriptors given as (low word, high word): only the low word (address and leading-dimension
// fields) changes between taps, so the issuing thread does its descriptor arithmetic in 32 bits.
__device__ __forceinline__ void mmaF16W(uint32_t dTmem, uint32_t aLo, uint32_t aHi, uint32_t bLo, uint32_t bHi,
                                        uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(dTmem),
      "r"(aLo), "r"(aHi), "r"(bLo), "r"(bHi), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void mmaCommit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar))
               : "memory");
}
// tcgen05.ld 32x32b: thread i of the warp gets TMEM lane (base lane + i), registers = consecutive columns.
__device__ __forceinline__ void tmemLoad16Async(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmemWaitLoads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: core matrix = 8 rows x 16 bytes stored contiguously (rows at
// 16-byte pitch), `sbo` = byte distance between 8-row groups, `lbo` = byte distance between the two 16-byte K chunks
// of one K8 step. Bits: [0,14) address >> 4, [16,30) lbo >> 4, [32,46) sbo >> 4, [46,48) version = 1, [61,64) layout 0.
__device__ __forceinline__ uint64_t makeDesc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return uint64_t((addr >> 4) & 0x3FFFu) | (uint64_t((lbo >> 4) & 0x3FFFu) << 16) |
         (uint64_t((sbo >> 4) & 0x3FFFu) << 32) | (uint64_t(1) << 46);
}
// Instruction descriptor: D f32 (bits 4-5 = 1), A and B tf32 (bits 7-9 / 10-12 = 2), both K-major, N >> 3 at bit 17,
// M >> 4 at bit 24.
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(NT >> 3) << 17) | (uint32_t(MT >> 4) << 24);
// kind::f16 with f16 operands (format 0) and f32 accumulation.
constexpr uint32_t kIdescF16 = (1u << 4) | (uint32_t(NT >> 3) << 17) | (uint32_t(MT >> 4) << 24);

__device__ __forceinline__ float tf32Round(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

// sin(u)^2 for any finite u, absolute error ~1.5e-7: u = n pi/2 + r with |r| <= pi/4 (three-term Cody-Waite),
// sin^2(u) = sin^2(r) for even n and 1 - sin^2(r) for odd n.
// Two elements at a time on the packed f32x2 pipe (fma.rn.f32x2 and friends: one instruction, two lanes of math),
// two independent lanes of the same operation sequence.
__device__ __forceinline__ float2 sinSq2(float2 u) {
  const float2 kMagic = make_float2(12582912.f, 12582912.f);
  const float2 t = __ffma2_rn(u, make_float2(0.6366197723675814f, 0.6366197723675814f), kMagic);
  const float2 n = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  float2 r = __ffma2_rn(n, make_float2(-1.5703125f, -1.5703125f), u);
  r = __ffma2_rn(n, make_float2(-4.837512969970703125e-4f, -4.837512969970703125e-4f), r);
  r = __ffma2_rn(n, make_float2(-7.54978995489188216e-8f, -7.54978995489188216e-8f), r);
  const float2 s2 = __fmul2_rn(r, r);
  float2 p = __ffma2_rn(s2, make_float2(2.7557319e-6f, 2.7557319e-6f), make_float2(-1.9841270e-4f, -1.9841270e-4f));
  p = __ffma2_rn(p, s2, make_float2(8.3333333e-3f, 8.3333333e-3f));
  p = __ffma2_rn(p, s2, make_float2(-1.6666667e-1f, -1.6666667e-1f));
  p = __ffma2_rn(p, s2, make_float2(1.f, 1.f));
  const float2 sn = __fmul2_rn(r, p);
  const float2 q = __fmul2_rn(sn, sn);
  return make_float2((__float_as_int(t.x) & 1) ? 1.f - q.x : q.x, (__float_as_int(t.y) & 1) ? 1.f - q.y : q.y);
}

// Prologue with per-channel constants folded once per launch (sPar rows mean, a, b, inv):
//   Snake: u = (x - mean) * (alpha scale) + alpha beta; result = (u + sin^2(u)) / alpha  (= v + sin^2(alpha v) / alpha)
//   leaky / none: v = (x - mean) * scale + beta
// Centering first keeps the precision when the variance is tiny next to the mean, as in the reference.
template <int ACT>
__device__ __forceinline__ float2 activate2(float2 x, float2 negm, float2 a, float2 b, float2 inv, float slope) {
  const float2 v = __ffma2_rn(__fadd2_rn(x, negm), a, b);
  if (ACT == 1) return __fmul2_rn(__fadd2_rn(v, sinSq2(v)), inv);
  if (ACT == 2) return make_float2(v.x >= 0.f ? v.x : v.x * slope, v.y >= 0.f ? v.y : v.y * slope);
  return v;
}

template <int N>
__device__ __forceinline__ void regInc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void regDec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// PARTIAL: Co is not a multiple of 128 (the last output-channel block has rows that do not exist).
// TS: 0 = conv1d; 6 / 10 = polyphase ConvTranspose1d of that stride (see the comment above convtTcPackKernel).
// TMAO: residual and output boxes travel by TMA (rows 16-byte aligned; conv1d with Co % 128 == 0 only).
template <int ACT, bool PARTIAL, int TS, bool F16, bool TMAO>
__global__ void __launch_bounds__(NTHREADS, 1)
    convTcKernel(const TcArgs a, const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapRes,
                 const __grid_constant__ CUtensorMap mapOut) {
  constexpr int W_STAGE_BYTES = Fmt<F16>::W_STAGE_BYTES, W_STAGE_FLOATS = Fmt<F16>::W_STAGE_FLOATS;
  const int NB = a.nb;
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  const int rows = a.rows, half = a.half;
  const SmemLayout lay = smemLayout(a.ci, rows, half, NB, a.wStages, a.wG, Fmt<F16>::ACT_BYTES_PER_ROW, W_STAGE_BYTES);
  const int actBufFloats = Fmt<F16>::ACT_BYTES_PER_ROW / 4 * rows;  // hi + lo
  const int rawBufFloats = 2 * KC * half;
  float* const sStage = reinterpret_cast<float*>(smemRaw);           // EPI_WARPS tiles
  float* const sAct = reinterpret_cast<float*>(smemRaw + lay.act);   // NB buffers of [2 (hi, lo)][16-byte K chunks][rows]
  float* const sRaw = reinterpret_cast<float*>(smemRaw + lay.raw);   // NRAW buffers of [2 runs][KC][half] raw input
  float* const sW = reinterpret_cast<float*>(smemRaw + lay.w);       // wStages slots of wG taps of [2 (hi, lo)][16-byte K chunks][MT]
  float* const sPar = reinterpret_cast<float*>(smemRaw + lay.par);   // [4][ci]: folded prologue constants
  uint64_t* const bFull = reinterpret_cast<uint64_t*>(smemRaw + lay.bar);
  uint64_t* const bEmpty = bFull + MAX_NB;
  uint64_t* const wFull = bEmpty + MAX_NB;
  uint64_t* const wEmpty = wFull + MAX_W_STAGES;
  uint64_t* const hiFull = wEmpty + MAX_W_STAGES;
  uint64_t* const hiEmpty = hiFull + 1;
  uint64_t* const loFull = hiEmpty + 1;
  uint64_t* const loEmpty = loFull + 1;
  uint64_t* const rawFull = loEmpty + 1;
  uint64_t* const rawEmpty = rawFull + NRAW;
  uint64_t* const resBar = rawEmpty + NRAW;  // one per epilogue warp
  uint32_t* const tmemSlot = reinterpret_cast<uint32_t*>(resBar + EPI_WARPS);
  volatile int* const abortFlag = reinterpret_cast<int*>(tmemSlot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (TMAO && (smemAddr(smemRaw) & 1023u)) {
    // the 128-byte swizzle of the boxes assumes a 1024-byte aligned base; report instead of computing garbage
    if (threadIdx.x == 0) atomicOr(a.status, (6 << 8) | 1);
    return;
  }
  // Two warp-role layouts. Isolated (a.balanced == 0): the three control warps on scheduler 1 (warp id % 4 == 1), no
  // producer next to the MMA issuer. Balanced: producers 8-15 (two per scheduler), control warps 16-18; for launches
  // that are bound by the activation producers, where the issuer's pace does not matter.
  const bool bal = a.balanced != 0;
  const int W_WARP = bal ? 16 : 9, MMA_WARP = bal ? 17 : 13, RAW_WARP = bal ? 18 : 17;
  const int numTiles = a.numTTiles * a.numCoBlk;
  const int nChunks16 = a.ci / KC;
  const int nGroups = (nChunks16 + a.drainN - 1) / a.drainN;  // Dhi drains per tile
  // tap groups of a chunk: the first tgExtra groups have tgBase + 1 taps, the others tgBase
  const int nTapGroups = (a.k + a.wG - 1) / a.wG, tgBase = a.k / nTapGroups, tgExtra = a.k % nTapGroups;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NB; ++i) mbarInit(&bFull[i], PRO_WARPS), mbarInit(&bEmpty[i], 1);
    for (int i = 0; i < MAX_W_STAGES; ++i) mbarInit(&wFull[i], 1), mbarInit(&wEmpty[i], 1);
    mbarInit(hiFull, 1), mbarInit(hiEmpty, EPI_WARPS), mbarInit(loFull, 1), mbarInit(loEmpty, EPI_WARPS);
    for (int i = 0; i < NRAW; ++i) mbarInit(&rawFull[i], 1), mbarInit(&rawEmpty[i], PRO_WARPS);
    for (int i = 0; i < EPI_WARPS; ++i) mbarInit(&resBar[i], 1);
    *abortFlag = 0;
    fenceBarrierInit();
  }
  if (warp == MMA_WARP) {  // the MMA warp owns the TMEM allocation
    tmemAlloc(tmemSlot, 512);
    tmemRelinquish();
  }
  tcFenceBefore();
  __syncthreads();
  tcFenceAfter();
  const uint32_t tmemBase = *tmemSlot;
  const uint32_t tmemHi = tmemBase, tmemLo = tmemBase + NT;

  // mbarWait that adds the cycles it spent to acc in the profiling build
  auto waitT = [&](uint64_t* bar, uint32_t parity, long long& acc, uint32_t sleepNs) -> bool {
    if constexpr (!kProf) {
      return mbarWait(bar, parity, abortFlag, sleepNs);
    } else {
      const long long t0 = clock64();
      const bool ok = mbarWait(bar, parity, abortFlag, sleepNs);
      acc += clock64() - t0;
      return ok;
    }
  };
  auto profAdd = [&](int slot, long long v) {
    if (kProf && a.prof && lane == 0)
      atomicAdd(reinterpret_cast<unsigned long long*>(a.prof + slot), (unsigned long long)v);
  };
  // First timeout wins the low 16 bits; the flag bits above them are kept.
  auto giveUp = [&](int role, int code) {
    if (lane == 0) {
      int old = *a.status;
      while ((old & kStatusWaitMask) == 0) {
        const int seen = atomicCAS(a.status, old, old | (role << 8) | code);
        if (seen == old) break;
        old = seen;
      }
      *abortFlag = 1;
    }
  };

  if (warp < EPI_WARPS) {
    // ------------------------------------------------------------------ accumulate + epilogue
    regInc<EPI_REGS>();
    const int q = warp & 3, g = warp >> 2;  // TMEM lane quarter, 128-column half of the tile
    float* const tile = sStage + warp * STAGE_FLOATS;                                  // unaligned route: [32][33]
    unsigned char* const box = smemRaw + warp * BOX_BYTES;                             // aligned route: swizzled 32 x 32
    unsigned char* const boxRow = box + lane * 128;                                    // this lane's row of the box
    const int swz = lane & 7;  // 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7)
    uint64_t* const myRes = &resBar[warp];
    static_assert(!TMAO || (TS == 0 && !PARTIAL), "boxes need whole 32-channel row groups of a conv1d");
    constexpr bool tmaOut = TMAO;
    const uint32_t laneBase = uint32_t(q * 32) << 16;
    uint32_t groupIt = 0, tileIt = 0, resIt = 0;
    bool dead = false, resInFlight = false;
    long long wHi = 0, wLo = 0, cPre = 0, cFin = 0;
    const long long tStart = kProf ? clock64() : 0;
    for (int t = blockIdx.x; t < numTiles && !dead; t += gridDim.x, ++tileIt) {
      const int tt = t / a.numCoBlk, cb = t - tt * a.numCoBlk;
      const long long tPre = kProf ? clock64() : 0;
      const int64_t tChunk = int64_t(tt) * NT + g * 128;  // first output column of this warp's 128-column chunk
      const int64_t nValid64 = a.lo - tChunk;
      const int nValid = nValid64 <= 0 ? 0 : (nValid64 < 128 ? int(nValid64) : 128);
      // conv: the warp's rows are 32 consecutive output channels. ConvTranspose: rows are (channel, phase) pairs,
      // CQ channels x TS phases per warp (lane = cl * TS + r), the last 32 - CQ * TS rows are zero padding.
      constexpr int CQ = TS ? 32 / TS : 32, ROWS = TS ? CQ * TS : 32;
      // Row pitch of the warp's transpose tile. ConvTranspose: 35 floats, so that both the row-wise accesses (lane =
      // row: 3 * lane mod 32 is a permutation) and the interleaved ones (phase r, column q -> bank 3 r + q: at most
      // two lanes per bank) stay cheap; its 30 rows still fit the tile (30 x 35 <= 32 x 33).
      constexpr int TP = TS ? 35 : STAGE_PITCH;
      static_assert(ROWS * TP <= STAGE_FLOATS, "transpose tile");
      const int coBase = TS ? (cb * 4 + q) * CQ : cb * MT + q * 32;
      const int co = TS ? coBase + lane / (TS ? TS : 1) : coBase + lane;
      const bool rowOk = TS ? (lane < ROWS && co < a.co) : (!PARTIAL || co < a.co);
      const float bias = (a.bias && rowOk) ? a.bias[co] : 0.f;
      // channels of this warp that exist (may be <= 0 in the last block)
      const int coValid = (TS || PARTIAL) ? (a.co - coBase < CQ ? a.co - coBase : CQ) : 32;
      // Running sums start from the bias. The residual is added one 32-column batch at a time: while the warp waits
      // for drain group c, residual batch c travels into the warp's tile (a TMA box, or cp.async with lanes along
      // time); after the group has been drained the batch is read back with lanes along channels and added.
      // The global latency hides behind a whole group of MMAs and no registers are held while waiting.
      float S[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) S[j] = bias;
      const bool hasRes = a.residual != nullptr;
      // ConvTranspose with the left reflect pad: out[co, 0] = unpadded[co, 1] + res[co, 0] (the reference copies
      // the column, then adds the residual). The lane that owns (column 0, phase 1) keeps that element's residual
      // out of its running sum and adds it last, so the reflect column gets the plain conv sum.
      const bool reflectLane = TS != 0 && a.padLeft != 0 && tChunk == 0 && lane < ROWS && (lane % (TS ? TS : 1)) == 1;
      float resHeld = 0.f;
      auto fetchResidual = [&](int b) {  // batch b of the warp's 128 columns -> tile (zero where out of range)
        if (tmaOut) {
          if (lane == 0) {
            bulkWaitRead();  // the stores of the previous tile have read the box
            mbarArriveExpectTx(myRes, BOX_BYTES);
            tmaLoad2d(box, &mapRes, int(tChunk) + b * BOX, coBase, myRes);
          }
          resInFlight = true;
          return;
        }
        if constexpr (TS == 0) {
          const bool ok = b * 32 + lane < nValid;
          const float* rp = a.residual + int64_t(coBase) * a.resPitch + tChunk + b * 32 + lane;
          float* tp = tile + lane;
          const int rowsOk = ok ? (PARTIAL ? (coValid < 0 ? 0 : coValid) : 32) : 0;  // rows this lane copies
          int i = 0;
#pragma unroll 8
          for (; i < rowsOk; ++i, tp += STAGE_PITCH, rp += a.resPitch) cpAsync4(tp, rp);
          for (; i < 32; ++i, tp += STAGE_PITCH) *tp = 0.f;
        } else {
          // channel cl: the 32 * TS output samples u = (tChunk + 32 b) * TS + idx are contiguous in memory; copy
          // i = cl * TS + f moves idx = 32 f + lane, which is column idx / TS of phase idx % TS
          // The tile offsets of the TS copies of a channel depend on the lane only: computed once per batch, then a
          // rolled loop over the channels with pointer increments (this runs four times per tile on every epilogue
          // warp; the index arithmetic of the (channel, copy) pair per element cost more than the copies).
          const int64_t uEnd = a.lo * TS, u0 = (tChunk + b * 32) * TS;
          int off[TS ? TS : 1];
#pragma unroll
          for (int f = 0; f < TS; ++f) off[f] = ((f * 32 + lane) % TS) * TP + (f * 32 + lane) / TS;
          const int64_t left = uEnd - u0 - lane;  // copy f of this lane is inside the row iff f * 32 < left
          const float* rp = a.residual + int64_t(coBase) * a.resPitch + a.padLeft + u0 + lane;
          float* tp = tile;
#pragma unroll 1
          for (int cl = 0; cl < CQ; ++cl, rp += a.resPitch, tp += TS * TP) {
            const bool chOk = cl < coValid;
#pragma unroll
            for (int f = 0; f < TS; ++f) {
              if (chOk && f * 32 < left) cpAsync4(tp + off[f], rp + f * 32);
              else tp[off[f]] = 0.f;
            }
          }
        }
        cpAsyncCommit();
      };
      auto addResidual = [&](int b) {
        if (tmaOut) {
          if (!mbarWait(myRes, resIt & 1, abortFlag, 32)) {
            giveUp(1, 3);
            dead = true;
            return;
          }
          ++resIt, resInFlight = false;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 v = *reinterpret_cast<const float4*>(boxRow + ((c ^ swz) << 4));
            S[b * 32 + 4 * c] += v.x, S[b * 32 + 4 * c + 1] += v.y, S[b * 32 + 4 * c + 2] += v.z,
                S[b * 32 + 4 * c + 3] += v.w;
          }
          __syncwarp();
          return;
        }
        cpAsyncWait<0>();
        __syncwarp();
        if (TS == 0 || lane < ROWS) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float r = tile[lane * TP + j];
            if (TS != 0 && b == 0 && j == 0 && reflectLane) resHeld = r;
            else S[b * 32 + j] += r;
          }
        }
        __syncwarp();
      };
      if (kProf) cPre += clock64() - tPre;
      // wait for the group's hi chain, add it to the running sums, hand Dhi back
      auto drainGroup = [&]() -> bool {
        if (!waitT(hiFull, groupIt & 1, wHi, SLEEP_EPI_NS)) {
          giveUp(1, 1);
          return false;
        }
        tcFenceAfter();
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          uint32_t v[16];
          tmemLoad16Async(tmemHi + laneBase + g * 128 + b * 16, v);
          tmemWaitLoads();
#pragma unroll
          for (int j = 0; j < 16; j += 2) {  // packed f32x2 adds: half the instructions of the accumulate loop
            const float2 sum = __fadd2_rn(make_float2(S[b * 16 + j], S[b * 16 + j + 1]),
                                          make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])));
            S[b * 16 + j] = sum.x, S[b * 16 + j + 1] = sum.y;
          }
        }
        tcFenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(hiEmpty);
        ++groupIt;
        return true;
      };
      // Four residual batches per tile. With four or more drains the first four each carry one (fetched before the
      // wait for the group, added after the drain); with fewer drains the surplus batches get steps of their own
      // where this warp would otherwise only wait for a group: right after the first drain (the second group's MMAs
      // hide their fetch latency; before the first drain the warp is still busy with the previous tile's final
      // phase), or before the only drain of a tile, instead of between the last drain and the final phase.
      // One copy of the fetch and of the drain in the code (this kernel is far larger than the instruction cache,
      // and straight-line code that runs once per tile is fetched at a fraction of the issue rate); only the add
      // needs static register indices.
      const int nPre = hasRes && nGroups < 4 ? 4 - nGroups : 0;
      const int nSteps = nPre + nGroups, preAt = nGroups == 1 ? 0 : 1;  // first step without a drain
      int rb = 0;  // next residual batch
#pragma unroll 1
      for (int c = 0; c < nSteps && !dead; ++c) {
        const bool doRes = hasRes && rb < 4;
        if (doRes) fetchResidual(rb);
        if (c == nSteps - 1) {
          // Last step of the tile (always a drain): Dlo is complete before the last hi MMAs are, so it is folded in
          // first and handed back, and the next tile's lo MMAs need not wait for the last drain and the final phase.
          if (!waitT(loFull, tileIt & 1, wLo, SLEEP_EPI_NS)) {
            giveUp(1, 2);
            dead = true;
            break;
          }
          tcFenceAfter();
#pragma unroll
          for (int b = 0; b < 4; ++b) {  // two 16-column loads in flight per wait
            uint32_t va[16], vb[16];
            tmemLoad16Async(tmemLo + laneBase + g * 128 + b * 32, va);
            tmemLoad16Async(tmemLo + laneBase + g * 128 + b * 32 + 16, vb);
            tmemWaitLoads();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float x = __uint_as_float(va[j]), y = __uint_as_float(vb[j]);
              S[b * 32 + j] = F16 ? fmaf(x, 1.f / kLoScale, S[b * 32 + j]) : S[b * 32 + j] + x;
              S[b * 32 + 16 + j] = F16 ? fmaf(y, 1.f / kLoScale, S[b * 32 + 16 + j]) : S[b * 32 + 16 + j] + y;
            }
          }
          tcFenceBefore();
          __syncwarp();
          if (lane == 0) mbarArrive(loEmpty);
        }
        if (c < preAt || c >= preAt + nPre) dead = !drainGroup();
        if (doRes && !dead) {
          switch (rb) {
            case 0: addResidual(0); break;
            case 1: addResidual(1); break;
            case 2: addResidual(2); break;
            default: addResidual(3); break;
          }
          ++rb;
        }
      }
      if (dead) break;
      const long long tFin = kProf ? clock64() : 0;
      if (a.residual && a.outScale != 1.f) {
#pragma unroll
        for (int j = 0; j < 128; ++j) S[j] *= a.outScale;
      }

      if constexpr (TS == 0) {
        // Per 32-column batch: chunk statistics of this lane's channel from the registers, and the store. Aligned
        // route: the registers go to the warp's box in the 128-byte swizzle (8 conflict-free 16-byte stores), one
        // lane sends the box with a bulk tensor store (clipped at the end of the row) and the statistics of the
        // batch run while the TMA unit reads it. Unaligned route: the registers go to the [32][33] tile and rolled
        // loops store it transposed, lanes along time (rolled loops stay in the instruction cache; the unrolled form
        // of this phase, 1100 instructions run once per tile, ran at about 20 clocks per instruction).
        float pMean[4], pM2[4];
        const int rowsValid = PARTIAL ? (coValid < 0 ? 0 : coValid) : 32;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int nb = nValid - b * 32 <= 0 ? 0 : (nValid - b * 32 < 32 ? nValid - b * 32 : 32);  // valid columns
          if (tmaOut) {
            if (nb > 0) {  // warp-uniform
              if (lane == 0) bulkWaitRead();  // the previous store has read the box
              __syncwarp();
#pragma unroll
              for (int c = 0; c < 8; ++c)
                *reinterpret_cast<float4*>(boxRow + ((c ^ swz) << 4)) =
                    make_float4(S[b * 32 + 4 * c], S[b * 32 + 4 * c + 1], S[b * 32 + 4 * c + 2], S[b * 32 + 4 * c + 3]);
              fenceProxyAsync();  // generic-proxy stores -> visible to the TMA unit
              __syncwarp();
              if (lane == 0) {
                tmaStore2d(&mapOut, int(tChunk) + b * BOX, coBase, box);
                bulkCommit();
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) tile[lane * STAGE_PITCH + j] = S[b * 32 + j];
            __syncwarp();
          }
          // statistics of the valid columns of this lane's channel (two passes over the registers, four chains)
          float m, q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
          {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            if (nb == 32) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                s0 += S[b * 32 + j], s1 += S[b * 32 + j + 1], s2 += S[b * 32 + j + 2], s3 += S[b * 32 + j + 3];
              m = ((s0 + s1) + (s2 + s3)) * (1.f / 32.f);
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float d0 = S[b * 32 + j] - m, d1 = S[b * 32 + j + 1] - m, d2 = S[b * 32 + j + 2] - m,
                            d3 = S[b * 32 + j + 3] - m;
                q0 = fmaf(d0, d0, q0), q1 = fmaf(d1, d1, q1), q2 = fmaf(d2, d2, q2), q3 = fmaf(d3, d3, q3);
              }
            } else {  // ragged end of a row: rolled loops over the copy in shared memory (rare: keeps the code small)
              auto at = [&](int j) -> float {
                return tmaOut ? *reinterpret_cast<const float*>(boxRow + (((j >> 2) ^ swz) << 4) + ((j & 3) << 2))
                              : tile[lane * STAGE_PITCH + j];
              };
#pragma unroll 1
              for (int j = 0; j < nb; ++j) s0 += at(j);
              m = nb > 0 ? s0 / float(nb) : 0.f;
#pragma unroll 1
              for (int j = 0; j < nb; ++j) {
                const float d = at(j) - m;
                q0 = fmaf(d, d, q0);
              }
            }
          }
          pMean[b] = m, pM2[b] = (q0 + q1) + (q2 + q3);
          if (!tmaOut) {
            // store with lanes along time
            if (lane < nb) {
              float* op = a.out + int64_t(coBase) * a.outPitch + tChunk + b * 32 + lane;
              const float* col = tile + lane;
              int i = 0;
#pragma unroll 1
              for (; i + 8 <= rowsValid; i += 8) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = col[(i + e) * STAGE_PITCH];
#pragma unroll
                for (int e = 0; e < 8; ++e) op[int64_t(i + e) * a.outPitch] = v[e];
              }
              for (; i < rowsValid; ++i) op[int64_t(i) * a.outPitch] = col[i * STAGE_PITCH];
            }
            __syncwarp();
          }
        }
        if (a.stats && nValid > 0 && (!PARTIAL || co < a.co)) {
          // exact combine of the four 32-column partials: mean = sum n_b m_b / n, M2 = sum M2_b + sum n_b (m_b - mean)^2
          float sum = 0.f;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int nb = nValid - b * 32 <= 0 ? 0 : (nValid - b * 32 < 32 ? nValid - b * 32 : 32);
            sum = fmaf(float(nb), pMean[b], sum);
          }
          const float mean = sum / float(nValid);
          float m2 = 0.f;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int nb = nValid - b * 32 <= 0 ? 0 : (nValid - b * 32 < 32 ? nValid - b * 32 : 32);
            const float d = pMean[b] - mean;
            m2 += pM2[b] + float(nb) * d * d;
          }
          float* st = a.stats + (int64_t(co) * a.nchunks + tChunk / 128) * 2;
          if ((reinterpret_cast<uintptr_t>(a.stats) & 7) == 0) *reinterpret_cast<float2*>(st) = make_float2(mean, m2);
          else st[0] = mean, st[1] = m2;
        }
      } else {
        // ConvTranspose: interleave the TS phases of each channel back into contiguous output samples
        const int64_t uEnd = a.lo * TS;
        float reflectVal = 0.f;
        if (reflectLane) {
          reflectVal = S[0];   // plain conv sum of (column 0, phase 1) = unpadded[co, 1]
          S[0] += resHeld;     // the element's own residual, added last
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int64_t u0 = (tChunk + b * 32) * TS;
          if (lane < ROWS) {
#pragma unroll
            for (int j = 0; j < 32; ++j) tile[lane * TP + j] = S[b * 32 + j];
          }
          __syncwarp();
          int off[TS ? TS : 1];  // as in the residual fetch: lane-only tile offsets, then pointer increments
#pragma unroll
          for (int f = 0; f < TS; ++f) off[f] = ((f * 32 + lane) % TS) * TP + (f * 32 + lane) / TS;
          const int64_t left = uEnd - u0 - lane;
          float* op = a.out + int64_t(coBase) * a.outPitch + a.padLeft + u0 + lane;
          const float* tp = tile;
#pragma unroll 1
          for (int cl = 0; cl < CQ; ++cl, op += a.outPitch, tp += TS * TP) {
            if (cl >= coValid) break;
#pragma unroll
            for (int f = 0; f < TS; ++f)
              if (f * 32 < left) op[f * 32] = tp[off[f]];
          }
          __syncwarp();
        }
        if (reflectLane && co < a.co && uEnd > 1) {
          const int64_t row = int64_t(co) * a.outPitch;
          a.out[row] = reflectVal + (a.residual ? a.residual[int64_t(co) * a.resPitch] : 0.f);
        }
      }
      if (kProf) cFin += clock64() - tFin;
    }
    // Copies of this warp still in flight must end before the CTA may exit: a residual box after an abort, and the
    // output boxes on every path.
    if (resInFlight) mbarWaitQuiet(myRes, resIt & 1);
    if (tmaOut && lane == 0) bulkWaitAll();
    if (kProf && warp == 0)
      profAdd(5, wHi), profAdd(6, wLo), profAdd(7, cPre), profAdd(8, cFin), profAdd(9, clock64() - tStart);
  } else if (bal ? warp < EPI_WARPS + PRO_WARPS : ((warp & 3) != 1 && warp != IDLE_WARP)) {
    // ------------------------------------------------------------------ activation producers
    regDec<PRO_REGS>();
    const int pw = bal ? warp - EPI_WARPS
                       : (warp - EPI_WARPS) - ((warp - EPI_WARPS + 2) >> 2);  // 8, 10, 11, 12, 14, 15, 16, 18 -> 0..7
    const int cg = pw & 3, hf = pw >> 2;  // channel group of 4 inside the 16-channel chunk; row half
    const int rowsHalf = (rows + 1) >> 1;
    const int r0 = hf * rowsHalf, r1 = (r0 + rowsHalf < rows) ? r0 + rowsHalf : rows;
    constexpr int SLOTS = (((NT + MAX_HALO + 1) >> 1) + 31) / 32;  // row slots of 32 lanes per warp
    const bool tmaIn = a.tmaIn != 0;
    const int runSkip = (KC - 1) * half;  // a raw window index i >= half sits in the second run: + runSkip floats
    // per-channel parameters, once: sPar = [mean | a | b | inv] with a = scale, b = beta (x alpha for Snake), inv = 1/alpha
    for (int c = pw * 32 + lane; c < a.ci; c += PRO_WARPS * 32) {
      const float al = ACT == 1 ? a.alpha[c] : 1.f;
      sPar[c] = a.affine ? a.affine[c] : 0.f;
      sPar[a.ci + c] = (a.affine ? a.affine[a.ci + c] : 1.f) * al;
      sPar[2 * a.ci + c] = (a.affine ? a.affine[2 * a.ci + c] : 0.f) * al;
      sPar[3 * a.ci + c] = 1.f / al;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(PRO_WARPS * 32) : "memory");  // producer warps only

    // Unaligned route: cp.async of this thread's part of the raw window of chunk c of the tile whose window starts at
    // input position posT (= tile column * NT - padding) into staging buffer rb. Pointer increments only: this runs
    // once per chunk on every producer thread.
    auto issueCopies = [&](int64_t posT, int c, int rb) {
      const float* xc = a.x + int64_t(c * KC + cg * 4) * a.xPitch + posT + r0 + lane;
      float* base = sRaw + rb * rawBufFloats + cg * 4 * half;
      int64_t pos = posT + r0 + lane;
      int r = r0 + lane;
#pragma unroll
      for (int sl = 0; sl < SLOTS; ++sl, r += 32, pos += 32, xc += 32) {
        if (r < r1 && pos >= 0 && pos < a.l) {
          float* dst = base + r + (r >= half ? runSkip : 0);
          cpAsync4(dst, xc);
          cpAsync4(dst + half, xc + a.xPitch);
          cpAsync4(dst + 2 * half, xc + 2 * a.xPitch);
          cpAsync4(dst + 3 * half, xc + 3 * a.xPitch);
        }
      }
    };

    int t = blockIdx.x, c = 0;
    uint32_t buf = 0, bufPar = 1, rawBuf = 0, rawPar = 0;  // activation buffer + parity of its last release; raw buffer + parity of its fill
    long long wB = 0, wCp = 0, cTr = 0;
    const long long tStart = kProf ? clock64() : 0;
    int64_t pos0 = int64_t(t / a.numCoBlk) * NT - a.padding;  // input position of row 0 of the current tile's window
    if (!tmaIn) {
      if (t < numTiles) issueCopies(pos0, c, 0);
      cpAsyncCommit();
    }
    while (t < numTiles) {
      int tn = t, cn = c + 1;
      int64_t posN = pos0;
      if (cn == nChunks16) {
        cn = 0, tn = t + gridDim.x;
        posN = int64_t(tn / a.numCoBlk) * NT - a.padding;
      }
      // the window's offset inside the staged runs: the aligned route loads from the 16-byte boundary below pos0
      int delta = 0;
      if (tmaIn) {
        delta = int(pos0 & 3);
        if (!waitT(&rawFull[rawBuf], rawPar, wCp, SLEEP_PRO_NS)) {
          giveUp(2, 2);
          break;
        }
      } else {
        if (tn < numTiles) issueCopies(posN, cn, rawBuf ^ 1);
        cpAsyncCommit();
        const long long tCp = kProf ? clock64() : 0;
        cpAsyncWait<1>();  // this chunk's copies (the older group) have landed; the next chunk's stay in flight
        if (kProf) wCp += clock64() - tCp;
      }
      if (!waitT(&bEmpty[buf], bufPar, wB, SLEEP_PRO_NS)) {
        giveUp(2, 1);
        break;
      }
      const long long tTr = kProf ? clock64() : 0;
      // tf32 split: [cg][rows][4 f32]; f16 split: [cg / 2][rows][8 f16], this thread's 4 channels = half of a chunk
      float* hi = F16 ? sAct + buf * actBufFloats + (cg >> 1) * rows * 4 + (cg & 1) * 2
                      : sAct + buf * actBufFloats + cg * rows * 4;
      float* lo = hi + actBufFloats / 2;
      const float* src = sRaw + rawBuf * rawBufFloats + cg * 4 * half + delta;
      // this thread's four channels: constants in registers for the whole chunk
      float2 nm[2], pa[2], pb[2], pi[2];  // channel pairs (0, 1) and (2, 3); nm = -mean
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float* par = sPar + c * KC + cg * 4 + 2 * h;
        nm[h] = make_float2(-par[0], -par[1]);
        pa[h] = make_float2(par[a.ci], par[a.ci + 1]);
        pb[h] = make_float2(par[2 * a.ci], par[2 * a.ci + 1]);
        pi[h] = make_float2(par[3 * a.ci], par[3 * a.ci + 1]);
      }
      float big = 0.f;  // largest |value| this thread staged in the chunk (f16 range check, once per chunk)
#pragma unroll
      for (int sl = 0; sl < SLOTS; ++sl) {
        // Branch-free body, so that the iterations' dependency chains interleave: rows beyond the thread's range
        // recompute its last row and skip the stores; positions outside the valid range select zero.
        const int rq = r0 + sl * 32 + lane;
        const bool inr = rq < r1;
        const int r = inr ? rq : r1 - 1;
        const int64_t pos = pos0 + r;
        const bool ok = pos >= a.validLo && pos < a.validHi;
        const float* sp = src + r + (r + delta >= half ? runSkip : 0);
        float2 v01 = activate2<ACT>(make_float2(sp[0], sp[half]), nm[0], pa[0], pb[0], pi[0], a.slope);
        float2 v23 = activate2<ACT>(make_float2(sp[2 * half], sp[3 * half]), nm[1], pa[1], pb[1], pi[1], a.slope);
        v01.x = ok ? v01.x : 0.f, v01.y = ok ? v01.y : 0.f, v23.x = ok ? v23.x : 0.f, v23.y = ok ? v23.y : 0.f;
        if constexpr (!F16) {
          float4 h, l;
          h.x = tf32Round(v01.x), h.y = tf32Round(v01.y), h.z = tf32Round(v23.x), h.w = tf32Round(v23.y);
          const float2 l01 = __fadd2_rn(v01, make_float2(-h.x, -h.y)), l23 = __fadd2_rn(v23, make_float2(-h.z, -h.w));
          l = make_float4(l01.x, l01.y, l23.x, l23.y);
          if (inr) {
            *reinterpret_cast<float4*>(hi + r * 4) = h;
            *reinterpret_cast<float4*>(lo + r * 4) = l;
          }
        } else {
          // hi = f16(v), lo = f16((v - hi) * 2^11); 4 channels = 8 bytes of the row's 16-byte K chunk (channel groups
          // 2 j and 2 j + 1 share chunk j). A value beyond the f16 range becomes infinite here and is reported below.
          big = fmaxf(big, fmaxf(fmaxf(fabsf(v01.x), fabsf(v01.y)), fmaxf(fabsf(v23.x), fabsf(v23.y))));
          const __half2 h01 = __float22half2_rn(v01), h23 = __float22half2_rn(v23);
          const float2 sc = make_float2(kLoScale, kLoScale);
          const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
          const __half2 l01 = __float22half2_rn(__fmul2_rn(__fadd2_rn(v01, make_float2(-f01.x, -f01.y)), sc));
          const __half2 l23 = __float22half2_rn(__fmul2_rn(__fadd2_rn(v23, make_float2(-f23.x, -f23.y)), sc));
          uint2 hw, lw;
          hw.x = *reinterpret_cast<const uint32_t*>(&h01), hw.y = *reinterpret_cast<const uint32_t*>(&h23);
          lw.x = *reinterpret_cast<const uint32_t*>(&l01), lw.y = *reinterpret_cast<const uint32_t*>(&l23);
          if (inr) {
            *reinterpret_cast<uint2*>(hi + r * 4) = hw;
            *reinterpret_cast<uint2*>(lo + r * 4) = lw;
          }
        }
      }
      if (F16 && big > 65504.f) atomicOr(a.status, kStatusF16Range);
      fenceProxyAsync();  // generic-proxy stores -> visible to the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) {
        mbarArrive(&bFull[buf]);
        if (tmaIn) mbarArrive(&rawEmpty[rawBuf]);  // the raw buffer may be refilled
      }
      if (kProf) cTr += clock64() - tTr;
      t = tn, c = cn, pos0 = posN;
      if (++rawBuf == NRAW) rawBuf = 0, rawPar ^= 1;
      if (++buf == uint32_t(NB)) buf = 0, bufPar ^= 1;
    }
    cpAsyncWait<0>();
    if (kProf && pw == 0) profAdd(10, wB), profAdd(11, wCp), profAdd(12, cTr), profAdd(13, clock64() - tStart);
  } else {
    regDec<CTL_REGS>();
    if (warp == W_WARP) {
      // ---------------------------------------------------------------- weight producer
      uint32_t wIt = 0, ws = 0, wPh = 1;  // stages issued, ring slot, parity of the slot's previous release
      bool dead = false;
      long long wW = 0;
      const long long tStart = kProf ? clock64() : 0;
      const int64_t blocksPerCo = int64_t(nChunks16) * a.k;  // one block (hi + lo of one tap) per chunk and tap
      const int slotFloats = a.wG * W_STAGE_FLOATS;
      for (int t = blockIdx.x; t < numTiles && !dead; t += gridDim.x) {
        const int tt = t / a.numCoBlk, cb = t - tt * a.numCoBlk;
        const float* src = a.wp + int64_t(cb) * blocksPerCo * W_STAGE_FLOATS;
        for (int c = 0; c < nChunks16 && !dead; ++c) {
          for (int gi = 0; gi < nTapGroups; ++gi, ++wIt) {
            const int n = tgBase + (gi < tgExtra ? 1 : 0);
            if (!waitT(&wEmpty[ws], wPh, wW, SLEEP_W_NS)) {
              giveUp(3, 1);
              dead = true;
              break;
            }
            if (lane == 0) {
              mbarArriveExpectTx(&wFull[ws], n * W_STAGE_BYTES);
              bulkCopyG2S(sW + ws * slotFloats, src, n * W_STAGE_BYTES, &wFull[ws]);
            }
            __syncwarp();
            src += n * W_STAGE_FLOATS;
            if (++ws == uint32_t(a.wStages)) ws = 0, wPh ^= 1;  // wrap counters: a division here cost more than the copy
          }
        }
      }
      if (kProf) profAdd(14, wW), profAdd(15, clock64() - tStart);
      // Every copy this warp issued must have landed before the CTA may exit. On the normal path the MMA warp has
      // consumed them all; after an abort, wait (bounded) for the stages still in flight.
      if (*abortFlag) {
        const uint32_t issued = wIt;
        for (uint32_t i = issued > uint32_t(a.wStages) ? issued - a.wStages : 0; i < issued; ++i)
          mbarWaitQuiet(&wFull[i % a.wStages], (i / a.wStages) & 1);
      }
    } else if (warp == RAW_WARP) {
      // ---------------------------------------------------------------- raw-window loader (aligned route)
      // Per (tile, chunk): the 16 channels' windows [pos0 & ~3, + 2 half) as two boxes of `half` columns (a box
      // holds at most 256 elements per dimension). Columns outside [0, L) arrive as zeros and are never used: the
      // producers write the zero padding themselves, after the activation.
      if (a.tmaIn && lane == 0) {
        uint32_t rb = 0, ph = 1, issued = 0;
        long long wR = 0;
        bool dead = false;
        const uint32_t bytes = uint32_t(rawBufFloats) * 4;
        for (int t = blockIdx.x; t < numTiles && !dead; t += gridDim.x) {
          const int64_t pos0 = int64_t(t / a.numCoBlk) * NT - a.padding;
          const int x0 = int(pos0 - (pos0 & 3));
          for (int c = 0; c < nChunks16; ++c, ++issued) {
            if (!waitT(&rawEmpty[rb], ph, wR, SLEEP_W_NS)) {
              giveUp(5, 1);
              dead = true;
              break;
            }
            float* dst = sRaw + rb * rawBufFloats;
            mbarArriveExpectTx(&rawFull[rb], bytes);
            tmaLoad2d(dst, &mapX, x0, c * KC, &rawFull[rb]);
            tmaLoad2d(dst + KC * half, &mapX, x0 + half, c * KC, &rawFull[rb]);
            if (++rb == NRAW) rb = 0, ph ^= 1;
          }
        }
        if (*abortFlag) {
          for (uint32_t i = issued > NRAW ? issued - NRAW : 0; i < issued; ++i)
            mbarWaitQuiet(&rawFull[i % NRAW], (i / NRAW) & 1);
        }
      }
    } else if (warp == MMA_WARP) {
      // ---------------------------------------------------------------- MMA issuer
      // One thread issues every MMA: hi*hi into Dhi, lo*hi and hi*lo into Dlo. It walks the (tile, chunk, tap group)
      // sequence, one tap group per round: a single wait for the group's weight slot, its MMAs back to back, a single
      // release. Measured on this part: a lone thread streams MMAs at the pipe's rate (128 clocks for M128 N256 K16)
      // as long as nothing but MMAs is issued; the thread is held while an MMA waits for the pipe, and what it
      // executes between two MMAs is covered by no more than the one MMA in flight. So the bookkeeping for the next
      // round (ring counters, a first poll of the next slot's barrier) sits where it is free, and only the release
      // and, rarely, a real wait separate two rounds.
      // Order inside a round: the lo MMAs first, then the hi MMAs, so that the wait for the Dhi drain at the start
      // of a drain group is covered by the round's own lo MMAs. The first round of a tile goes the other way round,
      // because there Dhi is handed back before Dlo. (Issuing hi first in the last round of a drain group as well,
      // which lengthens the cover of the drain to this round's and the next round's lo MMAs, shortened the waits
      // but not the tile: the extra code in this loop cost what the waits gave back.)
      const uint64_t dA0 = makeDesc(smemAddr(sW), MT * 16, 128);
      const uint64_t dB0 = makeDesc(smemAddr(sAct), rows * 16, 128);
      constexpr uint32_t kStageU = W_STAGE_BYTES >> 4, kLoAU = (W_STAGE_BYTES / 2) >> 4, kKsAU = (2 * MT * 16) >> 4;
      // activation buffer: hi half then lo half; one MMA spans two 16-byte K chunks (K8 of f32 or K16 of f16);
      // one staged time row = 16 bytes = one descriptor address unit
      const uint32_t bufU = uint32_t(actBufFloats * 4) >> 4, loBU = bufU >> 1, ksBU = 2 * uint32_t(rows);
      const uint32_t slotU = uint32_t(a.wG) * kStageU;
      const int dil = a.dilation, wStages = a.wStages, drainN = a.drainN;
      int slot = 0, buf = 0, g = 0;
      uint32_t slotPh = 0, bufPh = 0, groupPar = 0, tilePar = 0;
      bool dead = false, ready = false;  // ready: the next round's weight slot is already known to be full
      long long wBf = 0, wHe = 0, wWf = 0, wLe = 0;
      const long long tStart = kProf ? clock64() : 0;
      for (int tile = blockIdx.x; lane == 0 && tile < numTiles && !dead; tile += gridDim.x) {
        for (int c = 0; c < nChunks16 && !dead; ++c) {
          if (!waitT(&bFull[buf], bufPh, wBf, SLEEP_MMA_NS)) {
            giveUp(4, 2);
            dead = true;
            break;
          }
          const uint64_t dBc = dB0 + uint32_t(buf) * bufU;
          int kk = 0;
          for (int gi = 0; gi < nTapGroups; ++gi) {
            const int gN = tgBase + (gi < tgExtra ? 1 : 0);
            if (!ready && !waitT(&wFull[slot], slotPh, wWf, SLEEP_MMA_NS)) {
              giveUp(4, 3);
              dead = true;
              break;
            }
            tcFenceAfter();
            const uint64_t dA = dA0 + uint32_t(slot) * slotU, dB = dBc + uint32_t(kk * dil);
            const uint32_t accHi = (kk | g) == 0 ? 0u : 1u, accLo = (kk | c) == 0 ? 0u : 1u;
            const bool needHi = (kk | g) == 0, needLo = (kk | c) == 0;  // Dhi drained / Dlo of the last tile folded
            const uint32_t aLo = uint32_t(dA), aHi = uint32_t(dA >> 32), bLo = uint32_t(dB), bHi = uint32_t(dB >> 32);
            // Rolled issue loops: the issuer's code between two MMAs has to be fetched and issued while at most one
            // MMA is in flight, so the loops are kept to a handful of instructions and exist once per order.
            auto issueHi = [&](uint32_t acc) {
              if constexpr (F16) {
                uint32_t aj = aLo, bj = bLo;
#pragma unroll 1
                for (int j = 0; j < gN; ++j, aj += kStageU, bj += uint32_t(dil), acc = 1u)
                  mmaF16W(tmemHi, aj, aHi, bj, bHi, kIdescF16, acc);
              } else {
                uint64_t dAh = dA, dBh = dB;
#pragma unroll 1
                for (int j = 0; j < gN; ++j, dAh += kStageU, dBh += uint32_t(dil), acc = 1u) {
                  mmaTf32(tmemHi, dAh, dBh, kIdesc, acc);
                  mmaTf32(tmemHi, dAh + kKsAU, dBh + ksBU, kIdesc, 1u);
                }
              }
            };
            auto issueLo = [&](uint32_t acc) {
              if constexpr (F16) {
                uint32_t aj = aLo, bj = bLo;
#pragma unroll 1
                for (int j = 0; j < gN; ++j, aj += kStageU, bj += uint32_t(dil), acc = 1u) {
                  mmaF16W(tmemLo, aj + kLoAU, aHi, bj, bHi, kIdescF16, acc);
                  mmaF16W(tmemLo, aj, aHi, bj + loBU, bHi, kIdescF16, 1u);
                }
              } else {
                uint64_t dAh = dA, dBh = dB;
#pragma unroll 1
                for (int j = 0; j < gN; ++j, dAh += kStageU, dBh += uint32_t(dil), acc = 1u) {
                  const uint64_t dAl = dAh + kLoAU, dBl = dBh + loBU;
                  mmaTf32(tmemLo, dAl, dBh, kIdesc, acc);
                  mmaTf32(tmemLo, dAh, dBl, kIdesc, 1u);
                  mmaTf32(tmemLo, dAl + kKsAU, dBh + ksBU, kIdesc, 1u);
                  mmaTf32(tmemLo, dAh + kKsAU, dBl + ksBU, kIdesc, 1u);
                }
              }
            };
            int nslot = slot + 1;
            uint32_t nph = slotPh;
            if (nslot == wStages) nslot = 0, nph ^= 1;
            const bool lastRound = c == nChunks16 - 1 && gi == nTapGroups - 1;  // of the tile
            if (needLo) {  // first round of a tile: hi, then lo (Dhi is handed back before Dlo)
              if (needHi && !waitT(hiEmpty, groupPar ^ 1, wHe, SLEEP_MMA_NS)) {
                giveUp(4, 1);
                dead = true;
                break;
              }
              tcFenceAfter();
              issueHi(accHi);
              if (!waitT(loEmpty, tilePar ^ 1, wLe, SLEEP_MMA_NS)) {
                giveUp(4, 4);
                dead = true;
                break;
              }
              tcFenceAfter();
              issueLo(accLo);
              if (lastRound) mmaCommit(loFull);
            } else {
              issueLo(accLo);
              // the tile's lo chain is complete: the epilogue folds Dlo under the hi MMAs of this last round
              if (lastRound) mmaCommit(loFull);
              if (needHi) {
                if (!waitT(hiEmpty, groupPar ^ 1, wHe, SLEEP_MMA_NS)) {
                  giveUp(4, 1);
                  dead = true;
                  break;
                }
                tcFenceAfter();
              }
              issueHi(accHi);
            }
            // first poll of the next slot's barrier, with the whole round queued behind it
            ready = mbarTryWait(&wFull[nslot], nph);
            mmaCommit(&wEmpty[slot]);  // weight slot free once the MMAs have read it
            kk += gN;
            slot = nslot, slotPh = nph;
          }
          if (dead) break;
          const bool lastChunk = c == nChunks16 - 1;
          // the hi chain of a drain group (drainN chunks, or what is left of the tile) is complete
          if (g == drainN - 1 || lastChunk) mmaCommit(hiFull);
          mmaCommit(&bEmpty[buf]);  // activation buffer free once the MMAs have read it
          if (++buf == NB) buf = 0, bufPh ^= 1;
          if (++g == drainN || lastChunk) g = 0, groupPar ^= 1;
        }
        tilePar ^= 1;
      }
      __syncwarp();
      if (kProf) profAdd(0, wBf), profAdd(1, wHe), profAdd(2, wWf), profAdd(3, wLe), profAdd(4, clock64() - tStart);
    }
  }

  tcFenceBefore();
  __syncthreads();
  if (warp == MMA_WARP) {
    tcFenceAfter();
    tmemDealloc(tmemBase, 512);
  }
}

// One packed element: tf32 split -> f32 hi or lo; f16 split -> f16 hi or lo (lo scaled by 2^11).
__device__ __forceinline__ float splitTf32(float v, int part) {
  const float h = tf32Round(v);
  return part == 0 ? h : v - h;
}
// A weight beyond the f16 range is clamped and reported through the status word (kStatusF16Weights): the caller then
// packs this weight in the tf32 format, which has the range of f32.
__device__ __forceinline__ __half splitF16(float v, int part, int* status) {
  if (part == 0 && fabsf(v) > 65504.f) atomicOr(status, kStatusF16Weights);
  const __half h = __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
  return part == 0 ? h : __float2half_rn((v - __half2float(h)) * kLoScale);
}

// Conv weight pack: stage (cb, c16, kk) = [hi | lo], each [16-byte K chunk][128 rows][chunk elements]
// (4 f32 or 8 f16 per chunk). Rows past Co are zero.
template <bool F16>
__global__ void packWeightsKernel(const float* __restrict__ w, void* __restrict__ wpOut, int co, int ci, int k,
                                  int* status) {
  constexpr int CE = F16 ? 8 : 4, NCH = KC / CE;  // elements per chunk, chunks per 16 channels
  const int nC16 = ci / KC;
  const int64_t n = int64_t((co + MT - 1) / MT) * nC16 * k * 2 * NCH * MT * CE;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < n; idx += int64_t(gridDim.x) * blockDim.x) {
    int64_t r = idx;
    const int e = int(r % CE);
    r /= CE;
    const int col = int(r % MT);
    r /= MT;
    const int kc = int(r % NCH);
    r /= NCH;
    const int part = int(r % 2);
    r /= 2;
    const int kk = int(r % k);
    r /= k;
    const int c16 = int(r % nC16);
    const int cb = int(r / nC16);
    const int row = cb * MT + col;
    const float v = row < co ? w[(int64_t(row) * ci + (c16 * KC + kc * CE + e)) * k + kk] : 0.f;
    if constexpr (F16) static_cast<__half*>(wpOut)[idx] = splitF16(v, part, status);
    else static_cast<float*>(wpOut)[idx] = splitTf32(v, part);
  }
}

// Polyphase ConvTranspose1d (K = 2 s, 2 p = s) on the same kernel: out[co, j s + r] = sum_c sum_tt Wr[r][co][c][tt] *
// leaky(x)[c, j + q_r - 1 + tt], q_r = (r + p) div s, is a 3-tap conv over the window (j - 1, j, j + 1) whose output rows
// are (channel, phase) pairs: window tap wt carries Wr[..][tt = wt - q_r] when that is 0 or 1 and zero otherwise (one
// of the three taps of every row is zero). Rows are grouped so that each epilogue warp (32 accumulator rows) owns
// CQ = 32 / s whole channels with all their phases (row = cl * s + r, the last 32 - CQ s rows are zero), which lets it
// write each channel's samples j s + r as one contiguous run. One 128-row block therefore holds 4 CQ channels.
template <bool F16>
__global__ void convtTcPackKernel(const float* __restrict__ w, void* __restrict__ wpOut, int ci, int co, int k, int s,
                                  int p, int* status) {
  constexpr int CE = F16 ? 8 : 4, NCH = KC / CE;
  const int nC16 = ci / KC, cq = 32 / s, cpb = 4 * cq;
  const int64_t n = int64_t((co + cpb - 1) / cpb) * nC16 * 3 * 2 * NCH * MT * CE;
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < n; idx += int64_t(gridDim.x) * blockDim.x) {
    int64_t r = idx;
    const int e = int(r % CE);
    r /= CE;
    const int row = int(r % MT);
    r /= MT;
    const int kc = int(r % NCH);
    r /= NCH;
    const int part = int(r % 2);
    r /= 2;
    const int wt = int(r % 3);
    r /= 3;
    const int c16 = int(r % nC16);
    const int cb = int(r / nC16);
    const int q = row / 32, i = row % 32, cl = i / s, ph = i % s;
    const int o = (cb * 4 + q) * cq + cl, c = c16 * KC + kc * CE + e;
    const int tt = wt - (ph + p) / s;
    float v = 0.f;
    if (i < cq * s && o < co && (tt == 0 || tt == 1)) v = w[(int64_t(c) * co + o) * k + (ph + p) % s + (1 - tt) * s];
    if constexpr (F16) static_cast<__half*>(wpOut)[idx] = splitF16(v, part, status);
    else static_cast<float*>(wpOut)[idx] = splitTf32(v, part);
  }
}

}  // namespace

// Raw staging: every channel's window of rows + 3 floats (the slack of the 16-byte alignment) is kept as two runs of
// `half` floats, half a multiple of 4 and at most 256 (one TMA box each).
static int rawHalf(int rows) { return (((rows + 3 + 1) / 2) + 3) & ~3; }

// Dynamic shared memory of one CTA and the weight ring it leaves room for: the largest taps-per-slot (<= TAP_GROUP)
// that still gives PREF_W_STAGES slots, else the deepest ring. Returns 0 when even single-tap slots do not fit.
static size_t convTcSmemBytes(int64_t ci, int rows, int k, bool f16, int* wStages, int* wG) {
  const int tap = f16 ? Fmt<true>::W_STAGE_BYTES : Fmt<false>::W_STAGE_BYTES;
  const int actRow = f16 ? Fmt<true>::ACT_BYTES_PER_ROW : Fmt<false>::ACT_BYTES_PER_ROW;
  const int nb = f16 ? Fmt<true>::NB : Fmt<false>::NB;
  const int half = rawHalf(rows);
  if (half > 256) return 0;
  const SmemLayout base = smemLayout(int(ci), rows, half, nb, 0, 0, actRow, tap);
  if (base.total > uint32_t(kMaxSmem)) return 0;
  const size_t avail = size_t(kMaxSmem) - base.total;
  // Large groups matter more than a deep ring (measured: two slots of four taps beat four slots of three, and at
  // K = 11 two slots of six beat three of four).
  int bestG = 0, bestWs = 0;
  for (int g = TAP_GROUP; g >= 1; --g) {
    const int groups = (k + g - 1) / g, gmax = (k + groups - 1) / groups;  // near-equal groups, the largest has gmax taps
    int ws = int(avail / (size_t(gmax) * tap));
    if (ws > MAX_W_STAGES) ws = MAX_W_STAGES;
    if (ws >= PREF_W_STAGES) {
      bestG = gmax, bestWs = ws;
      break;
    }
    if (ws >= MIN_W_STAGES && ws > bestWs) bestG = gmax, bestWs = ws;
  }
  if (bestG == 0) return 0;
  if (wStages) *wStages = bestWs;
  if (wG) *wG = bestG;
  return smemLayout(int(ci), rows, half, nb, bestWs, bestG, actRow, tap).total;
}

// The hi chain between two drains holds at most MAX_CHAIN MMAs: whole chunks while they fit, and a chunk that alone
// has more (K > 24 with f16 halves, K > 12 with tf32 halves) goes to the CUDA-core kernel, so the chain (and the
// truncation drift it accumulates, about 1.5e-8 of the result per MMA: 3.7e-7 at 24) stays bounded.
static bool chainOk(int64_t k, bool f16) { return k * (f16 ? 1 : 2) <= MAX_CHAIN; }

bool convTcEligible(const ConvFusedParams& p, bool f16) {
  if (!(p.state != nullptr && p.x2 == nullptr && p.ci % KC == 0 && p.co >= 1 && p.ci >= KC && p.k >= 1 &&
        chainOk(p.k, f16) && (p.k - 1) * p.dilation <= MAX_HALO && p.lo >= 1 && p.padding <= (1 << 20) && p.ci <= 4096 &&
        p.l < (int64_t(1) << 30)))
    return false;
  return convTcSmemBytes(p.ci, NT + int((p.k - 1) * p.dilation), int(p.k), false, nullptr, nullptr) != 0;  // the larger format
}

int64_t convTcPackFloats(int64_t co, int64_t ci, int64_t k, bool f16) {
  return ((co + MT - 1) / MT) * (ci / KC) * k * (f16 ? Fmt<true>::W_STAGE_FLOATS : Fmt<false>::W_STAGE_FLOATS);
}

// Per-device constants, looked up once (the first call on a device must not be inside a stream capture).
struct DeviceInfo {
  int* status = nullptr;
  long long* prof = nullptr;
  int smCount = 0;
};
static int deviceInfo(const DeviceInfo** out) {
  static DeviceInfo info[64];
  int dev = 0;
  cudaGetDevice(&dev);
  LKC_REQUIRE(dev >= 0 && dev < 64, "conv (tensor-core): device index out of range");
  DeviceInfo& d = info[dev];
  if (!d.status) {
    int* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), gTcStatus);
    if (e != cudaSuccess) return failCuda("conv (tensor-core): cudaGetSymbolAddress", e);
    e = cudaDeviceGetAttribute(&d.smCount, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return failCuda("conv (tensor-core): cudaDeviceGetAttribute", e);
    long long* pp = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&pp), gTcProf);
    if (e != cudaSuccess) return failCuda("conv (tensor-core): cudaGetSymbolAddress", e);
    d.prof = pp;
    d.status = ptr;
  }
  *out = &d;
  return 0;
}

int convTcPack(const float* w, float* wp, int64_t co, int64_t ci, int64_t k, bool f16, cudaStream_t s) {
  LKC_REQUIRE(ci % KC == 0 && co > 0 && ci > 0 && k >= 1 && k <= 64,
              "conv1d_tc_pack_f32_cuda: needs Ci % 16 == 0, 1 <= K <= 64");
  const DeviceInfo* d = nullptr;
  if (int rc = deviceInfo(&d)) return rc;
  const int64_t n = convTcPackFloats(co, ci, k, f16) * (f16 ? 2 : 1);  // packed elements
  const int blocks = static_cast<int>(ceilDiv(n, 256) > 4096 ? 4096 : ceilDiv(n, 256));
  if (f16) packWeightsKernel<true><<<blocks, 256, 0, s>>>(w, wp, int(co), int(ci), int(k), d->status);
  else packWeightsKernel<false><<<blocks, 256, 0, s>>>(w, wp, int(co), int(ci), int(k), d->status);
  return launched("conv1d_tc_pack_f32_cuda");
}

// ---- tensor maps (cuTensorMapEncodeTiled, looked up through the runtime: the library does not link libcuda)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encodeTiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    cudaGetLastError();
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
static bool gTmaEnabled = true;  // lkc_set_conv_io: false forces the 4-byte route (A/B testing)

// Map of an f32 [rowsC, cols] tensor with row pitch `pitch` floats; box = boxCols x boxRows. False when the tensor's
// rows are not 16-byte aligned (or the driver entry point is missing): the caller then takes the 4-byte route.
static bool makeMap(CUtensorMap* map, const float* base, int64_t rowsC, int64_t cols, int64_t pitch, int boxCols,
                    int boxRows, bool swizzle128) {
  if (!gTmaEnabled || !base || (reinterpret_cast<uintptr_t>(base) & 15) || (pitch & 3) || pitch < cols || cols < 1 ||
      rowsC < 1 || cols >= (int64_t(1) << 31))
    return false;
  EncodeTiledFn fn = encodeTiled();
  if (!fn) return false;
  const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rowsC)};
  const cuuint64_t strides[1] = {cuuint64_t(pitch) * 4};
  const cuuint32_t box[2] = {cuuint32_t(boxCols), cuuint32_t(boxRows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int convTcSetIo(int mode) {
  LKC_REQUIRE(mode == 0 || mode == 1, "set_conv_io: mode must be 0 (TMA where rows are aligned) or 1 (4-byte route only)");
  gTmaEnabled = mode == 0;
  return 0;
}

struct TcMaps {
  CUtensorMap x, res, out;
};

template <int ACT, bool PARTIAL, int TS, bool F16, bool TMAO>
static int launchTc4(const TcArgs& a, const TcMaps& m, int grid, size_t smem, cudaStream_t s) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(convTcKernel<ACT, PARTIAL, TS, F16, TMAO>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return failCuda("conv (tensor-core): cudaFuncSetAttribute", e);
    configured[dev] = true;
  }
  convTcKernel<ACT, PARTIAL, TS, F16, TMAO><<<grid, NTHREADS, smem, s>>>(a, m.x, m.res, m.out);
  return launched("conv (tensor-core)");
}

template <int ACT, bool PARTIAL, int TS, bool F16>
static int launchTc3(const TcArgs& a, const TcMaps& m, int grid, size_t smem, cudaStream_t s) {
  if constexpr (TS == 0 && !PARTIAL) {
    if (a.tmaOut) return launchTc4<ACT, PARTIAL, TS, F16, true>(a, m, grid, smem, s);
  }
  return launchTc4<ACT, PARTIAL, TS, F16, false>(a, m, grid, smem, s);
}

template <int ACT, bool PARTIAL, int TS = 0>
static int launchTc2(const TcArgs& a, const TcMaps& m, bool f16, int grid, size_t smem, cudaStream_t s) {
  return f16 ? launchTc3<ACT, PARTIAL, TS, true>(a, m, grid, smem, s) : launchTc3<ACT, PARTIAL, TS, false>(a, m, grid, smem, s);
}

template <int ACT>
static int launchTc(const TcArgs& a, const TcMaps& m, bool f16, int grid, size_t smem, cudaStream_t s) {
  return a.co % MT == 0 ? launchTc2<ACT, false>(a, m, f16, grid, smem, s) : launchTc2<ACT, true>(a, m, f16, grid, smem, s);
}

static bool gProfileOn = false;

// Profiling counters of the tensor-core kernel (cycles, summed over CTAs and launches since the last reset; one
// representative warp per role): [0..4] MMA warp: wait activations, wait Dhi drained, wait weights, wait Dlo folded,
// total; [5..9] epilogue warp 0: wait Dhi, wait Dlo, residual preload, final phase, total; [10..13] producer warp 0:
// wait buffer free, wait raw window, transform, total; [14..15] weight producer: wait stage free, total.
int convTcProfile(int enable, long long* out16) {
  LKC_REQUIRE(kProf, "conv1d_tc_profile: the library was built without -DLKC_TC_PROF=1");
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return failCuda("conv1d_tc_profile: cudaDeviceSynchronize", e);
  gProfileOn = enable != 0;
  if (out16) {
    e = cudaMemcpyFromSymbol(out16, gTcProf, sizeof(long long) * 16);
    if (e != cudaSuccess) return failCuda("conv1d_tc_profile", e);
  }
  static const long long zeros[16] = {};
  e = cudaMemcpyToSymbol(gTcProf, zeros, sizeof zeros);
  if (e != cudaSuccess) return failCuda("conv1d_tc_profile", e);
  return 0;
}

// Launch geometry and tensor maps shared by the conv and ConvTranspose entry points.
static int finishArgs(TcArgs& a, TcMaps& m, bool f16, bool boxesOk, int* grid, size_t* smem) {
  *smem = convTcSmemBytes(a.ci, a.rows, a.k, f16, &a.wStages, &a.wG);
  LKC_REQUIRE(*smem != 0, "conv (tensor-core): window too large");
  a.half = rawHalf(a.rows);
  a.nb = f16 ? Fmt<true>::NB : Fmt<false>::NB;
  const DeviceInfo* d = nullptr;
  if (int rc = deviceInfo(&d)) return rc;
  a.status = d->status;
  a.prof = (kProf && gProfileOn) ? d->prof : nullptr;
  // Dhi is drained into the f32 running sums after as many whole chunks as fit in MAX_CHAIN chained MMAs.
  const int perChunk = a.k * (f16 ? 1 : 2);
  const int n = MAX_CHAIN / perChunk;
  a.drainN = n < 1 ? 1 : n;
  // Launches with at most 15 MMAs per chunk (K <= 5 with f16 halves; the ConvTranspose launches: three taps) are
  // bound by the activation producers: they take the balanced warp layout (measured at K = 3: the transform of a
  // chunk 17 % faster, the launch 4-7 %; at K = 7 the isolated layout is 3 % ahead).
  a.balanced = a.k * (f16 ? 3 : 6) <= 15 ? 1 : 0;
  const int tiles = a.numTTiles * a.numCoBlk;
  *grid = tiles < d->smCount ? tiles : d->smCount;
  // TMA routes: tensors whose rows are 16-byte aligned. A map that is not used still has to be a valid kernel
  // argument: it stays zero-filled and is never dereferenced.
  std::memset(&m, 0, sizeof m);
  a.tmaIn = makeMap(&m.x, a.x, a.ci, a.l, a.xPitch, a.half, KC, false) ? 1 : 0;
  a.tmaOut = 0;
  if (boxesOk && a.co % MT == 0 && makeMap(&m.out, a.out, a.co, a.lo, a.outPitch, BOX, BOX, true) &&
      (!a.residual || makeMap(&m.res, a.residual, a.co, a.lo, a.resPitch, BOX, BOX, true)))
    a.tmaOut = 1;
  return 0;
}

int convTc(const ConvFusedParams& p, const float* wp, bool f16, cudaStream_t s) {
  TcArgs a;
  TcMaps m;
  a.x = p.x, a.wp = wp, a.bias = p.bias, a.affine = p.affine, a.alpha = p.alpha, a.residual = p.residual;
  a.out = p.out, a.stats = p.stats;
  a.ci = int(p.ci), a.co = int(p.co), a.k = int(p.k), a.dilation = int(p.dilation), a.padding = int(p.padding);
  a.l = p.l, a.lo = p.lo, a.nchunks = p.statsStride ? p.statsStride : statChunks(p.lo), a.padLeft = 0;
  a.padding = int(p.padding - p.xOrigin);  // window row 0 of output column t is x column t - padding + xOrigin
  a.validLo = p.validLo, a.validHi = p.validHi < 0 ? p.l : p.validHi;
  a.xPitch = p.xPitch ? p.xPitch : p.l, a.resPitch = p.resPitch ? p.resPitch : p.lo;
  a.outPitch = p.outPitch ? p.outPitch : p.lo;
  a.slope = p.slope, a.outScale = p.outScale;
  a.rows = NT + (a.k - 1) * a.dilation;
  const int64_t tTiles = ceilDiv(p.lo, NT);
  const int64_t coBlk = ceilDiv(p.co, MT);  // output channels past Co are zero rows of the pack and never stored
  LKC_REQUIRE(tTiles * coBlk < (1 << 30), "conv (tensor-core): too many tiles");
  a.numTTiles = int(tTiles), a.numCoBlk = int(coBlk);
  int grid = 0;
  size_t smem = 0;
  if (int rc = finishArgs(a, m, f16, true, &grid, &smem)) return rc;
  switch (p.act) {
    case Act::None: return launchTc<0>(a, m, f16, grid, smem, s);
    case Act::Snake: return launchTc<1>(a, m, f16, grid, smem, s);
    case Act::Leaky: return launchTc<2>(a, m, f16, grid, smem, s);
  }
  return fail("conv (tensor-core): bad activation");
}

// ---- polyphase ConvTranspose1d on the tensor-core kernel

bool convtTcEligible(int64_t ci, int64_t co, int64_t k, int64_t stride, int64_t padding) {
  return (stride == 6 || stride == 10) && k == 2 * stride && 2 * padding == stride && ci % KC == 0 && ci >= KC &&
         ci <= 4096 && co >= 1 && convTcSmemBytes(ci, NT + 2, 3, false, nullptr, nullptr) != 0;
}

int64_t convtTcPackFloats(int64_t ci, int64_t co, int64_t stride, bool f16) {
  const int64_t cpb = 4 * (32 / stride);
  return ceilDiv(co, cpb) * (ci / KC) * 3 * (f16 ? Fmt<true>::W_STAGE_FLOATS : Fmt<false>::W_STAGE_FLOATS);
}

int convtTcPack(const float* w, float* wp, int64_t ci, int64_t co, int64_t k, int64_t stride, int64_t padding,
                bool f16, cudaStream_t s) {
  LKC_REQUIRE(convtTcEligible(ci, co, k, stride, padding),
              "convt_tc_pack_f32_cuda: needs stride 6 or 10, K = 2 stride, 2 padding = stride, Ci % 16 == 0");
  const DeviceInfo* d = nullptr;
  if (int rc = deviceInfo(&d)) return rc;
  const int64_t n = convtTcPackFloats(ci, co, stride, f16) * (f16 ? 2 : 1);
  const int blocks = static_cast<int>(ceilDiv(n, 256) > 4096 ? 4096 : ceilDiv(n, 256));
  if (f16)
    convtTcPackKernel<true><<<blocks, 256, 0, s>>>(w, wp, int(ci), int(co), int(k), int(stride), int(padding), d->status);
  else
    convtTcPackKernel<false><<<blocks, 256, 0, s>>>(w, wp, int(ci), int(co), int(k), int(stride), int(padding), d->status);
  return launched("convt_tc_pack_f32_cuda");
}

int convtTc(const ConvtParams& p, const float* wp, bool f16, cudaStream_t s) {
  TcArgs a;
  TcMaps m;
  a.x = p.x, a.wp = wp, a.bias = p.bias, a.affine = nullptr, a.alpha = nullptr, a.residual = p.res;
  a.out = p.out, a.stats = nullptr;
  // x holds haloLeft + l + haloRight columns; output (input-rate) column j reads x columns j + haloLeft + {-1, 0, 1}
  const int64_t lx = p.haloLeft + p.l + p.haloRight;
  a.ci = int(p.ci), a.co = int(p.co), a.k = 3, a.dilation = 1, a.padding = int(1 - p.haloLeft);
  const int64_t lo = p.l * p.stride + p.padLeft;
  a.l = lx, a.lo = p.l, a.nchunks = 0, a.padLeft = int(p.padLeft);
  a.validLo = 0, a.validHi = lx;
  a.xPitch = p.xPitch ? p.xPitch : lx, a.resPitch = p.resPitch ? p.resPitch : lo, a.outPitch = p.outPitch ? p.outPitch : lo;
  a.slope = p.slope, a.outScale = 1.f;
  a.rows = NT + 2;
  const int64_t tTiles = ceilDiv(p.l, NT), coBlk = ceilDiv(p.co, 4 * (32 / p.stride));
  LKC_REQUIRE(tTiles * coBlk < (1 << 30) && p.l < (int64_t(1) << 30), "conv_transpose1d_poly (tensor-core): too many tiles");
  a.numTTiles = int(tTiles), a.numCoBlk = int(coBlk);
  int grid = 0;
  size_t smem = 0;
  if (int rc = finishArgs(a, m, f16, false, &grid, &smem)) return rc;
  if (p.stride == 6) return launchTc2<2, false, 6>(a, m, f16, grid, smem, s);
  return launchTc2<2, false, 10>(a, m, f16, grid, smem, s);
}

// Reads (and optionally clears) the status word after all work queued on the device has finished: the kernels run on
// the caller's streams, which the default stream does not wait for, so the whole device is synchronised first.
int convTcStatus(int* out, bool reset) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return failCuda("conv1d_tc_status: cudaDeviceSynchronize", e);
  int v = 0;
  e = cudaMemcpyFromSymbol(&v, gTcStatus, sizeof v);
  if (e != cudaSuccess) return failCuda("conv1d_tc_status", e);
  if (reset && v != 0) {
    const int z = 0;
    e = cudaMemcpyToSymbol(gTcStatus, &z, sizeof z);
    if (e != cudaSuccess) return failCuda("conv1d_tc_status", e);
  }
  *out = v;
  return 0;
}

// Stream-ordered read of the status word: queues a 4-byte copy into `hostOut` (pinned host memory) behind the work
// already on `s`; nothing is synchronised and nothing is cleared. The caller looks at *hostOut after it has
// synchronised with `s` (an event, a stream synchronise).
int convTcStatusAsync(int* hostOut, cudaStream_t s) {
  const DeviceInfo* d = nullptr;
  if (int rc = deviceInfo(&d)) return rc;
  const cudaError_t e = cudaMemcpyAsync(hostOut, d->status, sizeof(int), cudaMemcpyDeviceToHost, s);
  return e == cudaSuccess ? 0 : failCuda("conv1d_tc_status_async: cudaMemcpyAsync", e);
}

}  // namespace lkc
