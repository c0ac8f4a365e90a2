// Exchange step of a time-sharded utterance: one GPU owns a contiguous time range of every activation tensor and keeps
// a margin of halo columns on both sides of it. After a kernel has produced a tensor's columns, the producer pushes
//   - its boundary columns into the neighbours' margins (the receptive-field halo of the next conv), and
//   - its slice of the per-(channel, 128-column chunk) statistics into every rank's copy of the full statistics
//     row (AdaIN needs the mean / variance over the whole utterance; every rank then runs the same exact combine),
// with plain stores to peer memory (mapped through CUDA IPC; no multicast, no library kernel ever sees a peer
// pointer), followed by one release store per destination flag. Consumers wait on their own flags before they read.
// The reference has no multi-GPU path; the semantics that must be preserved are the conv's (zero padding applied after
// the activation, only at the ends of the utterance: kernels/cpu/kokoro_conv_fused.cpp:127-135) and the statistics'
// (chunk grid from t = 0, exact combine in double: kokoro_conv_fused.cpp:641-664).
//
// Flags carry an epoch number (one per forward, bumped by epochBumpKernel), so a captured sequence can be replayed:
// nothing in the launch arguments changes between forwards. Every wait is bounded: when the limit runs out the wait
// kernel records a status word and returns; later kernels then run on stale halos and the host reports the status.
#include <cstring>

#include "lkc_common.h"

namespace lkc {
namespace {

constexpr int kMaxCopies = LKC_SHARD_MAX_COPIES, kMaxFlags = LKC_SHARD_MAX_FLAGS;

struct PushArgs {
  const float* src[kMaxCopies];
  float* dst[kMaxCopies];
  int64_t srcPitch[kMaxCopies], dstPitch[kMaxCopies];
  int rows[kMaxCopies], cols[kMaxCopies];
  int numCopies;
  int* flags[kMaxFlags];
  int numFlags;
  const int* epoch;
  unsigned* ticket;
  // exchange form: after its own flags are out, the last block waits for these (numWait = 0: push only)
  const int* waitFlags[kMaxFlags];
  int numWait, delta;
  unsigned long long limitNs;
  int* status;
};

__device__ __forceinline__ void storeReleaseSys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int loadAcquireSys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t timerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Gives up after limitNs: status |= 1 << 24 | flag index (first one wins the index bits).
__device__ __forceinline__ void waitFlag(const int* flag, int f, int want, unsigned long long limitNs, int* status) {
  const uint64_t t0 = timerNs();
  unsigned spins = 0;
  while (loadAcquireSys(flag) < want) {
    __nanosleep(64);
    if ((++spins & 15u) == 0 && timerNs() - t0 > limitNs) {
      atomicCAS(status, 0, (1 << 24) | f);
      return;
    }
  }
}

// All copies (lanes along the columns of a block), then a system-scope fence per thread; the last block to finish
// publishes the epoch in every destination flag and, in the exchange form, then waits for this rank's own flags (one
// thread per flag), so that one launch stands between the producing kernel and its consumer instead of two. The wait
// comes after the push: no rank waits before its own boundary data is out.
__global__ void __launch_bounds__(256) shardPushKernel(const PushArgs a) {
  __shared__ int sLast;
  for (int i = 0; i < a.numCopies; ++i) {
    const int64_t total = int64_t(a.rows[i]) * a.cols[i];
    for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
      const int64_t r = idx / a.cols[i], c = idx - r * a.cols[i];
      a.dst[i][r * a.dstPitch[i] + c] = a.src[i][r * a.srcPitch[i] + c];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(a.ticket, 1u);
    sLast = done == gridDim.x - 1;
    if (sLast) {
      *a.ticket = 0;  // ready for the next launch that uses this ticket
      __threadfence_system();
      const int e = *a.epoch;
      for (int f = 0; f < a.numFlags; ++f) storeReleaseSys(a.flags[f], e);
    }
  }
  if (a.numWait == 0) return;
  __syncthreads();
  if (sLast && int(threadIdx.x) < a.numWait)
    waitFlag(a.waitFlags[threadIdx.x], int(threadIdx.x), *a.epoch + a.delta, a.limitNs, a.status);
}

struct WaitArgs {
  const int* flags[kMaxFlags];
  int numFlags;
  const int* epoch;
  int delta;  // wait until flag >= epoch + delta
  unsigned long long limitNs;
  int* status;
};

// One thread per flag.
__global__ void shardWaitKernel(const WaitArgs a) {
  const int f = threadIdx.x;
  if (f >= a.numFlags) return;
  waitFlag(a.flags[f], f, *a.epoch + a.delta, a.limitNs, a.status);
}

__global__ void epochBumpKernel(int* epoch) { *epoch += 1; }

}  // namespace
}  // namespace lkc

using namespace lkc;

static int pushLaunch(const LkcShardPush* d, void* const* waitFlags, int numWait, int delta, uint64_t limitNs,
                      void* status, void* stream, const char* what) {
  LKC_REQUIRE(d && d->num_copies >= 0 && d->num_copies <= kMaxCopies && d->num_flags >= 0 && d->num_flags <= kMaxFlags,
              "shard_push: too many copies or flags");
  LKC_REQUIRE(d->epoch && d->ticket, "shard_push: null epoch or ticket");
  PushArgs a;
  int64_t most = 0;
  for (int i = 0; i < d->num_copies; ++i) {
    const LkcShardCopy& c = d->copies[i];
    LKC_REQUIRE(c.src && c.dst && c.rows >= 0 && c.cols >= 0 && c.rows < (1 << 24) && c.cols < (1 << 24) &&
                    c.src_pitch >= c.cols && c.dst_pitch >= c.cols,
                "shard_push: bad copy");
    a.src[i] = static_cast<const float*>(c.src), a.dst[i] = static_cast<float*>(c.dst);
    a.srcPitch[i] = c.src_pitch, a.dstPitch[i] = c.dst_pitch, a.rows[i] = int(c.rows), a.cols[i] = int(c.cols);
    const int64_t n = c.rows * c.cols;
    if (n > most) most = n;
  }
  a.numCopies = d->num_copies;
  for (int f = 0; f < d->num_flags; ++f) {
    LKC_REQUIRE(d->flags[f], "shard_push: null flag");
    a.flags[f] = static_cast<int*>(d->flags[f]);
  }
  a.numFlags = d->num_flags;
  a.epoch = static_cast<const int*>(d->epoch), a.ticket = static_cast<unsigned*>(d->ticket);
  LKC_REQUIRE(numWait >= 0 && numWait <= kMaxFlags && (numWait == 0 || (waitFlags && status)), "shard_exchange: bad wait");
  for (int f = 0; f < numWait; ++f) {
    LKC_REQUIRE(waitFlags[f], "shard_exchange: null flag");
    a.waitFlags[f] = static_cast<const int*>(waitFlags[f]);
  }
  a.numWait = numWait, a.delta = delta, a.limitNs = limitNs, a.status = static_cast<int*>(status);
  int blocks = int(ceilDiv(most, 256));
  blocks = blocks < 1 ? 1 : (blocks > 64 ? 64 : blocks);
  shardPushKernel<<<blocks, 256, 0, S(stream)>>>(a);
  return launched(what);
}

extern "C" LKC_API int lkc_shard_push(const LkcShardPush* d, void* stream) {
  return pushLaunch(d, nullptr, 0, 0, 0, nullptr, stream, "shard_push");
}

extern "C" LKC_API int lkc_shard_exchange(const LkcShardPush* d, void* const* wait_flags, int num_wait, int delta,
                                          uint64_t limit_ns, void* status, void* stream) {
  return pushLaunch(d, wait_flags, num_wait, delta, limit_ns, status, stream, "shard_exchange");
}

extern "C" LKC_API int lkc_shard_wait(void* const* flags, int num_flags, const void* epoch, int delta,
                                      uint64_t limit_ns, void* status, void* stream) {
  LKC_REQUIRE(flags && num_flags >= 0 && num_flags <= kMaxFlags && epoch && status, "shard_wait: bad arguments");
  if (num_flags == 0) return 0;
  WaitArgs a;
  for (int f = 0; f < num_flags; ++f) {
    LKC_REQUIRE(flags[f], "shard_wait: null flag");
    a.flags[f] = static_cast<const int*>(flags[f]);
  }
  a.numFlags = num_flags, a.epoch = static_cast<const int*>(epoch), a.delta = delta;
  a.limitNs = limit_ns, a.status = static_cast<int*>(status);
  shardWaitKernel<<<1, 32 * int(ceilDiv(num_flags, 32)), 0, S(stream)>>>(a);
  return launched("shard_wait");
}

extern "C" LKC_API int lkc_shard_epoch_bump(void* epoch, void* stream) {
  LKC_REQUIRE(epoch, "shard_epoch_bump: null epoch");
  epochBumpKernel<<<1, 1, 0, S(stream)>>>(static_cast<int*>(epoch));
  return launched("shard_epoch_bump");
}

// ---- peer memory (set-up time; these are the only entry points of the library that allocate device memory on
// purpose): one arena per rank, allocated with cudaMalloc so that it can be exported through CUDA IPC, and the
// mapping of a peer's arena into this process.

extern "C" LKC_API int lkc_peer_alloc(uint64_t bytes, void** ptr) {
  LKC_REQUIRE(ptr && bytes > 0, "peer_alloc: bad arguments");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return failCuda("peer_alloc: cudaMalloc", e);
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return failCuda("peer_alloc: cudaMemset", e);
  }
  *ptr = p;
  return 0;
}

extern "C" LKC_API int lkc_peer_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? 0 : failCuda("peer_free: cudaFree", e);
}

extern "C" LKC_API int lkc_peer_handle(void* ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  LKC_REQUIRE(ptr && handle, "peer_handle: bad arguments");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return failCuda("peer_handle: cudaIpcGetMemHandle", e);
  std::memcpy(handle, &h, sizeof h);
  return 0;
}

extern "C" LKC_API int lkc_peer_open(const unsigned char handle[64], void** ptr) {
  LKC_REQUIRE(ptr && handle, "peer_open: bad arguments");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof h);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return failCuda("peer_open: cudaIpcOpenMemHandle", e);
  *ptr = p;
  return 0;
}

extern "C" LKC_API int lkc_peer_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? 0 : failCuda("peer_close: cudaIpcCloseMemHandle", e);
}
