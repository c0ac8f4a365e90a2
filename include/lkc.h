/* lkc: C-ABI of the B200 (sm_100a) kernel library for lokinfer's Kokoro iSTFTNet generator path.
 *
 * Every entry point mirrors one kernel of the reference's registry and takes the reference's own argument
 * packing (include/lokinfer/runtime/kernel.h:3-39, struct KernelArgs), so a registry adapter on the reference
 * side is a one-line forward:
 *
 *   ptrs   : operands in order, then outs in order (device pointers; f32 unless said otherwise)
 *   ints   : every operand's shape dims, then every out's shape dims, then the integer attrs in
 *            attribute-name order
 *   floats : float attrs in attribute-name order
 *   state  : result of the matching *_prepare call, or NULL
 *
 * Layout: frame-rate tensors are channel-first [C, L], row-major, like the reference CPU path.
 * Row pitch (an extension with no counterpart in the reference, whose tensors are always contiguous): the entry
 * points that say so accept, after their regular ints, one more int per [C, L] activation tensor = its row pitch in
 * floats (>= L). Without them rows are L floats apart. A caller that owns its intermediates can round the pitch up
 * to a multiple of 4 floats and keep base pointers 16-byte aligned: the tensor-core kernels then move those
 * tensors with the TMA unit (tiled bulk loads and stores) instead of 4-byte accesses. Results do not depend on
 * the pitch; the padding columns of an output row (between L and the pitch) may be overwritten.
 * Window extension (likewise no counterpart in the reference; used for time-sharded tensors, see the shard section):
 * after the row pitches the conv entry points accept further ints that describe x as a window into a longer row:
 * x_origin (output column t reads x columns x_origin + t * stride - padding + kk * dilation), valid_lo / valid_hi (x
 * columns outside [valid_lo, valid_hi) count as the zero padding, applied after the activation, as at the ends of an
 * unsharded row), and for the fused family stats_chunks (row stride of `stats` in chunks, so the chunk statistics can
 * land in a slice of the whole utterance's statistics row). With a window the output length is taken from `out`.
 * Ownership: the caller owns every buffer and all work is queued on the caller's stream (a cudaStream_t passed as
 * void*). No entry point allocates or frees device memory or synchronises the host, with these exceptions, each
 * stated at its declaration: lkc_harmonic_source_f32_cuda (grow-only scratch: cudaMalloc when n grows), the
 * host-side readers lkc_conv1d_tc_status / lkc_conv1d_tc_profile (they synchronise the device), and the lkc_peer_*
 * set-up calls of the time-sharding section.
 * Errors: every function returns 0 on success and non-zero on failure; lkc_last_error() then returns a
 * message (thread-local, valid until the next failing call on the thread). Nothing throws or aborts.
 * The stats tensors are f32[C, ceil(L / 128), 2] = per-(channel, 128-sample chunk) (mean, M2).
 */
#ifndef LKC_H_
#define LKC_H_

#include <stdint.h>

#if defined(__GNUC__)
#define LKC_API __attribute__((visibility("default")))
#else
#define LKC_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct LkcArgs {
  void* const* ptrs;
  const int64_t* ints;
  const double* floats;
  const void* state;
  uint32_t numPtrs;
  uint32_t numInts;
} LkcArgs;

typedef int (*LkcRunFn)(const LkcArgs* args, void* stream);

/* Registry, as registerKernel / findKernel / registeredKernels (include/lokinfer/runtime/kernel.h:60-74,
 * src/runtime/registry.cpp). Names are "<op>_f32_cuda"; the `_cuda` token plays the role of the reference's
 * `_gpu` device token (src/ir/ir.cpp:67-77). */
LKC_API int lkc_kernel_count(void);
LKC_API const char* lkc_kernel_name(int index); /* sorted */
LKC_API LkcRunFn lkc_find_kernel(const char* name); /* NULL if unknown */
LKC_API const char* lkc_last_error(void);
/* Library build info: "sm_100a" and the compile-time feature list. */
LKC_API const char* lkc_build_info(void);

/* ---- basic (unfused) layer ------------------------------------------------------------------------------ */

/* conv1d_f32_cpu (kernels/cpu/kokoro_conv.cpp:32-69, adapter :276-280).
 * ptrs x[Ci,L] w[Co,Ci,K] b[Co] | out[Co,Lo]; ints x(2) w(3) b(1) out(2) dilation padding stride
 * [x_pitch out_pitch [x_origin valid_lo valid_hi]]. */
LKC_API int lkc_conv1d_f32_cuda(const LkcArgs* a, void* stream);
/* conv1d_nobias_f32_cpu (kokoro_conv.cpp:282-286). ptrs x w | out; ints x(2) w(3) out(2) dilation padding stride
 * [x_pitch out_pitch]. */
LKC_API int lkc_conv1d_nobias_f32_cuda(const LkcArgs* a, void* stream);
/* conv_transpose1d_f32_cpu (kokoro_conv.cpp:71-95, adapter :288-292).
 * ptrs x[Ci,L] w[Ci,Co,K] b[Co] | out[Co,Lo]; ints x(2) w(3) b(1) out(2) output_padding padding stride. */
LKC_API int lkc_conv_transpose1d_f32_cuda(const LkcArgs* a, void* stream);
/* adain1d_f32_cpu (kernels/cpu/kokoro_norm.cpp:49-58, adapter :82-85). ptrs x[C,L] gb[2C] | out; ints x(2) gb(1)
 * out(2); floats eps. */
LKC_API int lkc_adain1d_f32_cuda(const LkcArgs* a, void* stream);
/* snake_f32_cpu (kernels/cpu/kokoro_misc.cpp:197-214). ptrs x[C,L] alpha[C] | out; ints x(2) alpha(1) out(2). */
LKC_API int lkc_snake_f32_cuda(const LkcArgs* a, void* stream);
/* leaky_relu_f32_cpu (kokoro_misc.cpp:172-180). ptrs x | out (any rank r); ints x(r) out(r); floats slope. */
LKC_API int lkc_leaky_relu_f32_cuda(const LkcArgs* a, void* stream);
/* add_f32_cpu (kernels/cpu/elementwise.cpp:58). ptrs a b | out; ints a(r) b(r) out(r). */
LKC_API int lkc_add_f32_cuda(const LkcArgs* a, void* stream);
/* add3_scale_f32_cpu (kokoro_misc.cpp:189-195): ((a + b) + c) * scale. ptrs a b c | out; floats scale. */
LKC_API int lkc_add3_scale_f32_cuda(const LkcArgs* a, void* stream);
/* scale_f32_cpu (kokoro_misc.cpp:182-187). ptrs x | out; floats scale. */
LKC_API int lkc_scale_f32_cuda(const LkcArgs* a, void* stream);
/* pad_reflect1d_f32_cpu (kokoro_conv.cpp:249-258, adapter :318-320). ptrs x[C,L] | out[C,left+L+right];
 * ints x(2) out(2) left right. */
LKC_API int lkc_pad_reflect1d_f32_cuda(const LkcArgs* a, void* stream);
/* gemm_bias_f32_cpu_accelerate as used for the style bank (models/kokoro/model.py:135-144): out = x @ wt + b.
 * ptrs x[M,K] wt[K,N] b[N] | out[M,N]; ints x(2) wt(2) b(1) out(2). */
LKC_API int lkc_gemm_bias_f32_cuda(const LkcArgs* a, void* stream);

/* ---- fused layer ---------------------------------------------------------------------------------------- */

/* channel_stats_f32_cpu (kernels/cpu/kokoro_conv_fused.cpp:631-639, adapter :775-777).
 * ptrs x[C,L] | stats[C,ceil(L/128),2]; ints x(2) stats(3) [x_pitch [stats_chunks]]. */
LKC_API int lkc_channel_stats_f32_cuda(const LkcArgs* a, void* stream);
/* adain_affine_f32_cpu (kokoro_conv_fused.cpp:641-664, adapter :780-783).
 * ptrs stats[C,S,2] gb[2C] | affine[3,C]; ints stats(3) gb(1) affine(2) length; floats eps. */
LKC_API int lkc_adain_affine_f32_cuda(const LkcArgs* a, void* stream);

/* conv1d_{snake,leaky,affine}[_res]_f32_cpu (kokoro_conv_fused.cpp:117-150, adapter :678-708):
 *   out = (conv1d(act((x - mean) * scale + beta), w) + b [+ res]) [* oscale], stride 1, zero padding applied
 *   after act; stats = chunk stats of out.
 * ptrs x[Ci,L] w[Co,Ci,K] b[Co] affine[3,Ci] [alpha[Ci]] [res[Co,Lo]] | out[Co,Lo] stats[Co,S,2]
 * ints x(2) w(3) b(1) affine(2) [alpha(1)] [res(2)] out(2) stats(3) dilation padding tile [x_pitch [res_pitch] out_pitch
 *      [stats_chunks x_origin valid_lo valid_hi]]
 * floats (name order) [oscale (leaky_res only)] [slope (leaky only)]. `tile` is accepted and ignored.
 * state: NULL, or the LkcConvState returned by lkc_conv1d_state_create for this weight (tensor-core path). */
LKC_API int lkc_conv1d_snake_f32_cuda(const LkcArgs* a, void* stream);
LKC_API int lkc_conv1d_snake_res_f32_cuda(const LkcArgs* a, void* stream);
LKC_API int lkc_conv1d_leaky_f32_cuda(const LkcArgs* a, void* stream);
LKC_API int lkc_conv1d_leaky_res_f32_cuda(const LkcArgs* a, void* stream);
LKC_API int lkc_conv1d_affine_f32_cuda(const LkcArgs* a, void* stream);
/* conv1d_leaky_wino_mean3_f32_cpu's contract as a direct conv (kokoro_conv_fused.cpp:744-772): the input is
 * ((x + x2) + x3) * in_scale.
 * ptrs x x2 x3 [Ci,L] w[Co,Ci,K] b[Co] affine[3,Ci] | out stats
 * ints x(2) x2(2) x3(2) w(3) b(1) affine(2) out(2) stats(3) dilation padding tile; floats in_scale slope. */
LKC_API int lkc_conv1d_leaky_mean3_f32_cuda(const LkcArgs* a, void* stream);

/* Tensor-core path of the fused conv family (tcgen05, TMEM accumulators, split operands): the counterpart of the
 * reference's prepare / destroy hooks (PrepareFn / DestroyFn, include/lokinfer/runtime/kernel.h:56-58) and of its
 * build-time weight packing (models/kokoro/model.py:60-65). Run once per constant weight:
 *   n = lkc_conv1d_tc_pack_floats(Co, Ci, K)       floats of the pack; 0 = shape not eligible (needs Ci % 16 == 0,
 *                                                  K <= 64), the CUDA-core kernel serves it. Co is padded to a
 *                                                  multiple of 128 with zero rows inside the pack
 *   lkc_conv1d_tc_pack_f32_cuda: ptrs w[Co,Ci,K] | wp[n]; ints w(3) wp(1)     hi / lo operand split in the UMMA layout
 *   st = lkc_conv1d_state_create(wp, Co, Ci, K)    host-side handle; pass it as LkcArgs.state of the conv1d_* calls
 * A conv call with a state whose shape is eligible ((K - 1) * dilation <= 50, K <= 24 for an f16 pack and <= 12 for
 * a tf32 pack, no mean3 input) runs on the tensor cores; anything else runs on the CUDA-core kernel with identical
 * semantics. lkc_conv1d_tc_status waits for all work queued on the current device (cudaDeviceSynchronize; do not call
 * it inside a stream capture), then reads (and optionally clears) the device status word: low 16 bits = role << 8 |
 * code of the first bounded wait that gave up (0 = none); bit 0x10000 = an activation exceeded the f16 range (65504)
 * under the f16 operand split (it became an infinite operand: the output of that launch is not finite); bit 0x20000
 * = a weight exceeded that range when an f16 pack was made
 * (pack it again after lkc_set_conv_path(2): the tf32 format has the range of f32). lkc_set_conv_io(1) makes later
 * launches use 4-byte accesses even for aligned rows, lkc_set_conv_io(0) (default) the TMA unit where rows are
 * 16-byte aligned (A/B testing). lkc_set_conv_path chooses the path and the operand format of packs made
 * AFTER the call: 0 (default) tensor cores with operands split into f16 hi + f16 lo * 2^-11 (3 kind::f16 MMAs per
 * 16 channels and tap), 2 tensor cores with tf32 hi + tf32 lo (6 kind::tf32 MMAs), 1 the CUDA-core kernel only
 * (A/B testing). lkc_*_pack_floats report sizes for the current format; a state remembers the format of its pack. */
typedef struct LkcConvState LkcConvState;
LKC_API int64_t lkc_conv1d_tc_pack_floats(int64_t co, int64_t ci, int64_t k);
LKC_API int lkc_conv1d_tc_pack_f32_cuda(const LkcArgs* a, void* stream);
LKC_API LkcConvState* lkc_conv1d_state_create(const void* wp, int64_t co, int64_t ci, int64_t k);
LKC_API void lkc_conv1d_state_destroy(LkcConvState* st);
LKC_API int lkc_conv1d_tc_status(int* status, int reset);
/* Stream-ordered form for callers that keep several utterances in flight: queues a 4-byte copy of the status word
 * into status_host (pinned host memory) behind the work already on `stream`; synchronises nothing, clears nothing. */
LKC_API int lkc_conv1d_tc_status_async(int* status_host, void* stream);
LKC_API int lkc_set_conv_path(int mode);
LKC_API int lkc_set_conv_io(int mode);
/* Role-level cycle counters of the tensor-core kernel (the counterpart of the reference's per-kernel profiler,
 * include/lokinfer/runtime/runtime.h:69-74), present only in a library built with -DLKC_TC_PROF=1 (the product
 * build returns an error): enable != 0 turns recording on for later launches; counters16 (may be NULL) receives
 * the 16 sums recorded so far (MMA / epilogue / producer / weight-producer wait and phase cycles, see conv_tc.cu)
 * and the counters are cleared. Synchronises the device. */
LKC_API int lkc_conv1d_tc_profile(int enable, int64_t* counters16);

/* conv_transpose1d_poly[_mean3]_f32_cpu (kernels/cpu/kokoro_conv.cpp:139-229, adapters :294-309):
 *   out = reflect_pad_left(conv_transpose1d(leaky(xin, slope), w, b, stride, padding), pad_left) + res,
 *   xin = x or ((x + x2) + x3) * in_scale; needs K = taps * stride and 2 padding = (taps - 1) stride.
 * wp is this library's polyphase weight pack f32[Ci, stride, taps, Co] made by lkc_convt_poly_pack_f32_cuda
 * (the counterpart of ops.convt_poly_weights_cpu, python/lokinfer/ops/kokoro.py:289-314).
 * ptrs x[Ci,L] wp b[Co] res[Co,L*s+pad_left] | out;  ints x(2) wp(4) b(1) res(2) out(2) pad_left padding stride
 * taps [x_pitch res_pitch out_pitch [halo_left halo_right]] (tensor-core route only; halo_* in {0, 1}: x holds that
 * many real columns before / after the L - halo_left - halo_right columns that produce output, instead of the zero
 * padding of an unsharded row); floats slope.   mean3: ptrs x x2 x3 wp b res | out; ints x(2) x2(2) x3(2) wp(4) b(1) res(2) out(2)
 * pad_left padding stride taps; floats in_scale slope. */
LKC_API int lkc_conv_transpose1d_poly_f32_cuda(const LkcArgs* a, void* stream);
LKC_API int lkc_conv_transpose1d_poly_mean3_f32_cuda(const LkcArgs* a, void* stream);
/* Weight pack for the two ops above, run once on constants. ptrs w[Ci,Co,K] | wp[Ci,stride,taps,Co] with
 * wp[c][r][tt][co] = w[c][co][(r + padding) % stride + (taps - 1 - tt) * stride];
 * ints w(3) wp(4) padding stride. */
LKC_API int lkc_convt_poly_pack_f32_cuda(const LkcArgs* a, void* stream);
/* Tensor-core path of conv_transpose1d_poly_f32_cuda (no mean3 input; strides 6 and 10 with K = 2 stride,
 * 2 padding = stride, Ci % 16 == 0: the two Kokoro upsamplers), prepared like the conv one:
 *   n = lkc_convt_tc_pack_floats(Ci, Co, K, stride, padding)     0 = not eligible
 *   lkc_convt_tc_pack_f32_cuda: ptrs w[Ci,Co,K] | wp[n]; ints w(3) wp(1) padding stride
 *   st = lkc_convt_state_create(wp, Ci, Co, K, stride, padding)   pass as LkcArgs.state of the poly call (the `wp`
 *        operand of that call stays the CUDA-core pack); destroy with lkc_conv1d_state_destroy.
 * The left reflect column is unpadded[co, 1] + res[co, 0] with the plain conv sum, as in the reference
 * (kokoro_conv.cpp:226). */
LKC_API int64_t lkc_convt_tc_pack_floats(int64_t ci, int64_t co, int64_t k, int64_t stride, int64_t padding);
LKC_API int lkc_convt_tc_pack_f32_cuda(const LkcArgs* a, void* stream);
LKC_API LkcConvState* lkc_convt_state_create(const void* wp, int64_t ci, int64_t co, int64_t k, int64_t stride,
                                             int64_t padding);

/* istft_logits_f32_cpu (kernels/cpu/kokoro_signal.cpp:275-359, adapter :388-391).
 * ptrs x[n_fft+2,L] | out[hop*(L-1)]; ints x(2) out(1) hop n_fft [x_pitch [frames frame0 i0]]. Fails when
 * n_fft/2+1 > 64, like the reference. Shard form: x holds frames frame0 .. frame0 + L of a signal of `frames` frames
 * and out receives its samples i0 .. i0 + len(out); x must hold every frame those samples overlap. */
LKC_API int lkc_istft_logits_f32_cuda(const LkcArgs* a, void* stream);

/* harmonic_source_f32_cpu (kernels/cpu/kokoro_signal.cpp:97-190, adapter :370-373; rule python/lokinfer/ops/kokoro.py
 * :417-426): Kokoro's SourceModuleHnNSF with the noise draw as an operand.
 * ptrs f0[n] noise[300n,9] w[9] b[1] | out[300n]; ints f0(1) noise(2) w(1) b(1) out(1). n <= 27962 (sample indices are
 * converted to float32, as in the reference). The float32 operation order of the reference kernel is part of the
 * contract (the phase reaches ~1e6 rad). Uses a phase table of 9 n floats as scratch between its two kernels: the
 * library keeps one grow-only buffer per device, so the first call on a device (and any call with a larger n) calls
 * cudaMalloc and must not be inside a stream capture; calls on one device must not overlap in time. */
LKC_API int lkc_harmonic_source_f32_cuda(const LkcArgs* a, void* stream);
/* harmonic_source_rng_f32_cpu (kokoro_signal.cpp:42-96, 192, adapter :375-380; rule ops/kokoro.py:429-435): the same
 * op with the noise drawn in the kernel: Philox4x32-10 keyed by the 64-bit seed, counters (sample_lo, sample_hi, blk,
 * 0x6C6B6E7A) for blk = 0..2, Box-Muller on the word pairs; deterministic per seed and independent of the launch
 * geometry (not torch's bit stream, as in the reference).
 * ptrs f0[n] w[9] b[1] seed | out[300n], where ptrs[3] points at an 8-byte HOST slot holding the i64 seed (the
 * reference's packing of scalar operands); ints f0(1) w(1) b(1) out(1). Same scratch rule as above. */
LKC_API int lkc_harmonic_source_rng_f32_cuda(const LkcArgs* a, void* stream);
/* The same op (same packing, same kernels, bit-identical result) for callers that must not allocate; it has no
 * counterpart in the reference. The phase table lives in a fixed device array of the library, so no call path
 * allocates or frees device memory. Limit: n <= 4096 frames (51 s of audio); larger inputs are rejected. The first
 * call on a device looks the array up and should come before any stream capture; calls on one device share the
 * array, so calls that overlap in time race on it. Not in the kernel registry. */
LKC_API int lkc_harmonic_source_noalloc_f32_cuda(const LkcArgs* a, void* stream);

/* stft_magphase_f32_cpu (kernels/cpu/kokoro_signal.cpp:196-272, adapter :382-385; rule ops/kokoro.py:438-449):
 * torch.stft(center, reflect, periodic hann(n_fft), onesided) -> cat(abs, angle).
 * ptrs x[S] | out[n_fft+2, S/hop+1]; ints x(1) out(2) hop n_fft. n_fft even, <= 64; S > n_fft/2. */
LKC_API int lkc_stft_magphase_f32_cuda(const LkcArgs* a, void* stream);

/* ---- decoder AdainResBlk1d stack (the producer of the generator's input, models/kokoro/model.py:158-221, 704-717):
 * its convs are the fused family above; these are the three ops it needs besides them. */
/* conv_transpose1d_dw_f32_cpu (kernels/cpu/kokoro_conv.cpp:97-127, adapter :304-307): depthwise
 * F.conv_transpose1d(groups = C). ptrs x[C,L] w[C,1,K] b[C] | out[C,(L-1)s-2p+K+op]; ints x(2) w(3) b(1) out(2)
 * output_padding padding stride. */
LKC_API int lkc_conv_transpose1d_dw_f32_cuda(const LkcArgs* a, void* stream);
/* No counterpart in the reference: the polyphase view of a strided conv's input, y[ci * s + r, t] = x[ci, s t + r -
 * pad] (zero outside [0, L); rows from Ci * s on are zero), so that conv1d(x, w, stride s, padding pad) with K = taps *
 * s becomes a stride-1 conv with `taps` taps over y with w'[co, ci * s + r, j] = w[co, ci, s j + r]: the shape the
 * tensor-core conv takes (the generator's noise_convs, models/kokoro/model.py:736-739). ptrs x | y; ints x(2) y(2)
 * pad stride [x_pitch y_pitch]. */
LKC_API int lkc_space_to_depth_f32_cuda(const LkcArgs* a, void* stream);
/* upsample_nearest1d_f32_cpu (kokoro_conv.cpp:231-247, adapter :310-312): F.interpolate(mode = 'nearest'), integer
 * scale. ptrs x[C,L] | out[C,L*scale]; ints x(2) out(2) scale. */
LKC_API int lkc_upsample_nearest1d_f32_cuda(const LkcArgs* a, void* stream);
/* concat_rows_f32_cpu (kernels/cpu/kokoro_misc.cpp:220-226, adapter :330-339): torch.cat(xs, dim = 0) of 2..8
 * f32[R_i, C]. ptrs x_0 .. x_{n-1} | out[sum R, C]; ints x_i(2) each, out(2). */
LKC_API int lkc_concat_rows_f32_cuda(const LkcArgs* a, void* stream);

/* ---- memory planner (host code) ----------------------------------------------------------------------------------
 * Offsets of n tensors (in allocation order) inside one arena, for a program that forks into num_streams streams: the
 * counterpart of the reference's planner (src/compiler/plan_memory.cpp; the arena of src/runtime/executable.cpp:
 * 732-815). alloc_clock[i * S + s] = vector clock of the allocating stream at tensor i's allocation; last_use[i * S +
 * s] = largest count of stream s at which tensor i was used (allocation included, 0 = never). A tensor's bytes are
 * reused by a later allocation only if each of its uses happens-before that allocation (last_use <= alloc_clock on
 * every stream) and it is not pinned. Greedy lowest-offset placement in program order; sizes rounded up to align. */
LKC_API int lkc_plan_memory(int64_t n, int64_t num_streams, const int64_t* bytes, const int32_t* pinned,
                            const int64_t* alloc_clock, const int64_t* last_use, int64_t align, int64_t* offsets,
                            int64_t* total);

/* ---- device-side test harness (the data path of the reference's RUN2 message, include/lokinfer/remote/server.h:30-47)
 * lkc_generate_cuda fills a tensor from a seed with the reference's generator (src/remote/server.cpp:739-782;
 * python/lokinfer/remote.py:96-119): splitmix64 of seed + (2 i + 1) golden and seed + (2 i + 2) golden, u = (mix >> 11)
 * 2^-53, dist 0 normal(a, b) by Box-Muller, 1 uniform [a, b), 2 integers in [floor a, floor b), computed in double.
 * ptrs seed | out, where ptrs[0] points at an 8-byte HOST slot holding the u64 seed; ints n dtype (0 f32, 1 i32,
 * 2 i64) dist; floats a b. Uniform and integer draws are bit-exact against the reference's generator, f32 normals
 * to an ulp (double log / cos of the device against the host's libm).
 * lkc_compare_stats_cuda compares two tensors on the device (src/remote/server.cpp:686-736): ptrs got ref | stats
 * workspace; ints n dtype; floats rtol atol. stats = 64 bytes: i64 count, nonfinite, mismatches (|got - ref| > atol +
 * rtol |ref|), worst index (largest excess, first on a tie; -1 if none), then f64 max_abs_err, max_abs_ref, sum_sq_err,
 * sum_sq_ref; workspace = LKC_COMPARE_WORKSPACE_BYTES bytes of device memory owned by the caller. Neither call
 * synchronises; the caller reads stats after its own synchronisation. */
#define LKC_COMPARE_WORKSPACE_BYTES 32768
LKC_API int lkc_generate_cuda(const LkcArgs* a, void* stream);
LKC_API int lkc_compare_stats_cuda(const LkcArgs* a, void* stream);

/* ---- time sharding of one utterance across GPUs ------------------------------------------------------------
 * No counterpart in the reference (it has no multi-GPU path). One rank owns a contiguous time range of every
 * activation tensor, with a margin of halo columns on both sides, in memory that its peers have mapped (CUDA IPC).
 * lkc_shard_push copies 2-D blocks of f32 (boundary columns into the neighbours' margins, this rank's slice of the
 * chunk statistics into every rank's statistics row) with plain stores, peer pointers included, and then
 * release-stores *epoch into every flag; lkc_shard_wait blocks the stream until every flag is >= *epoch + delta, for
 * at most limit_ns nanoseconds per flag: after that it sets *status = 1 << 24 | flag index (if it was 0) and returns,
 * so that nothing hangs when a peer is gone. lkc_shard_epoch_bump adds 1 to *epoch (one forward = one epoch, which
 * makes a captured launch sequence replayable). flags, epoch, ticket (one unsigned per call site, zero at start)
 * and status are device pointers; flags usually point into a peer's memory. */
#define LKC_SHARD_MAX_COPIES 16
#define LKC_SHARD_MAX_FLAGS 16
typedef struct LkcShardCopy {
  const void* src; /* f32, rows x cols, row pitch src_pitch floats */
  void* dst;
  int64_t src_pitch, dst_pitch, rows, cols;
} LkcShardCopy;
typedef struct LkcShardPush {
  LkcShardCopy copies[LKC_SHARD_MAX_COPIES];
  int32_t num_copies;
  void* flags[LKC_SHARD_MAX_FLAGS];
  int32_t num_flags;
  const void* epoch;
  void* ticket;
} LkcShardPush;
LKC_API int lkc_shard_push(const LkcShardPush* desc, void* stream);
LKC_API int lkc_shard_wait(void* const* flags, int num_flags, const void* epoch, int delta, uint64_t limit_ns,
                           void* status, void* stream);
LKC_API int lkc_shard_epoch_bump(void* epoch, void* stream);
/* lkc_shard_push followed by lkc_shard_wait on wait_flags in ONE launch (the block that publishes the flags then waits
 * for this rank's own): one kernel between a producer and its consumer instead of two. Only for ranks on different
 * GPUs: ranks that share a GPU queue every push before any wait (separate calls), since a kernel that waits for a
 * later launch on its own GPU would only run out its limit. */
LKC_API int lkc_shard_exchange(const LkcShardPush* desc, void* const* wait_flags, int num_wait, int delta,
                               uint64_t limit_ns, void* status, void* stream);
/* Set-up of the peer-mapped memory the calls above work on (the only entry points that allocate device memory on
 * purpose; none of them is on the data path): lkc_peer_alloc = cudaMalloc + zero fill of one arena, lkc_peer_handle
 * exports it (64-byte CUDA IPC handle, to be sent to the other ranks by any host channel), lkc_peer_open maps a
 * peer's arena into this process (peer access enabled on demand), lkc_peer_close / lkc_peer_free undo them. */
LKC_API int lkc_peer_alloc(uint64_t bytes, void** ptr);
LKC_API int lkc_peer_free(void* ptr);
LKC_API int lkc_peer_handle(void* ptr, unsigned char handle[64]);
LKC_API int lkc_peer_open(const unsigned char handle[64], void** ptr);
LKC_API int lkc_peer_close(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* LKC_H_ */
