/*
 * intent_b200 - C ABI of the sm_100a quantized-contraction library.
 *
 * Calling convention (every entry point):
 *   - Slot order follows the reference's native ABI for CPU providers
 *     (lib/Serialization/NativeABI.cpp:77-99, python/intent/runtime/native.py:56-120):
 *     for each public parameter in declaration order a view contributes
 *     `void* aP`, then one int64 extent per axis (`aP_dA`), then one int64
 *     ELEMENT stride per axis (`aP_sA`); a scalar contributes one slot.
 *   - Two things are added to that convention: the compile-time constants of
 *     the program (group size, zero point, ...) follow the parameters as int32
 *     slots, then a trailing `void* stream` (a cudaStream_t; NULL = the legacy
 *     default stream), and every entry returns an `int` status instead of void.
 *   - All pointers are DEVICE pointers, borrowed for the duration of the call.
 *     The library never frees or retains them.  Launches are asynchronous on
 *     `stream`; no entry synchronises the device or allocates device memory.
 *   - No exceptions, no exit(), no device traps.  Status 0 is success.
 */
#ifndef INTENT_B200_H
#define INTENT_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define INTENT_B200_API __attribute__((visibility("default")))
#else
#define INTENT_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum intent_b200_status {
  INTENT_B200_OK = 0,
  INTENT_B200_ERR_SHAPE = 1,        /* extents disagree with each other or with a constant */
  INTENT_B200_ERR_LAYOUT = 2,       /* strides are not the canonical contiguous ones / pointer misaligned */
  INTENT_B200_ERR_UNSUPPORTED = 3,  /* legal program, but no kernel specialisation covers it */
  INTENT_B200_ERR_TIMEOUT = 4,      /* a bounded device-side wait gave up (read back from the status word) */
  INTENT_B200_ERR_WORKSPACE = 5,    /* workspace missing or too small */
  INTENT_B200_ERR_NULL = 6,         /* a required pointer is NULL */
  INTENT_B200_ERR_SCRATCH_LIMIT = 7,/* problem needs more scratch than the built-in array of a no-allocation entry */
  INTENT_B200_ERR_INDEX = 8,        /* an index read from device memory (an expert id) was out of range; the rows it
                                       governs were computed with zero weights (read back from the status word) */
  INTENT_B200_ERR_CUDA = 1000       /* 1000 + cudaError_t of a failed runtime call */
};

#define INTENT_B200_VIEW1(p) void* p, int64_t p##_d0, int64_t p##_s0
#define INTENT_B200_VIEW2(p) void* p, int64_t p##_d0, int64_t p##_d1, int64_t p##_s0, int64_t p##_s1
#define INTENT_B200_VIEW3(p) void* p, int64_t p##_d0, int64_t p##_d1, int64_t p##_d2, \
                             int64_t p##_s0, int64_t p##_s1, int64_t p##_s2

/* Library identity: returns a static string "intent_b200 <version> sm_100a". */
INTENT_B200_API const char* intent_b200_version(void);
/* Human-readable name of a status code (static string). */
INTENT_B200_API const char* intent_b200_status_string(int status);
/* Number of kernels this library has launched in the calling process (all
 * entries, all streams).  Used by the benchmark to report its launch count. */
INTENT_B200_API int64_t intent_b200_launch_count(void);

/* Dry-run observation (the reference's NativeObservation reports registers, spills, shared memory and the
 * selected configuration of the latest native call, python/intent/runtime/diagnostics.py:119-137).  Between
 * begin and end, on the calling thread, the entries of the bandwidth / dense / grouped kernels launch nothing
 * and record what they would launch into `facts`: eight int32 (valid, registers per thread, local-memory bytes
 * per thread = spills, static shared bytes, dynamic shared bytes, threads per CTA, CTAs, CTAs per cluster)
 * followed by 64 bytes holding the kernel family and the plan's choice.  The small routing kernels do not
 * take part (they launch as usual). */
INTENT_B200_API int intent_b200_observe_begin(void* facts);
INTENT_B200_API int intent_b200_observe_end(void);

/* ------------------------------------------------------------------------
 * weight_only_int4_matmul  (W4A16)
 * Replaces the provider lowering of
 *   examples/kernels/contraction/weight_only_int4.py:18-51
 *   (torch-CPU reference experiments/cpu/baselines/pytorch/cpu_runtime.py:97-102).
 *   a0 activation   [M, K]   f16 | bf16, row-major contiguous
 *   a1 packed       [K/8, N] i32, N contiguous; nibble j of a word = k%8 == j
 *   a2 scales       [K/G, N] same dtype as the activation
 *   a3 output       [M, N]   same dtype as the activation
 *   group_size G: 32-multiple dividing K (reference constant 64; benchmark 128)
 *   zero_point: -1 = two's-complement nibble (the reference's decoding),
 *                8 = unsigned nibble minus 8 (benchmark configurations)
 * Y[m,n] = T( sum_k f32(X[m,k]) * f32(w[k,n]) ), f32 accumulation.
 * K must be positive (an empty contraction returns INTENT_B200_ERR_UNSUPPORTED;
 * M == 0 or N == 0 succeed without a launch).
 * The plain entries pick the kernel from M (M = 1: the single-problem bandwidth
 * kernel; M = 2 .. 8: the ride-along kernel of the table entries below, as a table
 * of one problem; M = 9 .. 16: the bandwidth kernel; above: the tcgen05 tensor-core
 * kernel); the _gemv / _gemm entries force the bandwidth / tensor-core kernel.
 *
 * workspace: device scratch of at least ..._workspace_bytes(M, K, N) bytes,
 * 16-byte aligned (NULL / 0 when that query returns 0).  It must be zero-filled
 * once after allocation; every launch that ends with status word 0 leaves it
 * zero-filled again, so it can be reused by later launches on the SAME stream.
 * Launches that may overlap on the GPU (different streams) need separate
 * workspaces.  Byte 0..3 is a status word: a launch whose bounded device wait
 * expired stores INTENT_B200_ERR_TIMEOUT there, stops early (parts of the output
 * are then unwritten) and leaves ticket counters behind, so the workspace must
 * not be reused as it is.  intent_b200_w4a16_gemv_workspace_status reads the
 * word and, when it is set, clears the workspace for reuse.
 * ------------------------------------------------------------------------ */
#define INTENT_B200_W4A16_SLOTS                                                                   \
  INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),     \
      int32_t group_size, int32_t zero_point, void *workspace, int64_t workspace_bytes, void *stream
INTENT_B200_API int intent_b200_weight_only_int4_matmul_f16(INTENT_B200_W4A16_SLOTS);
INTENT_B200_API int intent_b200_weight_only_int4_matmul_bf16(INTENT_B200_W4A16_SLOTS);
INTENT_B200_API int intent_b200_w4a16_gemv_f16(INTENT_B200_W4A16_SLOTS);
INTENT_B200_API int intent_b200_w4a16_gemv_bf16(INTENT_B200_W4A16_SLOTS);
INTENT_B200_API int intent_b200_w4a16_gemm_f16(INTENT_B200_W4A16_SLOTS);
INTENT_B200_API int intent_b200_w4a16_gemm_bf16(INTENT_B200_W4A16_SLOTS);
INTENT_B200_API int64_t intent_b200_weight_only_int4_matmul_workspace_bytes(int64_t M, int64_t K, int64_t N);
INTENT_B200_API int64_t intent_b200_w4a16_gemv_workspace_bytes(int64_t M, int64_t K, int64_t N);
/* Synchronises `stream`, returns the status word of a bandwidth-kernel workspace (0 or
 * INTENT_B200_ERR_TIMEOUT) and, when it is set, zero-fills the workspace again so that it can be reused.
 * Call it wherever the host synchronises anyway (end of a decode step, before results are consumed). */
INTENT_B200_API int intent_b200_w4a16_gemv_workspace_status(void* workspace, int64_t workspace_bytes, void* stream);
/* Status word of the tensor-core W4A16 kernels (single-CTA and CTA-pair): 0, INTENT_B200_ERR_TIMEOUT if a
 * bounded device-side wait expired in an earlier launch, or INTENT_B200_ERR_INDEX if a grouped entry met an
 * expert id outside [0, E).  Synchronises the device and clears the word. */
INTENT_B200_API int intent_b200_w4a16_gemm_device_status(void);
/* Dense W4A16 with M >= 512 runs on CTA pairs (tcgen05 cta_group::2); 0 forces the single-CTA kernel.
 * For measurement and tests; process-global. */
INTENT_B200_API int intent_b200_w4a16_gemm_pairs(int32_t enable);
/* Launch-latency overlap of the bandwidth kernel (programmatic dependent
 * launch).  When enabled, a launch may start and request its packed weights
 * while the kernel before it on the stream is still running; it waits for that
 * kernel before it reads the activations or writes the output.  Only enable it when the packed weights are not written by the kernel
 * launched immediately before (they are static model state in a decode loop).
 * Process-global; off by default. */
INTENT_B200_API int intent_b200_w4a16_gemv_overlap(int32_t enable);
/* Number of CTAs of the bandwidth kernel (0 = one per SM).  For measurement
 * sweeps; process-global. */
INTENT_B200_API int intent_b200_w4a16_gemv_grid(int32_t ctas);
/* Warps per CTA of the bandwidth kernel for M <= 8 (16 or 32; 0 = built-in choice).
 * For measurement sweeps; process-global. */
INTENT_B200_API int intent_b200_w4a16_gemv_warps(int32_t warps);

/* ------------------------------------------------------------------------
 * weight_only_int4_matmul over a TABLE of independent problems in one persistent launch
 * (same program and numerics as intent_b200_w4a16_gemv_*, M <= 16 per problem; the order of the
 * additions over K differs between the kernels, so results agree to rounding, not bit for bit;
 * every kernel is bitwise reproducible from launch to launch).  The
 * reference launches one kernel per contraction (python/intent/runtime/artifact.py:130-136);
 * a decode step's projections are small enough that launch ramp and drain cost as much as
 * the weight stream itself, so several of them can share one launch here: the weight stream
 * of problem i+1 starts while problem i is still being reduced.
 *   problems: HOST array of `count` entries; x [M,K], packed [K/8,N] i32, scales [K/G,N],
 *             y [M,N] are contiguous DEVICE buffers, 16-byte aligned; x, scales, y of type T.
 *   The problems must be independent: no problem may read (as x) what another problem of
 *   the same call writes (as y).  Tables longer than 8 problems run as several launches.
 *   workspace: ..._table_workspace_bytes(problems, count, group_size) bytes, zero-filled
 *   once, 16-byte aligned; same reuse and status-word rules as the single-problem entries
 *   (intent_b200_w4a16_gemv_workspace_status reads and recovers it).
 * ------------------------------------------------------------------------ */
typedef struct intent_b200_w4a16_problem {
  const void* x;
  const void* packed;
  const void* scales;
  void* y;
  int64_t M, K, N;
} intent_b200_w4a16_problem;
INTENT_B200_API int64_t intent_b200_w4a16_gemv_table_workspace_bytes(const intent_b200_w4a16_problem* problems,
                                                                     int32_t count, int32_t group_size);
INTENT_B200_API int intent_b200_w4a16_gemv_table_f16(const intent_b200_w4a16_problem* problems, int32_t count,
                                                     int32_t group_size, int32_t zero_point, void* workspace,
                                                     int64_t workspace_bytes, void* stream);
INTENT_B200_API int intent_b200_w4a16_gemv_table_bf16(const intent_b200_w4a16_problem* problems, int32_t count,
                                                      int32_t group_size, int32_t zero_point, void* workspace,
                                                      int64_t workspace_bytes, void* stream);
/* Programmatic dependent launch for the table entries (see intent_b200_w4a16_gemv_overlap); process-global. */
INTENT_B200_API int intent_b200_w4a16_gemv_table_overlap(int32_t enable);
/* Problems of at most eight rows run in the ride-along kernel (every unit brings its own activations, the
 * warps take units by ticket, no CTA-wide barrier separates the problems); 0 forces the staged kernel for
 * them too.  For measurement and tests; process-global; set it before querying the workspace size. */
INTENT_B200_API int intent_b200_w4a16_gemv_table_ride(int32_t enable);
/* Measurement knobs (process-global): "single" 0 = intent_b200_weight_only_int4_matmul_* never runs a problem
 * of two to eight rows as a table of one (1 = it does: the default); "slots" = upper limit on the slot ring
 * (8 .. 64, 0 = built-in choice); "unit_rows" 64 = units of 64 packed rows for problems of up to four rows
 * (measured slower; 0 = the built-in 32; set it before querying the workspace size); "corr_mma" 1 / 0 = the
 * ride-along kernel takes its per-group correction sums from two extra MMAs per step / adds them up from the
 * activations, -1 = built-in choice (MMAs for three rows and more); "probe" 1 = the arithmetic of every unit is skipped, 2 = the reduction too,
 * 3 = only the packed weights are loaded, 4 / 5 = arithmetic skipped and the reduction stops after the segment
 * sums / before the cross-CTA hand-over, 7 = the ride-along kernel returns at once.  Every probe value but 0 gives WRONG results by design: such launches
 * only show where the time goes. */
INTENT_B200_API int intent_b200_w4a16_gemv_table_tune(const char* knob, int32_t value);
/* Measurement only, no counterpart in the reference: the bare skeleton of the decode kernels - one CTA per SM,
 * a ring of `slots` 4 KiB shared-memory slots filled by TMA boxes of 32 x 32 words, no arithmetic - streams
 * `planes` contiguous [rows][cols] int32 matrices once and returns the milliseconds of that launch (or minus a
 * status code).  sync_mode adds, every sync_every-th unit of a CTA: 1 = __threadfence(); 2 = eight 16-byte
 * stores + atom.acq_rel.gpu; 3 = the stores + a relaxed atomic; 4 = the stores + atom.release.gpu; 5 = the
 * stores + a relaxed reduction; 0 = nothing.  rows, cols multiples of 32; slots 16, 32 or 48; scratch = at
 * least 8192 + SMs * 8192 bytes of zero-filled device memory (word 0 is non-zero afterwards if a wait gave up). */
INTENT_B200_API double intent_b200_ring_probe_ms(const void* matrices, int32_t planes, int32_t rows, int32_t cols,
                                                 int32_t slots, int32_t sync_mode, int32_t sync_every, void* scratch,
                                                 void* stream);

/* ------------------------------------------------------------------------
 * Tiled copy of a packed int4 weight for the tensor-core kernels.  The caller-visible format stays the
 * reference's [K/8, N] int32 (examples/kernels/contraction/weight_only_int4.py:31-39); a weight that is static
 * model state can be re-laid ONCE so that the four packed words a dequantiser thread needs per 64-wide k block
 * are adjacent (one 16-byte load instead of four loads N*4 bytes apart):
 *   tiled[n / 128][k / 64][(k % 64) / 32][n % 128][4 words], rows past K/8 and columns past N stored as zeros.
 * The reference pays one-off costs once and persists the result in the same spirit (generated programs and
 * native builds: python/intent/compiler/artifact.py:105-157, python/intent/runtime/native_artifact.py:151-190).
 *   ..._words(K, N): 32-bit words of the tiled copy (0 for an invalid shape).
 *   prelayout:         a0 packed [K/8, N] i32 -> a1 tiled [words] i32
 *   prelayout_grouped: a0 packed [E, K/8, N] i32 -> a1 tiled [E, words] i32 (each expert on its own)
 * The *_tiled entries are the tensor-core entries of the same name with the tiled copy in place of the
 * packed matrix (K is taken from the activation, N from the scales).
 * ------------------------------------------------------------------------ */
INTENT_B200_API int64_t intent_b200_w4a16_prelayout_words(int64_t K, int64_t N);
INTENT_B200_API int intent_b200_w4a16_prelayout(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), void* stream);
INTENT_B200_API int intent_b200_w4a16_prelayout_grouped(INTENT_B200_VIEW3(a0), INTENT_B200_VIEW2(a1), void* stream);
INTENT_B200_API int intent_b200_w4a16_gemm_tiled_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1),
                                                     INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),
                                                     int32_t group_size, int32_t zero_point, void* stream);
INTENT_B200_API int intent_b200_w4a16_gemm_tiled_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1),
                                                      INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),
                                                      int32_t group_size, int32_t zero_point, void* stream);
#define INTENT_B200_GROUPED_TILED_SLOTS                                                                    \
  INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW2(a3),              \
      INTENT_B200_VIEW3(a4), INTENT_B200_VIEW2(a5), int32_t group_size, int32_t zero_point,               \
      int32_t block_rows, void *stream
INTENT_B200_API int intent_b200_moe_grouped_w4a16_upgate_silu_tiled_bf16(INTENT_B200_GROUPED_TILED_SLOTS);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_upgate_silu_tiled_f16(INTENT_B200_GROUPED_TILED_SLOTS);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_f32_tiled_bf16(INTENT_B200_GROUPED_TILED_SLOTS);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_f32_tiled_f16(INTENT_B200_GROUPED_TILED_SLOTS);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_scatter_tiled_bf16(
    INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW2(a3), INTENT_B200_VIEW3(a4),
    INTENT_B200_VIEW1(a5), INTENT_B200_VIEW2(a6), INTENT_B200_VIEW2(a7), int32_t group_size, int32_t zero_point,
    int32_t block_rows, void* stream);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_scatter_tiled_f16(
    INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW2(a3), INTENT_B200_VIEW3(a4),
    INTENT_B200_VIEW1(a5), INTENT_B200_VIEW2(a6), INTENT_B200_VIEW2(a7), int32_t group_size, int32_t zero_point,
    int32_t block_rows, void* stream);

/* ------------------------------------------------------------------------
 * gemm_i8: C[m,n] = i32(sum_k A[m,k] * B[k,n]) + bias[n], wrapping int32.
 * Replaces the provider lowering of examples/kernels/contraction/gemm.py:29-39.
 *   a0 A [M,K] i8 (K contiguous)   a1 B [K,N] i8 (N contiguous)
 *   a2 bias [N] i32 (pointer may be NULL = zero bias)   a3 C [M,N] i32
 * K and N must be multiples of 16.
 * ------------------------------------------------------------------------ */
INTENT_B200_API int intent_b200_gemm_i8(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                        INTENT_B200_VIEW2(a3), void* stream);
/* w8a8_gemm: Y[m,n] = bf16( (f32(acc[m,n]) * sa[m]) * sb[n] ) on the exact int32
 * accumulator of gemm_i8 (the benchmark's per-token x per-channel epilogue; nearest
 * reference precedent: the per-channel scale of quantized_gemm, gemm.py:83-106).
 *   a0 A [M,K] i8   a1 B [K,N] i8   a2 sa [M] f32   a3 sb [N] f32   a4 Y [M,N] bf16 */
INTENT_B200_API int intent_b200_w8a8_gemm_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                               INTENT_B200_VIEW1(a3), INTENT_B200_VIEW2(a4), void* stream);
/* Status word of the int8 tensor-core kernel (see intent_b200_w4a16_gemm_device_status). */
INTENT_B200_API int intent_b200_i8_gemm_device_status(void);

/* ------------------------------------------------------------------------
 * MoE router, route alignment, permutation and grouped int4 contractions.
 * Integer outputs are bit-exact and deterministic.
 * ------------------------------------------------------------------------ */
/* Top-2 experts per token by logit, ties to the lower expert id (strict '>' insertion,
 * examples/kernels/sampling/top_k.py:10-33), and their f32 softmax probabilities
 * (examples/kernels/normalization/softmax.py:23-37).
 *   a0 logits [T,E] f32 -> a1 ids [T,2] i32, a2 weights [T,2] f32 */
INTENT_B200_API int intent_b200_moe_route_top2(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                               void* stream);
/* examples/kernels/routing/moe_align.py:14-29: a0 topk_ids [T,K] i32, a1 expert_counts [E] i32 (accumulated) */
INTENT_B200_API int intent_b200_moe_count_routes(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), void* stream);
/* moe_align.py:32-49: a0 counts [E] -> a1 offsets [E+1] (block-padded exclusive prefix), a2 total_padded [1] */
INTENT_B200_API int intent_b200_moe_prefix_routes(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                                  int32_t block_size, void* stream);
/* moe_align.py:52-73: a0 topk_ids [T,K], a1 offsets [E+1], a2 cursors [E] (InOut: += count),
 * a3 sorted_route_ids [capacity] (InOut).  Stable: ascending route id inside each expert span (the order of
 * the reference's torch implementation, cpu_runtime.py:1081-1097); span padding is set to T*K. */
INTENT_B200_API int intent_b200_moe_scatter_routes(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                                   INTENT_B200_VIEW1(a3), void* stream);
/* moe_align.py:76-86: a0 offsets [E+1] -> a1 expert_blocks [B] (blocks past the padded total are not written) */
INTENT_B200_API int intent_b200_moe_mark_expert_blocks(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1),
                                                       int32_t block_size, void* stream);
/* Inverse of the alignment: a0 sorted_route_ids [capacity], a1 total_padded [1] -> a2 route_positions [R] */
INTENT_B200_API int intent_b200_moe_route_positions(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1),
                                                    INTENT_B200_VIEW1(a2), void* stream);
/* Token rows in expert-sorted order (the I.gather of examples/kernels/ragged/moe.py:34-36):
 * a0 x [T,H] 16-bit, a1 sorted_route_ids [P], a2 total_padded [1] -> a3 rows [P,H]; padding rows are zero. */
INTENT_B200_API int intent_b200_moe_gather_rows(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                                INTENT_B200_VIEW2(a3), int32_t top_k, void* stream);
/* Grouped int4 contractions over expert-sorted rows padded to block_rows (128 or 256, the alignment's
 * BLOCK_SIZE) per expert; a1 expert_blocks holds one expert id per block_rows rows (tcgen05 kernel of
 * weight_only_int4_matmul with a per-block expert; reference programs
 * examples/kernels/ragged/grouped_gemm.py:42-70 and examples/kernels/ragged/moe.py:37-47):
 *   a0 rows [P,K] T, a1 expert_blocks [B] i32, a2 total_padded [1] i32, a3 packed [E,K/8,WN] i32,
 *   a4 scales [E,K/G,WN] T, a5 output.
 * upgate_silu: WN = 2*I, columns 0..I-1 gate and I..2I-1 up (I a multiple of 128);
 *              output [P,I] T = T(silu(gate) * up), f32 evaluation, one rounding.
 * down_f32:    output [P,WN] f32. */
#define INTENT_B200_GROUPED_SLOTS                                                                          \
  INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3),              \
      INTENT_B200_VIEW3(a4), INTENT_B200_VIEW2(a5), int32_t group_size, int32_t zero_point,               \
      int32_t block_rows, void *stream
INTENT_B200_API int intent_b200_moe_grouped_w4a16_upgate_silu_bf16(INTENT_B200_GROUPED_SLOTS);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_upgate_silu_f16(INTENT_B200_GROUPED_SLOTS);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_f32_bf16(INTENT_B200_GROUPED_SLOTS);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_f32_f16(INTENT_B200_GROUPED_SLOTS);
/* Down projection with the weighted combine of examples/kernels/ragged/moe.py:43-53 in its epilogue:
 *   a0 hidden rows [P,K] T, a1 expert_blocks [B], a2 total_padded [1], a3 packed [E,K/8,WN], a4 scales [E,K/G,WN],
 *   a5 sorted_route_ids [>= P] i32 (route of every expert-sorted row; values outside [0, T*K) mark padding rows),
 *   a6 route_weights [T,K] f32, a7 y [T,WN] f32 (InOut):
 *   y[route / K, :] += route_weights[route] * (rows[r, :] . W[e]) with relaxed vector atomics, in no fixed order -
 *   the reference's own GPU lowering of scatter_reduce(add) (lib/Target/Triton/Transforms/Access/Scatter.cpp:43-60).
 *   With K <= 2 on a zeroed y the result is still bit-reproducible: (0 + a) + b == (0 + b) + a. */
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_scatter_bf16(
    INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3), INTENT_B200_VIEW3(a4),
    INTENT_B200_VIEW1(a5), INTENT_B200_VIEW2(a6), INTENT_B200_VIEW2(a7), int32_t group_size, int32_t zero_point,
    int32_t block_rows, void* stream);
INTENT_B200_API int intent_b200_moe_grouped_w4a16_down_scatter_f16(
    INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3), INTENT_B200_VIEW3(a4),
    INTENT_B200_VIEW1(a5), INTENT_B200_VIEW2(a6), INTENT_B200_VIEW2(a7), int32_t group_size, int32_t zero_point,
    int32_t block_rows, void* stream);
/* Weighted combine (the scatter_reduce add of moe.py:48-53, made order-fixed):
 * y[t,:] += sum over choices c in order of weights[t,c] * rows[route_positions[t*K + c], :]
 *   a0 rows [P,H] f32, a1 route_positions [T*K] i32, a2 weights [T,K] f32, a3 y [T,H] f32 (InOut);
 *   accumulate = 0 starts the sum from zero instead of the old y (the caller then need not clear it) */
INTENT_B200_API int intent_b200_moe_combine(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW2(a2),
                                            INTENT_B200_VIEW2(a3), int32_t accumulate, void* stream);

/* ------------------------------------------------------------------------
 * Expert-parallel exchange over peer memory (NVLink), no collective on the data path.  The caller maps
 * every rank's row buffer [capacity_rows, H] (16-bit) and result buffer [capacity_rows, H] (f32) into this
 * process (symmetric memory / CUDA IPC) and passes the device addresses as int64 tables; it orders the
 * phases across ranks with stream-ordered barriers (all rows written before any owner computes, all
 * results written before any rank combines).  No kernel waits on another GPU.
 * Owner layout: local experts in order, spans padded to block_rows; inside a span source rank 0 first.
 * ------------------------------------------------------------------------ */
/* Cross-rank sync points without a collective: every rank owns a flag array [channels, W] i32 that all ranks can
 * address.  post bumps this rank's sequence number of the channel, optionally copies a small payload (a3, C ints)
 * into row `rank` of every rank's table [W, C] (a2: their addresses; extent 0 = no payload), fences, and stores the
 * number into slot [channel][rank] of every rank's flag array (a0: their addresses).  wait returns when every slot
 * [channel][*] of this rank's own array (a0) has reached this rank's number; it gives up after max_polls polls
 * (about a microsecond apart) and then writes INTENT_B200_ERR_TIMEOUT into a2 status[0] instead of hanging; while
 * status[0] is non-zero every later wait returns at once (the caller clears it after handling the failure).
 * a1 sequence [2 * channels] i32 is private to the rank (post and wait counters), zero before the first use. */
INTENT_B200_API int intent_b200_moe_peer_post(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                              INTENT_B200_VIEW1(a3), int32_t rank, int32_t channel, void* stream);
INTENT_B200_API int intent_b200_moe_peer_wait(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                              int32_t channel, int32_t max_polls, void* stream);
/* a0 counts [W,E] i32 (routes of every source rank to every global expert, E = W * experts per rank)
 * -> a1 dest_base [E] (first row, in the owner's buffer, of this rank's routes to expert e),
 *    a2 local_offsets [E/W + 1] (span starts of this rank's own experts; last = padded total), a3 total_padded [1],
 *    a4 expert_blocks [B] (local expert of every block_rows-row block of this rank's buffer, as moe_align.py:76-86) */
INTENT_B200_API int intent_b200_moe_peer_layout(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                                INTENT_B200_VIEW1(a3), INTENT_B200_VIEW1(a4), int32_t rank,
                                                int32_t block_rows, void* stream);
/* a0 x [T,H] 16-bit, a1 sorted_routes [R] (route ids grouped by expert, stable, no padding), a2 send_offsets [E+1]
 * (exclusive prefix of this rank's per-expert counts), a3 dest_base [E], a4 peer_rows [W] i64
 * -> writes row x[route / top_k] to peer_rows[owner] + position * H; a5 route_dest [R,2] = (owner, position) */
INTENT_B200_API int intent_b200_moe_peer_dispatch(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                                  INTENT_B200_VIEW1(a3), INTENT_B200_VIEW1(a4), INTENT_B200_VIEW2(a5),
                                                  int32_t top_k, int32_t capacity_rows, void* stream);
/* a0 peer_out [W] i64, a1 route_dest [R,2], a2 weights [T,K] f32, a3 y [T,H] f32 (InOut):
 * y[t,:] (+)= sum over choices c in order of weights[t,c] * (peer_out[owner] + position * H)[:];
 * accumulate = 0 starts from zero instead of the old y (the caller then need not clear it) */
INTENT_B200_API int intent_b200_moe_peer_combine(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                                 INTENT_B200_VIEW2(a3), int32_t capacity_rows, int32_t accumulate,
                                                 void* stream);

/* ------------------------------------------------------------------------
 * Ragged grouped contractions with dense 16-bit weights (tcgen05 kind::f16, f32 accumulation).
 * Group offsets are read on the device (clamped to the row count); K and N multiples of 8,
 * at most 1024 groups.  Rows of an empty group and rows outside every group are not written.
 * ------------------------------------------------------------------------ */
/* ragged_grouped_gemm / ragged_grouped_gemm_bf16 (examples/kernels/ragged/grouped_gemm.py:11-39, 42-70):
 *   a0 x [R,K] T, a1 group_offsets [G+1] i32, a2 weight [G,K,N] T -> a3 y [R,N] T
 *   y[r,:] = T(x[r,:] . weight[g]) for offsets[g] <= r < offsets[g+1] */
INTENT_B200_API int intent_b200_ragged_grouped_gemm_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1),
                                                        INTENT_B200_VIEW3(a2), INTENT_B200_VIEW2(a3), void* stream);
INTENT_B200_API int intent_b200_ragged_grouped_gemm_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1),
                                                         INTENT_B200_VIEW3(a2), INTENT_B200_VIEW2(a3), void* stream);
/* routed_expert_projection_bf16 (grouped_gemm.py:101-138; the f16 entry is the same program on f16):
 *   a0 x [T,K] T, a1 expert_offsets [E+1] i32, a2 member_routes [R] i32, a3 weight [E,N,K] T
 *   -> a4 output [T,TOP_K,N] T;  for route = member_routes[i], offsets[e] <= i < offsets[e+1]:
 *   output[route / TOP_K, route % TOP_K, :] = T(x[route / TOP_K, :] . weight[e]^T)
 *   workspace: at least R*K*2 bytes rounded up to 256 (the gathered rows), 16-byte aligned, not cleared. */
INTENT_B200_API int intent_b200_routed_expert_projection_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1),
                                                              INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3),
                                                              INTENT_B200_VIEW3(a4), int32_t top_k, void* workspace,
                                                              int64_t workspace_bytes, void* stream);
INTENT_B200_API int intent_b200_routed_expert_projection_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1),
                                                             INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3),
                                                             INTENT_B200_VIEW3(a4), int32_t top_k, void* workspace,
                                                             int64_t workspace_bytes, void* stream);
/* moe_expert_ffn (examples/kernels/ragged/moe.py:12-53; the bf16 entry is the same program on bf16):
 *   a0 x [T,D] T, a1 route_offsets [E+1] i32, a2 member_routes [R] i32, a3 route_token [NR] i32,
 *   a4 route_weights [NR] f32, a5 w1 [E,D,F] T, a6 w2 [E,F,D] T, a7 y [T,D] f32 (InOut)
 *   for route = member_routes[i] of expert e, token = route_token[route]:
 *   y[token,:] += route_weights[route] * (T(relu(x[token,:] . w1[e])) . w2[e])
 *   The additions are relaxed float reductions in no fixed order, as in the reference's GPU lowering
 *   (lib/Target/Triton/Transforms/Access/Scatter.cpp:43-60).
 *   workspace: R*D*2 rounded up to 256, plus R*F*2 rounded up to 256 bytes; not cleared. */
INTENT_B200_API int intent_b200_moe_expert_ffn_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                                   INTENT_B200_VIEW1(a3), INTENT_B200_VIEW1(a4), INTENT_B200_VIEW3(a5),
                                                   INTENT_B200_VIEW3(a6), INTENT_B200_VIEW2(a7), void* workspace,
                                                   int64_t workspace_bytes, void* stream);
INTENT_B200_API int intent_b200_moe_expert_ffn_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                                    INTENT_B200_VIEW1(a3), INTENT_B200_VIEW1(a4), INTENT_B200_VIEW3(a5),
                                                    INTENT_B200_VIEW3(a6), INTENT_B200_VIEW2(a7), void* workspace,
                                                    int64_t workspace_bytes, void* stream);
/* Dense forms on the same kernel (examples/kernels/contraction/gemm.py:40-106); K and N multiples of 8.
 * gemm: a0 a [M,K] f16, a1 b [K,N] f16 -> a2 c [M,N] f16; activation 0 = none, 1 = ReLU (the ACTIVATION constexpr).
 * bf16_gemm: the same on bf16 without activation.
 * quantized_gemm: a0 a [M,K] f16, a1 b [K,N] f16, a2 bias [N] f32, a3 residual [M,N] f16, a4 output_scale [N] f32
 *   -> a5 output [M,N] i8 = i8(trunc(clamp((relu(acc + bias[n]) + f32(residual[m,n])) / scale[n], -128, 127))). */
INTENT_B200_API int intent_b200_gemm_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                         int32_t activation, void* stream);
INTENT_B200_API int intent_b200_bf16_gemm(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                          void* stream);
INTENT_B200_API int intent_b200_quantized_gemm_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                                   INTENT_B200_VIEW2(a3), INTENT_B200_VIEW1(a4), INTENT_B200_VIEW2(a5),
                                                   void* stream);
/* Status word of the dense grouped kernels (a bounded device wait that expired); synchronises the device. */
INTENT_B200_API int intent_b200_grouped_gemm16_device_status(void);

/* ------------------------------------------------------------------------
 * Packed-weight contractions next to weight_only_int4_matmul
 * (examples/kernels/contraction/weight_only_int4.py:54-175).  The packed operand is decoded once
 * into the workspace (K contiguous) and contracted by the dense tcgen05 kernels; the integer
 * programs are exact with wrapping int32 arithmetic.  The workspace is not cleared.
 * ------------------------------------------------------------------------ */
/* w4a8_packed_matmul (weight_only_int4.py:54-91): a0 activation i8 [M,K], a1 packed_weight u8 [N,K/2]
 * (low nibble = even k, two's-complement int4) -> a2 output i32 [N,M].  K % 32 == 0, M % 16 == 0.
 * workspace >= N*K bytes rounded up to 256. */
INTENT_B200_API int intent_b200_w4a8_packed_matmul(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                   INTENT_B200_VIEW2(a2), void* workspace, int64_t workspace_bytes,
                                                   void* stream);
/* bitnet_int2_matmul (weight_only_int4.py:94-123): a0 activation i8 [M,K], a1 packed_weight u8 [N,K/4]
 * (value k of a 16-value word: byte k % 4, bit 2 * (k / 4), values 0..3) -> a2 output i32 [M,N].
 * K % 16 == 0, N % 16 == 0.  workspace >= N*K bytes rounded up to 256. */
INTENT_B200_API int intent_b200_bitnet_int2_matmul(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                   INTENT_B200_VIEW2(a2), void* workspace, int64_t workspace_bytes,
                                                   void* stream);
/* dequant_bf16_fp4_matmul (weight_only_int4.py:126-175): a0 activation bf16 [M,K], a1 packed_weight u8 [N,K/2]
 * (four e2m1 codes per big-endian 16-bit word) -> a2 output bf16 [M,N], f32 accumulation.
 * K % 8 == 0, N % 8 == 0.  workspace >= N*K*2 rounded up to 256, plus 256 bytes. */
INTENT_B200_API int intent_b200_dequant_bf16_fp4_matmul(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                        INTENT_B200_VIEW2(a2), void* workspace,
                                                        int64_t workspace_bytes, void* stream);

/* quantized_projection (examples/kernels/quantization/quantized_projection.py:5-19; record formats and
 * rounding order doc/dsl/quantized-operations.en.md sections 2-4): a0 weights u8 [N,G,144] (Q4_K records),
 * a1 activation f32 [G,256] -> a2 output f32 [N].  The activation is quantized to Q8_K records inside the
 * call; workspace >= G*292 bytes rounded up to 256, not cleared. */
INTENT_B200_API int intent_b200_quantized_projection(INTENT_B200_VIEW3(a0), INTENT_B200_VIEW2(a1),
                                                     INTENT_B200_VIEW1(a2), void* workspace,
                                                     int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------
 * entry_benchmark counterparts of the reference's native ABI, which exports
 * `double entry_benchmark(slots..., int64 repetitions)` beside every `entry(slots...)`
 * (python/intent/runtime/mojo/compilation.py:54-96, python/intent/runtime/mojo/program.py:253-257).
 * Same slots as the entry, then `repetitions`, then the stream.  One untimed call first, then
 * `repetitions` calls between two CUDA events on `stream` (the events are the only synchronisation).
 * Returns the mean milliseconds per call, or minus the status code of a failed call.
 * ------------------------------------------------------------------------ */
#define INTENT_B200_W4A16_BENCHMARK_SLOTS                                                         \
  INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),     \
      int32_t group_size, int32_t zero_point, void *workspace, int64_t workspace_bytes,          \
      int64_t repetitions, void *stream
INTENT_B200_API double intent_b200_weight_only_int4_matmul_f16_benchmark(INTENT_B200_W4A16_BENCHMARK_SLOTS);
INTENT_B200_API double intent_b200_weight_only_int4_matmul_bf16_benchmark(INTENT_B200_W4A16_BENCHMARK_SLOTS);
INTENT_B200_API double intent_b200_gemm_i8_benchmark(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                     INTENT_B200_VIEW1(a2), INTENT_B200_VIEW2(a3),
                                                     int64_t repetitions, void* stream);
INTENT_B200_API double intent_b200_w8a8_gemm_bf16_benchmark(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                            INTENT_B200_VIEW1(a2), INTENT_B200_VIEW1(a3),
                                                            INTENT_B200_VIEW2(a4), int64_t repetitions,
                                                            void* stream);

/* ------------------------------------------------------------------------
 * W4A16 bandwidth kernel (f16) without any workspace argument.
 * This entry has no counterpart in the reference.  It exists for callers that
 * cannot allocate device memory on behalf of the library: a host that runs
 * with a frozen memory pool, a plugin ABI that carries only an operator's
 * inputs and outputs, or code between stream-capture begin and end, where
 * cudaMalloc is not allowed.  Same arguments and result as
 * intent_b200_w4a16_gemv_f16 minus the workspace pair; the scratch is a fixed
 * 8 MiB device array inside the library image (held by every GPU that loads
 * the library until the process exits).
 *   - Problems whose scratch need (intent_b200_w4a16_gemv_workspace_bytes)
 *     exceeds 8 MiB return INTENT_B200_ERR_SCRATCH_LIMIT; nothing is launched.
 *   - The entry calls no cudaMalloc / cudaFree and no allocating library
 *     routine.  It clears the part of the array that must start at zero with
 *     a cudaMemsetAsync on `stream`, then launches the kernel on `stream`.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, that device current); make that first call
 *     before any stream capture begins.
 *   - All calls on one device share the one array: calls that can overlap on
 *     the GPU (different streams, or different host threads on unordered
 *     streams) race on it and produce wrong results.  Order them on one
 *     stream or use the workspace entries.
 *   - A bounded device wait that expired is recorded in the array's first word;
 *     intent_b200_w4a16_gemv_builtin_scratch_status(stream) synchronises the
 *     stream and returns it (0 = fine).  Read it before the next call of the
 *     entry on that device: each call clears the word.
 * ------------------------------------------------------------------------ */
INTENT_B200_API int intent_b200_w4a16_gemv_f16_builtin_scratch(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                               INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),
                                                               int32_t group_size, int32_t zero_point,
                                                               void* stream);
INTENT_B200_API int intent_b200_w4a16_gemv_builtin_scratch_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INTENT_B200_H */
