/*
 * kiln_w4a16.h -- C ABI of the B200 (sm_100a) W4A16 quantised-linear library.
 *
 * Drop-in boundary for kiln's `kiln-marlin-gemm` crate: packed symmetric int4
 * weights (Marlin tile/fragment layout, group 128 along K or per-column) +
 * fp16 scales + bf16 activations -> bf16 output, fp32 accumulation.
 * All pointers are plain device (or, where stated, host) pointers; every
 * matrix is row-major and contiguous.  No entry point synchronises the stream
 * unless it says so.  Paths in the comments are relative to the kiln tree.
 */
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int kiln_w4a16_status_t;

/* 0..2 keep the reference's meaning (crates/kiln-marlin-gemm/csrc/marlin_kernel.cu:728-729,
 * crates/kiln-marlin-gemm/csrc/marlin_kernel.h:35-38). */
#define KILN_W4A16_OK 0
#define KILN_W4A16_ERR_PROB_SHAPE 1 /* k % 128, n % 256 (n % 64 for a shard), bad groupsize */
#define KILN_W4A16_ERR_KERN_SHAPE 2 /* no kernel configuration for the request */
#define KILN_W4A16_ERR_ALIGNMENT 3  /* a pointer is not 16-byte aligned */
#define KILN_W4A16_ERR_WORKSPACE 4  /* workspace missing or too small */
#define KILN_W4A16_ERR_CUDA 5       /* a CUDA runtime/driver call failed (see kiln_w4a16_last_cuda_error) */
#define KILN_W4A16_ERR_TIMEOUT 6    /* a bounded device-side wait gave up (read from the status word) */
#define KILN_W4A16_ERR_ARG 7        /* null pointer / negative size / size above a stated maximum */
#define KILN_W4A16_ERR_STATIC_SCRATCH 8 /* kiln_w4a16_gemm_bf16_noalloc: problem needs more than the built-in scratch */

/* Replaces kiln_marlin_w4a16_gemm (crates/kiln-marlin-gemm/csrc/marlin_kernel.h:39-55,
 * crates/kiln-marlin-gemm/csrc/marlin_kernel.cu:831-860; Rust declaration
 * crates/kiln-marlin-gemm/src/lib.rs:50-68).  Same symbol, same argument order.
 * Differences, all removing work from the caller:
 *   - A [prob_m, prob_k] and C [prob_m, prob_n] are bf16 (the reference kernel is
 *     fp16-only and its wrapper casts on both sides, lib.rs:169, 269);
 *   - `workspace` is never read or written: the reference's lock array of (prob_n / 128) * max_par int32
 *     (lib.rs:174-178) may be passed unchanged, or NULL.  In exchange this entry point keeps the tcgen05
 *     kernel to tilings without split-K or stream-K, which costs up to ~30 % at large prob_m on narrow
 *     projections; kiln_w4a16_gemm_bf16, with a sized workspace, has no such limit;
 *   - `dev` is ignored: the launch goes to the device that owns `stream`'s context
 *     (the reference hard-codes ordinal 0, lib.rs:210-215);
 *   - thread_k / thread_n / sms / max_par are accepted for signature compatibility;
 *     only -1 ("auto", what the reference wrapper always passes, lib.rs:252-255)
 *     or the reference's own legal values are accepted, and they do not select a tile.
 * B is int32 [prob_k/16, 2*prob_n] in the Marlin layout, s is fp16
 * [prob_k/groupsize, prob_n] (one row for groupsize -1) in the Marlin scale order.
 * Stream-ordered, asynchronous, capturable in a CUDA graph after one warm-up call
 * per device (function attributes and tensor maps are created on first use). */
kiln_w4a16_status_t kiln_marlin_w4a16_gemm(const void *A, const void *B, void *C, void *s, int prob_m,
                                           int prob_n, int prob_k, void *workspace, int groupsize,
                                           int dev, void *stream, int thread_k, int thread_n, int sms,
                                           int max_par);

/* Same operation with an explicit workspace size (checked) and without the
 * reference's unused tuning arguments.  New; the reference has one entry point
 * (marlin_kernel.h:39-55). */
kiln_w4a16_status_t kiln_w4a16_gemm_bf16(const void *A, const void *B, void *C, const void *s, int m,
                                         int n, int k, int groupsize, void *workspace,
                                         size_t workspace_bytes, void *stream);

/* Epilogue options of kiln_w4a16_gemm_bf16_ex.  They fuse what the reference does in separate kernels after its
 * Marlin call: the LoRA delta `x @ A^T @ B^T * scale` (crates/kiln-model/src/lora_loader.rs:213-233, added at
 * crates/kiln-model/src/forward.rs:2935-2939) and, for the gate+up projection, SiLU and the elementwise product
 * (forward.rs:2769-2839).
 *   lora_a    bf16 [lora_rank, k], lora_b bf16 [n, lora_rank] (device, 16-byte aligned), lora_rank a multiple of 8 up to
 *             128, lora_scale = alpha / rank.  lora_b is read like the packed weights, before the previous kernel in the
 *             stream is known to have finished: it must not be the output of the kernel launched just before.  The rank-r projection scale * x * A^T is computed first by a small kernel
 *             into the workspace (fp32), the GEMM adds its product with B^T to the fp32 sums before rounding to bf16.
 *   swiglu    1: the packed matrix holds the gate and up projections as ONE matrix whose columns alternate in runs of
 *             32 (columns 64c .. 64c+31 are gate columns 32c .. 32c+31, columns 64c+32 .. 64c+63 the up columns of the
 *             same indices; n = 2 * intermediate size).  C is then [m, n/2] = silu(gate) * up, computed in fp32 from the
 *             unrounded sums (the reference rounds gate and up to bf16 first).  lora_b follows the same column order.
 * For batch sizes the decode kernel serves the options are fused into that kernel's final reduction.  For larger ones
 * the LoRA delta rides in the tcgen05 kernels as extra K-steps (grouped scales; t is then written as bf16), and SwiGLU is
 * fused into the epilogue of the small-batch kernel (up to 128 rows, K not split) and of the general kernel's tilings
 * that write whole tiles from one accumulator per M-tile; what is not fused is applied by a second kernel to the bf16
 * GEMM result kept in the workspace. */
typedef struct kiln_w4a16_epilogue {
    int swiglu;
    const void *lora_a;
    const void *lora_b;
    int lora_rank;
    float lora_scale;
} kiln_w4a16_epilogue_t;

/* kiln_w4a16_gemm_bf16 with epilogue options (NULL or all-zero options: the same call).  The workspace must hold
 * kiln_w4a16_workspace_bytes_ex(m, n, k, ep) bytes.  New; the reference has no fused form. */
size_t kiln_w4a16_workspace_bytes_ex(int m, int n, int k, const kiln_w4a16_epilogue_t *ep);
kiln_w4a16_status_t kiln_w4a16_gemm_bf16_ex(const void *A, const void *B, void *C, const void *s, int m, int n, int k,
                                            int groupsize, const kiln_w4a16_epilogue_t *ep, void *workspace,
                                            size_t workspace_bytes, void *stream);

/* Several independent GEMMs in one launch: sibling projections of one layer that the reference issues as separate
 * Marlin calls (q, k, v: crates/kiln-model/src/forward.rs; gate and up: forward.rs:2769-2839).  The problems may
 * differ in every argument.  When every problem is at a decode batch size (kiln_w4a16_workspace_bytes == 0) and all
 * have either at most 8 rows or more than 8, ONE decode-kernel launch covers all their column blocks; otherwise the
 * problems are launched one after another with the given workspace (sized for the largest).  count <= 8. */
#define KILN_W4A16_MAX_GROUP 8
typedef struct kiln_w4a16_problem {
    const void *A;
    const void *B;
    void *C;
    const void *s;
    int m, n, k, groupsize;
} kiln_w4a16_problem_t;
kiln_w4a16_status_t kiln_w4a16_gemm_bf16_grouped(const kiln_w4a16_problem_t *problems, int count, void *workspace,
                                                 size_t workspace_bytes, void *stream);

/* No counterpart in the reference.  The same GEMM for callers that can neither allocate device
 * memory when they call nor lend a workspace: a server whose start-up gave all remaining HBM to
 * its KV-cache pool, or a serving loop that cannot take the device-wide synchronisation that
 * cudaMalloc / cudaFree imply.  It always runs the tcgen05 kernel (whatever m is); where that kernel
 * splits K, the fp32 partial sums go to a fixed array inside the library's device image instead of
 * a caller buffer.  Limits and rules:
 *   - the array is KILN_W4A16_NOALLOC_SCRATCH_BYTES (16 MiB) per GPU, held from library load to
 *     process exit; a problem whose split needs more (splits * m * n * 4 bytes) is refused with
 *     KILN_W4A16_ERR_STATIC_SCRATCH and nothing is launched; the tiling is chosen among those that fit (a
 *     tiling without a split always does), so in practice only a tiling forced through the tuning hook is refused;
 *   - the call makes no cudaMalloc, cudaFree or other allocating call.  The first call on each
 *     device looks up the array's device address (that device must be current) and sets the
 *     kernel's shared-memory attribute; make that first call before any stream capture;
 *   - every call on a GPU shares the one array, and it keeps the previous call's contents.
 *     Nothing in it needs clearing (each split overwrites its slab before it is read), but two
 *     calls that overlap on the same GPU (different streams) race on it: serialise them;
 *   - bounded-wait failures of these launches are recorded in a status word of the same kind
 *     inside the library image; kiln_w4a16_check_device_status reads and clears it too. */
#define KILN_W4A16_NOALLOC_SCRATCH_BYTES (16u << 20)
kiln_w4a16_status_t kiln_w4a16_gemm_bf16_noalloc(const void *A, const void *B, void *C, const void *s, int m,
                                                 int n, int k, int groupsize, void *stream);
/* Diagnostic: the tiling that entry point uses for (m, n, k), as {bn, splits, m_tiles, stream_k}; splits > 1 means the
 * built-in array is in use.  No counterpart in the reference. */
void kiln_w4a16_noalloc_plan(int m, int n, int k, int out[4]);

/* Column-parallel GEMM with the all-gather fused into its epilogue.  The reference is single-GPU (its
 * wrapper hard-codes device 0, crates/kiln-marlin-gemm/src/lib.rs:210-215); this replaces "GEMM on the local
 * columns + ncclAllGather of the slices".  B [k/16, 2*n_local] and s [k/g, n_local] are this rank's column
 * slice.  C_peers is a HOST array of n_peers (1..8) device pointers, one per GPU of the group (this GPU's
 * own buffer included), each a row-major bf16 [m, ldc] buffer mapped into this process (peer access /
 * symmetric memory).  The tcgen05 kernel writes rows x columns [col0, col0 + n_local) of every finished tile into
 * all of them: the buffer that lives on the current device (found with cudaPointerGetAttributes; exactly one is
 * expected, else it is treated like the others) through the kernel's ordinary TMA-store path, the other GPUs' buffers
 * with plain 16-byte stores over NVLink; no TMA touches another GPU's memory and no multicast is involved.  The call returns when the launch is enqueued; the gathered matrix is complete on a GPU once
 * every rank's launch has finished, so callers follow it with a stream-ordered barrier across the group
 * (kiln_b200.shard does).  ldc and col0 are in elements and multiples of 8. */
kiln_w4a16_status_t kiln_w4a16_gemm_bf16_allgather(const void *A, const void *B, const void *s, int m, int n_local,
                                                   int k, int groupsize, void *const *C_peers, int n_peers, int ldc,
                                                   int col0, void *stream);

/* The same with ONE pointer: C_multicast is the NVSwitch multicast address of the group's [m, ldc] buffers (all
 * GPUs' buffers bound to one multicast object, e.g. torch symmetric memory's multicast_ptr).  Every 16-byte piece is
 * written once with multimem.st and the switch replicates it into every GPU's buffer, this GPU's included, so a tile
 * leaves this GPU once instead of n_peers - 1 times.  Same completion rule as above.  No counterpart in the reference. */
kiln_w4a16_status_t kiln_w4a16_gemm_bf16_allgather_multicast(const void *A, const void *B, const void *s, int m,
                                                             int n_local, int k, int groupsize, void *C_multicast,
                                                             int ldc, int col0, void *stream);

/* Scratch bytes the GEMM needs for (m, n, k); replaces the reference wrapper's
 * fixed `(n/128) * 16` int32 lock array (crates/kiln-marlin-gemm/src/lib.rs:176-178). */
size_t kiln_w4a16_workspace_bytes(int m, int n, int k);

/* Shape rule of the path (crates/kiln-model/src/marlin_proj.rs:53-55): 1 if supported. */
int kiln_w4a16_shape_is_supported(int k, int n);

/* ---- packer (crates/kiln-marlin-gemm/src/lib.rs:284-529, `mod pack`) ------------ */

/* pack::build_weight_perm / build_scale_perm / build_scale_perm_single
 * (lib.rs:296-327, 333-341, 348-357).  out: 1024 / 64 / 32 int32. */
void kiln_w4a16_build_weight_perm(int32_t *out);
void kiln_w4a16_build_scale_perm(int32_t *out);
void kiln_w4a16_build_scale_perm_single(int32_t *out);

/* pack::quantize_and_pack on the HOST (lib.rs:370-491), multi-threaded inside one
 * matrix.  weight: f32 [k,n] row-major (host).  Outputs (host): b_packed int32
 * [k/16, 2n]; scales fp16 bits [k/g, n] (Marlin order); dequant f32 [k,n] or NULL.
 * num_threads <= 0 means "all hardware threads".  Bit-exact with the reference. */
kiln_w4a16_status_t kiln_w4a16_quantize_and_pack_host(const float *weight, int k, int n, int groupsize,
                                                      int32_t *b_packed, uint16_t *scales_f16,
                                                      float *dequant, int num_threads);

/* The same on the DEVICE, straight from the bf16 or f32 [k,n] weight already in HBM
 * (replaces the download -> CPU pack -> upload round trip of
 * crates/kiln-model/src/marlin_proj.rs:87-182).  weight_is_bf16: 1 = bf16, 0 = f32.
 * dequant may be NULL.  Stream-ordered. */
kiln_w4a16_status_t kiln_w4a16_quantize_and_pack_device(const void *weight, int weight_is_bf16, int k,
                                                        int n, int groupsize, int32_t *b_packed,
                                                        uint16_t *scales_f16, float *dequant,
                                                        void *stream);

/* Steps 3-5 only (lib.rs:429-488) for already-quantised weights: q uint8 [k,n] with
 * values 0..15, scales fp16 bits [k/g, n] in natural column order -> Marlin layout.
 * Host and device variants. */
kiln_w4a16_status_t kiln_w4a16_repack_host(const uint8_t *q, const uint16_t *scales, int k, int n,
                                           int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                           int num_threads);
kiln_w4a16_status_t kiln_w4a16_repack_device(const uint8_t *q, const uint16_t *scales, int k, int n,
                                             int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                             void *stream);

/* GPTQ checkpoint tensors -> this format without dequantising.  kiln dequantises GPTQ to bf16 on the CPU at load
 * (crates/kiln-model/src/quantized.rs:70-163) and its Marlin path then re-quantises; for symmetric checkpoints (every
 * zero-point 8) the direct repack is exact.  qweight int32 [k/8, n] (nibble i = input row 8*row + i), qzeros int32
 * [k/g, n/8] (nibble j = output column 8*col + j), scales fp16 bits [k/g, n] in natural column order (quantized.rs:6-14).
 * Host: refuses with KILN_W4A16_ERR_PROB_SHAPE when a zero-point is not 8; *asymmetric (host, optional) = how many.
 * Device: stream-ordered, cannot refuse without synchronising, so *asymmetric (DEVICE uint32, optional) receives the count
 * and the caller discards the output if it is not 0.  No act-order (g_idx) support. */
kiln_w4a16_status_t kiln_w4a16_repack_gptq_host(const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                                                int k, int n, int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                                uint32_t *asymmetric, int num_threads);
kiln_w4a16_status_t kiln_w4a16_repack_gptq_device(const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                                                  int k, int n, int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                                  uint32_t *asymmetric, void *stream);

/* ---- diagnostics --------------------------------------------------------------- */

/* Last CUDA error code seen by this library on the calling thread (0 = none). */
int kiln_w4a16_last_cuda_error(void);

/* Reads and clears the device status words that bounded device-side waits write
 * when they give up (the one of the ordinary launches, the one of the no-allocation
 * entry, and the decode kernel's: 0x800 = a CTA never received the split-K partial sums
 * of its cluster peers and left its part of C unwritten).  Synchronises `stream`.  Returns KILN_W4A16_OK or KILN_W4A16_ERR_TIMEOUT;
 * *detail (optional) receives the raw word. */
kiln_w4a16_status_t kiln_w4a16_check_device_status(void *stream, uint32_t *detail);

/* Tuning hook for sweeps: force the decode kernel's decomposition (cluster size
 * along K, K-warps and N-warps per CTA).  Pass 0,0,0 to restore the heuristic.
 * Process-wide, not thread-safe; has no counterpart in the reference. */
void kiln_w4a16_set_decode_override(int cluster_k, int warps_k, int warps_n);

/* Diagnostic: the decomposition the decode kernel would use for (m, n, k) on the current device (148 SMs are
 * assumed when no device is present), as out = {cluster_k, warps_k, warps_n, K groups staged per pass}.
 * Follows kiln_w4a16_set_decode_override.  No counterpart in the reference. */
void kiln_w4a16_decode_plan(int m, int n, int k, int out[4]);

/* Tuning hook: the M at and above which the tcgen05 kernels are used.  <= 0 restores the
 * built-in rule (M > 256 for projections of at most 1024 columns; otherwise M >= 17 for a plain GEMM,
 * which the small-batch kernel takes up to 128 rows; with fused epilogue options M >= 33, or M >= 17
 * for projections of 1025..3072 columns whose activation matrix is at least 128 KB); a huge value disables those kernels,
 * 1 forces them. */
void kiln_w4a16_set_prefill_min_m(int min_m);

/* Tuning hook for sweeps: force the tcgen05 kernel's tiling: bn = 128 or 256 columns per tile, K splits (1..8, fp32
 * slabs in the workspace), m_tiles = 1 or 2 (128-row tiles sharing a dequantised stage), stream_k = 1 for equal shares of the
 * (tile, K-step) space per CTA.  A combination that is not legal for a problem falls back to the built-in rule; 0,0,0,0
 * restores the rule.  kiln_w4a16_workspace_bytes follows the override.  Process-wide, not thread-safe; no counterpart in
 * the reference. */
void kiln_w4a16_set_prefill_override(int bn, int splits, int m_tiles, int stream_k);

/* Tuning hook: 0 keeps problems of at most 128 rows on the general tcgen05 kernel instead of the one that holds the
 * dequantised weights in tensor memory (default 1).  Results of the two kernels are the same up to fp32 summation
 * order.  Process-wide, not thread-safe; no counterpart in the reference. */
void kiln_w4a16_set_small_batch_kernel(int enabled);

/* How long a bounded device-side wait of the tcgen05 kernel polls before it gives up (nanoseconds; 0 restores the
 * default of 400 ms).  When a wait gives up the kernel records a code, every other wait of the CTA stops, outstanding
 * copies are drained, tensor memory is freed and the launch returns; kiln_w4a16_check_device_status then reports
 * KILN_W4A16_ERR_TIMEOUT and the next launch starts clean.  Replaces the unbounded spin of the reference's barrier
 * (crates/kiln-marlin-gemm/csrc/marlin_kernel.cu:162-171).  Process-wide, not thread-safe. */
void kiln_w4a16_set_wait_limit_ns(unsigned long long ns);

/* TEST HOOK for the give-up path above: the activation tile of K-step `k_step` (counted per CTA from 0) is announced
 * to its barrier but never copied, so the wait for it runs out.  Nothing faults or spins past the limit.  -1 switches
 * the hook off.  Process-wide, not thread-safe; no counterpart in the reference. */
void kiln_w4a16_test_drop_activation_load(int k_step);

/* Diagnostic: the tiling the tcgen05 kernel would use for (m, n, k) on the current device, as
 * out = {bn, splits, m_tiles, stream_k} (the arguments of kiln_w4a16_set_prefill_override). */
void kiln_w4a16_prefill_plan(int m, int n, int k, int out[4]);

/* Library version, and number of kernels this library launched since load
 * (diagnostic: lets a harness prove the native path ran). */
int kiln_w4a16_version(void);
unsigned long long kiln_w4a16_launch_count(void);

#ifdef __cplusplus
}
#endif
