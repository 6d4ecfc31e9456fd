/*
 * sglb200 — C ABI of the B200 (sm_100a) block-FP8 W8A8 hot path.
 *
 * One shared library, plain pointers and sizes, no C++ or torch types.  Every entry point
 *   - works on DEVICE pointers and enqueues on the CUDA stream passed as `stream`
 *     (a cudaStream_t cast to void*; NULL = the legacy default stream),
 *   - validates shapes / strides / alignment on the host BEFORE launching anything and
 *     returns 0 (SGLB200_OK) or a negative SGLB200_ERR_* code; it never throws, never
 *     synchronises the device, and never allocates device memory unless its comment says so,
 *   - borrows its inputs (never freed or written) and writes only the caller-allocated
 *     outputs and the caller-provided scratch buffers named in its signature.
 * sglb200_status_string() turns a code into text; sglb200_last_error_detail() returns a
 * thread-local message describing the last failed check (which argument, which value).
 *
 * Threads and devices: the entry points may be called from several host threads, with one exception.  The FIRST call of a
 * kernel family on a device does per-device set-up (cudaFuncSetAttribute, device properties, the address of the built-in
 * scratch array) and records it in plain per-device tables; make that first call per device from one thread (a warm-up
 * call at start-up does it).  Later calls only read those tables.  Device ordinals 0..63 are supported by the tables;
 * a higher ordinal repeats the set-up on every call, and sglb200_fp8_blockwise_scaled_mm_noalloc refuses it.
 *
 * Reference files cited below are paths inside the vincent-shop/sglang tree.
 */
#ifndef SGLB200_H_
#define SGLB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SGLB200_OK 0
#define SGLB200_ERR_SHAPE (-1)       /* a size or stride is inconsistent or unsupported        */
#define SGLB200_ERR_ALIGN (-2)       /* a pointer or leading dimension is not aligned as required */
#define SGLB200_ERR_ARCH (-3)        /* the current device is not compute capability 10.x      */
#define SGLB200_ERR_LAUNCH (-4)      /* the CUDA runtime refused the launch or a set-up call   */
#define SGLB200_ERR_DTYPE (-5)       /* unsupported element type code                           */
#define SGLB200_ERR_NULL (-6)        /* a required pointer is NULL                              */
#define SGLB200_ERR_WORKSPACE (-7)   /* scratch buffer too small                                */

/* element type codes used by the `*_dtype` arguments */
#define SGLB200_BF16 0
#define SGLB200_F16 1
#define SGLB200_F32 2

const char* sglb200_status_string(int status);
const char* sglb200_last_error_detail(void);
/* Library version, "major.minor". */
const char* sglb200_version(void);

/*
 * Upper bound on the SMs the persistent kernels of this library occupy (GEMM, grouped GEMM, few-rows GEMM and the
 * grid-sized helpers): their grids are sized from min(num_sms, SMs of the device).  0 lifts the bound.  Process-wide,
 * read at every launch; set it from the thread that launches.  Use: leave SMs free for a communication kernel that runs
 * beside a GEMM (a persistent GEMM that fills every SM makes a concurrent kernel wait for one of its CTAs to finish).
 * Replaces: deep_gemm.set_num_sms / get_num_sms as used by configure_deep_gemm_num_sms,
 *           python/sglang/srt/layers/deep_gemm_wrapper/entrypoint.py:94-104.
 * sglb200_get_num_sms returns the bound in force (the device's SM count when none is set).
 */
int sglb200_set_num_sms(int num_sms);
int sglb200_get_num_sms(void);

/*
 * Grouped GEMMs (sglb200_fp8_blockwise_scaled_grouped_mm, its masked form and sglb200_fp8_ue8m0_scaled_grouped_mm) whose
 * experts hold at most max_avg_rows rows on average (total rows / experts; the row bound per expert in the masked layout) run on the
 * few-rows kernel: operands swapped, 128 weight rows x 16 / 32 / 64 activation rows per MMA, only the weights of
 * experts that have rows are streamed.  This is the decode case of a mixture-of-experts layer, where the 128 x 128
 * kernel spends a full tile of tensor-core work (and, with fp32 scales, of promotion) on a handful of rows: no slower
 * in a burst, but sustained that work runs the board into its power cap at half the SM clock.  Default 20 (measured
 * cross-over on the DeepSeek-V3 layer shape under sustained load: faster up to ~24 rows per expert, level at 32-48);
 * 0 = always the 128 x 128 kernels; at most 64.  With UE8M0 scales the few-rows kernel decodes the exponent bytes and
 * applies the scales in fp32 after each k-block (exact for powers of two).
 * The results of the two kernels are bit-identical (same products, same fp32 accumulation order per k-block).
 * Process-wide, read at every launch.
 * Replaces: the small-M tile configurations of the reference's grouped kernel,
 *           sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:440-560 (dispatch on the row count).
 */
int sglb200_set_grouped_few_rows(int max_avg_rows);
int sglb200_get_grouped_few_rows(void);

/*
 * Q — per-token-group quantisation to e4m3.
 * Replaces: sgl_per_token_group_quant_8bit  sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:116-217
 *           (schema sgl-kernel/csrc/common_extension.cc:173-176) for the e4m3 destination type.
 *
 * input  [num_rows, hidden] contiguous, dtype in_dtype (bf16 / f16 / f32), 16-byte aligned.
 * out_q  [num_rows, hidden] e4m3 bytes, contiguous, 8-byte aligned.
 * out_s  one scale per (row, group), group = group_size consecutive elements of a row,
 *        group_size in {16, 32, 64, 128}, hidden % group_size == 0:
 *          scale_ue8m0 == 0: float at out_s[row * s_stride_row + g * s_stride_group]
 *                            (row-major: (G, 1); column-major: (1, M) or (1, align(M,4)))
 *          scale_ue8m0 != 0: out_s is int32; byte g % 4 of the int32 at
 *                            out_s[row * s_stride_row + (g / 4) * s_stride_group] is the biased
 *                            exponent of the power-of-two scale; bytes of a word past the last
 *                            group are written as zero.  (Strides count int32 words.)
 * Arithmetic (bit-exact with native_per_token_group_quant_fp8, python/sglang/test/test_block_fp8.py:23-48):
 *   amax = max(max|x|, eps); s = amax / fp8_max (IEEE); UE8M0: s = 2^ceil(log2 s);
 *   q = RNE_e4m3(clamp(x / s, fp8_min, fp8_max)) with a correctly rounded fp32 quotient.
 * `eps` is used as given, in fp32: a caller that wants the torch-native behaviour for bf16 input
 * passes eps already rounded to bf16 (the Python wrapper does).
 * UE8M0: the power-of-two rounding is applied to amax / fp8_max as it is; no further floor on the scale (the
 * torch-native / Triton behaviour).  The reference's v1 CUDA kernel clamps the scale at 1e-10 before rounding, so its
 * exponent byte for an all-zero group is 94 where this entry point writes the exponent of eps / fp8_max rounded up.
 */
int sglb200_per_token_group_quant_fp8(const void* input, int in_dtype, void* out_q, void* out_s,
                                      int64_t num_rows, int64_t hidden, int group_size, float eps,
                                      float fp8_min, float fp8_max, int scale_ue8m0,
                                      int64_t s_stride_row, int64_t s_stride_group, void* stream);

/*
 * Fused SiLU-and-mul + per-token-group quantisation (one pass over the gate_up activations).
 * Replaces: sgl_per_token_group_quant_8bit_v2 with fuse_silu_and_mul, unmasked layout
 *           sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:336-347,394-514.
 * input [num_rows, 2 * hidden] (gate = first half, up = second half, as SiluAndMul,
 * python/sglang/srt/layers/activation.py:68-70); act = round_in_dtype(round_in_dtype(silu(gate)) * up);
 * outputs as sglb200_per_token_group_quant_fp8 over act [num_rows, hidden].
 * If out_act is not NULL the activation (in_dtype, [num_rows, hidden]) is also stored.
 */
int sglb200_silu_mul_group_quant_fp8(const void* input, int in_dtype, void* out_q, void* out_s, void* out_act,
                                     int64_t num_rows, int64_t hidden, int group_size, float eps,
                                     float fp8_min, float fp8_max, int scale_ue8m0,
                                     int64_t s_stride_row, int64_t s_stride_group, void* stream);

/*
 * Q in the batched / masked layout of the low-latency MoE path: input [num_batches, rows_per_batch, hidden] (with
 * fuse_silu_and_mul != 0: [.., 2 * hidden], gate first), out_q [num_batches, rows_per_batch, hidden]; the scale of
 * (batch b, row r, group g) at out_s[b * s_stride_batch + r * s_stride_row + g * s_stride_group] (UE8M0: int32 words,
 * g / 4, as above).  With masked_m != NULL (int32 [num_batches], device) only rows r < masked_m[b] are read and
 * written.  bf16 / f16 input.  Same arithmetic as sglb200_per_token_group_quant_fp8.
 * Replaces: sgl_per_token_group_quant_8bit_v2 with masked_m
 *           sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:194-238,394-514 (schema common_extension.cc:178-181).
 */
int sglb200_group_quant_fp8_batched(const void* input, int in_dtype, void* out_q, void* out_s, int64_t num_batches,
                                    int64_t rows_per_batch, int64_t hidden, int group_size, float eps, float fp8_min,
                                    float fp8_max, int scale_ue8m0, int fuse_silu_and_mul, const int32_t* masked_m,
                                    int64_t s_stride_batch, int64_t s_stride_row, int64_t s_stride_group, void* stream);

/*
 * G — block-scaled FP8 GEMM:  out[m, n] = cast( sum_kb ( sum_{k in kb} a[m,k] * b[n,k] ) * sa[m,kb] * sb[n/128,kb] ).
 * Replaces: fp8_blockwise_scaled_mm  sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:368-465
 *           (schema common_extension.cc:168-171) and the Triton twin w8a8_block_fp8_matmul_triton
 *           python/sglang/srt/layers/quantization/fp8_kernel.py:1068-1145.
 *
 * a   [M, K] e4m3, row stride lda bytes (lda % 16 == 0, pointer 16-byte aligned).
 * b   [N, K] e4m3 K-contiguous (the weight as stored; the reference's column-major mat_b [K, N] is the
 *     same memory), row stride ldb bytes (ldb % 16 == 0, pointer 16-byte aligned).
 * sa  float, element (m, kb) at sa[m * sa_stride_m + kb * sa_stride_k]   (M-major or K-major).
 * sb  float, element (nb, kb) at sb[nb * sb_stride_n + kb * sb_stride_k], nb = n / 128, kb = k / 128.
 * out [M, N] out_dtype (bf16 / f16), row stride ldc ELEMENTS, (ldc * 2) % 16 == 0, pointer 16-byte aligned.
 * K need not be a multiple of 128 (the tail block is zero-filled), but K % 16 == 0.
 * fp32 accumulation; each 128-deep partial product is scaled and added in registers.
 * Any M >= 0 is accepted with no padding copy (the reference pads M to a multiple of 4).
 * Up to 128 rows the weight-streaming kernel with swapped operands runs (128 weight rows x 16 / 32 / 64 activation rows
 * per MMA; from 65 rows two such sub-tiles per work item share every weight stage), above that the 128 x 128 kernel.
 */
int sglb200_fp8_blockwise_scaled_mm(const void* a, const void* b, const float* sa, const float* sb, void* out,
                                    int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                    int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                                    int64_t sb_stride_k, int out_dtype, void* stream);

/*
 * G with split-K for small M.  When the output tiles alone cannot occupy the SMs (M <= 128 at most shapes) the kernel is
 * bound by streaming the weights; cutting K into ranges that run on different SMs restores the bandwidth.  The ranges
 * write fp32 partial sums to `workspace` ([splits, M, N] floats) and a second small kernel adds them in ascending
 * split order and casts.  sglb200_fp8_blockwise_scaled_mm_workspace_bytes() returns the size this needs for a shape on
 * the current device (0 = split-K would not be used); with workspace == NULL or a workspace that is too small the call
 * is exactly sglb200_fp8_blockwise_scaled_mm.  The workspace is scratch: contents on entry are ignored, calls on the
 * same stream may share it.  Replaces the per-call cudaMalloc'ed CUTLASS workspace of the reference
 * (sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:162-163) and its stream-K path
 * (sgl-kernel/csrc/cutlass_extensions/gemm/fp8_blockwise_gemm_sm90_dispatch.cuh:179-197).
 */
int64_t sglb200_fp8_blockwise_scaled_mm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int sglb200_fp8_blockwise_scaled_mm_ws(const void* a, const void* b, const float* sa, const float* sb, void* out,
                                       int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                       int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                                       int64_t sb_stride_k, int out_dtype, void* workspace, int64_t workspace_bytes,
                                       void* stream);

/*
 * G with split-K for callers that cannot allocate.  No counterpart in the reference.
 *
 * Same arguments and result as sglb200_fp8_blockwise_scaled_mm, same split-K decision as the _ws entry, but the
 * scratch is a fixed 16 MiB device array inside the library image (sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes()),
 * so this call never touches cudaMalloc, cudaFree or any allocating routine.  It exists for hosts that must not
 * allocate where they run the GEMM: an engine that gave all device memory to its own pool, a region in which
 * allocation is forbidden, a C caller without an allocator.
 *   - Shapes whose split-K scratch (sglb200_fp8_blockwise_scaled_mm_workspace_bytes) exceeds the built-in buffer are
 *     REJECTED with SGLB200_ERR_WORKSPACE (nothing is launched); shapes that do not use split-K run as usual.
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress, that device current);
 *     make that first call outside any stream capture.
 *   - Every call on a device shares the one array, which keeps whatever the previous call left in it.  The kernels
 *     overwrite every element they later read, so nothing needs clearing, but two calls that overlap on the GPU
 *     (different streams, no dependency between them) race on it: serialise them.
 *   - Every GPU that loads the library holds the 16 MiB until the process exits.
 */
int64_t sglb200_fp8_blockwise_scaled_mm_noalloc_max_bytes(void);
int sglb200_fp8_blockwise_scaled_mm_noalloc(const void* a, const void* b, const float* sa, const float* sb, void* out,
                                            int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                            int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                                            int64_t sb_stride_k, int out_dtype, void* stream);
/*
 * G on CTA pairs: the same result contract as sglb200_fp8_blockwise_scaled_mm (dense, any M), computed by clusters of
 * two CTAs that share one tcgen05.mma.cta_group::2 over a 256 x tile_n output tile (tile_n = 128 or 256).  Each CTA
 * loads its own 128 rows of A and half of the B rows with its own TMA copies (nothing is broadcast), which lowers the
 * L2 -> shared-memory bytes per flop to 3/4 (tile_n 128) or 1/2 (tile_n 256) of the single-CTA kernel's.  An explicit
 * alternative, not the default: measured on B200 it is level with the single-CTA kernel at tile_n = 128 and behind it at
 * tile_n = 256 on most of the benchmark's shapes (the promotion of the partial sums, not operand delivery, is what bounds
 * both).  No split-K, no scratch.
 * Replaces: the 2-SM configuration of the reference's sm_100 kernels
 *           (KernelPtrArrayTmaWarpSpecializedBlockwise2SmSm100, sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:300-310;
 *           dense launch sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:39-196).
 */
int sglb200_fp8_blockwise_scaled_mm_pair(const void* a, const void* b, const float* sa, const float* sb, void* out,
                                         int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                         int64_t sa_stride_m, int64_t sa_stride_k, int64_t sb_stride_n,
                                         int64_t sb_stride_k, int out_dtype, int tile_n, void* stream);


/*
 * G with power-of-two (UE8M0) scales, scaled by the tensor core itself (tcgen05.mma kind::mxf8f6f4.block_scale):
 *   out[m, n] = cast( sum_k a[m,k] * 2^ea[m, k/128] * b[n,k] * 2^eb[n/128, k/128] ),  fp32 accumulation over all of K.
 * Replaces: the reference's Blackwell route through DeepGEMM with UE8M0 scales, w8a8_block_fp8_matmul_deepgemm /
 *           deep_gemm.fp8_gemm_nt (python/sglang/srt/layers/quantization/fp8_kernel.py:1047-1065,
 *           deep_gemm_wrapper/entrypoint.py:68-112, configurer.py:24-25; weights requantised by
 *           fp8_utils.py:416-512).
 * a [M, K], b [N, K] e4m3 as for sglb200_fp8_blockwise_scaled_mm.
 * sfa  packed exponents of the activation scales exactly as the quantiser writes them with scale_ue8m0 != 0:
 *      int32 word (m, kg) at sfa[kg * sfa_ld + m], byte j = biased exponent of k-block 4*kg + j.
 * sfb  packed exponents of the weight scales: int32 word (nb, kg) at sfb[nb * sfb_stride_n + kg * sfb_stride_k],
 *      nb = n / 128, same byte order.
 * Exact for power-of-two scales (the same products and an fp32 sum); scales that are not powers of two cannot be
 * expressed and must use sglb200_fp8_blockwise_scaled_mm.
 */
int sglb200_fp8_ue8m0_scaled_mm(const void* a, const void* b, const int32_t* sfa, const int32_t* sfb, void* out,
                                int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sfa_ld,
                                int64_t sfb_stride_n, int64_t sfb_stride_k, int out_dtype, void* stream);
/* The same with optional split-K scratch for M <= 64 (size: sglb200_fp8_blockwise_scaled_mm_workspace_bytes; NULL = no
 * split).  Up to 64 rows both entries run the weight-streaming kernel of sglb200_fp8_blockwise_scaled_mm, which decodes
 * the exponent bytes itself (the scales stay exact powers of two); above that the block-scaling kernel. */
int sglb200_fp8_ue8m0_scaled_mm_ws(const void* a, const void* b, const int32_t* sfa, const int32_t* sfb, void* out,
                                   int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t sfa_ld,
                                   int64_t sfb_stride_n, int64_t sfb_stride_k, int out_dtype, void* workspace,
                                   int64_t workspace_bytes, void* stream);

/*
 * MG with UE8M0 scales: the kernel above with the expert tile scheduler of
 * sglb200_fp8_blockwise_scaled_grouped_mm.  Rows of expert e are [expert_offsets[e], expert_offsets[e + 1])
 * (num_experts + 1 entries); b [num_experts, N, K] with strides ldb (row) and ldb_e (expert);
 * sfa word (row, kg) at sfa[row * sfa_stride_m + kg * sfa_stride_k] (row-major after a row shuffle, or the quantiser's
 * column-major layout); sfb word (e, nb, kg) at sfb[e * sfb_stride_e + nb * sfb_stride_n + kg * sfb_stride_k].
 * Replaces: the grouped DeepGEMM calls of the reference's Blackwell MoE route with UE8M0 scales
 *           (python/sglang/srt/layers/moe/moe_runner/deep_gemm.py:131-207: m_grouped_fp8_gemm_nt_contiguous via
 *           deep_gemm_wrapper/entrypoint.py:52-66), with expert offsets instead of a per-row expert index.
 */
int sglb200_fp8_ue8m0_scaled_grouped_mm(const void* a, const void* b, const int32_t* sfa, const int32_t* sfb, void* out,
                                        const int32_t* expert_offsets, int64_t total_rows, int64_t num_experts,
                                        int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldb_e, int64_t ldc,
                                        int64_t sfa_stride_m, int64_t sfa_stride_k, int64_t sfb_stride_e,
                                        int64_t sfb_stride_n, int64_t sfb_stride_k, int out_dtype, void* stream);

/*
 * MG — grouped (per-expert) block-scaled FP8 GEMM over rows sorted by expert.
 * Replaces: fp8_blockwise_scaled_grouped_mm  sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:650-810
 *           and its pointer-table helper sgl-kernel/csrc/moe/cutlass_moe_helper.cu:17-142
 *           (schema common_extension.cc:274-279).  No pointer arrays, layout tables or workspace are needed.
 *
 * a   [total_rows, K] e4m3 (row stride lda bytes), rows of expert e are expert_offsets[e] .. expert_offsets[e+1]-1.
 * b   [E, N, K] e4m3, K-contiguous, expert stride ldb_e bytes, row stride ldb bytes.
 * sa  float [total_rows, ceil(K/128)] with strides (sa_stride_m, sa_stride_k).
 * sb  float [E, ceil(N/128), ceil(K/128)] with strides (sb_stride_e, sb_stride_n, sb_stride_k).
 * out [total_rows, N] out_dtype, row stride ldc elements.
 * expert_offsets  int32 on the device, non-decreasing; [E + 1] entries when problem_sizes is NULL.
 * problem_sizes   optional int32 [E, 3] on the device (the reference's table): when given, expert e owns
 *                 problem_sizes[3e] rows starting at expert_offsets[e] and only E offsets are read.
 */
int sglb200_fp8_blockwise_scaled_grouped_mm(const void* a, const void* b, const float* sa, const float* sb,
                                            void* out, const int32_t* expert_offsets,
                                            const int32_t* problem_sizes, int64_t total_rows,
                                            int64_t num_experts, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                            int64_t ldb_e, int64_t ldc, int64_t sa_stride_m, int64_t sa_stride_k,
                                            int64_t sb_stride_e, int64_t sb_stride_n, int64_t sb_stride_k,
                                            int out_dtype, void* stream);

/*
 * MP — routing tables for the sorted-by-expert layout.
 * Replaces: prepare_moe_input  sgl-kernel/csrc/moe/prepare_moe_input.cu:13-167 (schema common_extension.cc:281-285).
 *
 * topk_ids [num_tokens, topk] int32.  Outputs (all int32, device):
 *   expert_offsets [E + 1]; problem_sizes1 [E, 3] = (count, 2n, k); problem_sizes2 [E, 3] = (count, k, n)
 *   (either may be NULL); a_map [num_tokens * topk]: sorted row -> source token;
 *   c_map [num_tokens * topk]: token-major slot -> sorted row, -1 for ids outside [0, E).
 * Rows of one expert keep ascending slot order (deterministic; the reference's order is atomic order).
 * One launch, one thread block: num_tokens * topk <= 2^24, E <= 1024.
 */
int sglb200_prepare_moe_input(const int32_t* topk_ids, int32_t* expert_offsets, int32_t* problem_sizes1,
                              int32_t* problem_sizes2, int32_t* a_map, int32_t* c_map, int64_t num_tokens,
                              int64_t topk, int64_t num_experts, int64_t n, int64_t k, void* stream);

/*
 * MS — out[i, :] = in[dst2src[i], :] for i < num_dst_rows; rows are row_bytes long (multiple of 4).
 * Replaces: shuffle_rows  sgl-kernel/csrc/moe/prepare_moe_input.cu:169-256 (schema common_extension.cc:287-288).
 */
int sglb200_shuffle_rows(const void* input, const int32_t* dst2src, void* output, int64_t num_dst_rows,
                         int64_t row_bytes, void* stream);

/*
 * MS — out[i, :] = cast( sum_j factors[i*topk+j] * in[perm[i*topk+j], :] ), fp32 sum in ascending j;
 * slots with perm < 0 are skipped; factors may be NULL (= 1).  dtype bf16 / f16 for in, out and factors.
 * round_products == 0: products stay in fp32 (the arithmetic of the reference's CUDA kernel);
 * round_products != 0: each product is rounded to dtype before it is added, which is what the torch-native
 * expert MLP computes ((out * w.to(dtype)).sum(1), python/sglang/test/test_block_fp8.py:445-447).
 * Replaces: apply_shuffle_mul_sum  sgl-kernel/csrc/moe/prepare_moe_input.cu:258-392 (schema common_extension.cc:289-290).
 */
int sglb200_apply_shuffle_mul_sum(const void* input, void* output, const int32_t* perm, const void* factors,
                                  int64_t m, int64_t topk, int64_t hidden, int dtype, int round_products,
                                  void* stream);

/*
 * SA — out[t, :] = round(silu(in[t, :d])) * in[t, d:], d = hidden; in [num_rows, 2*hidden].
 * Replaces: silu_and_mul  sgl-kernel/csrc/elementwise/activation.cu:82-101 (schema common_extension.cc:82-83).
 */
int sglb200_silu_and_mul(const void* input, void* output, int64_t num_rows, int64_t hidden, int dtype,
                         void* stream);

/*
 * MG in the masked layout: group g owns the rows [g * max_m, g * max_m + masked_m[g]) of a / sa / out; rows past
 * masked_m[g] are neither read as results nor written (masked_m is clamped to [0, max_m]).
 *   a   [num_groups * max_m, K] e4m3, row stride lda;  sa element (g, local row, kb) at
 *       sa[g * sa_stride_g + row * sa_stride_m + kb * sa_stride_k] (row-major or MN-major per group)
 *   b   [num_groups, N, K] e4m3, strides ldb (row) and ldb_e (group);  sb element (g, nb, kb) at
 *       sb[g * sb_stride_e + nb * sb_stride_n + kb * sb_stride_k]
 *   out [num_groups * max_m, N], row stride ldc elements;  masked_m [num_groups] int32 on the device.
 * Same kernel and arithmetic as sglb200_fp8_blockwise_scaled_grouped_mm; alignment rules as there.
 * Replaces: deep_gemm.fp8_m_grouped_gemm_nt_masked as called from
 *           python/sglang/srt/layers/deep_gemm_wrapper/entrypoint.py:26-49 (third-party DeepGEMM, not in the tree;
 *           semantics pinned by torch_w8a8_block_fp8_bmm, python/sglang/test/test_block_fp8.py:549-563,586-635).
 */
int sglb200_fp8_blockwise_scaled_masked_grouped_mm(const void* a, const void* b, const float* sa, const float* sb,
                                                   void* out, const int32_t* masked_m, int64_t num_groups,
                                                   int64_t max_m, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                                   int64_t ldb_e, int64_t ldc, int64_t sa_stride_g, int64_t sa_stride_m,
                                                   int64_t sa_stride_k, int64_t sb_stride_e, int64_t sb_stride_n,
                                                   int64_t sb_stride_k, int out_dtype, void* stream);

/*
 * Router front end: probabilities = softmax(gating_output[t, :]) in fp32, then the topk largest in
 * descending order (ties go to the lower expert index); with renormalize != 0 the selected weights are
 * divided by their sum.
 *   gating_output [num_tokens, num_experts] contiguous, dtype = SGLB200_BF16 | SGLB200_F16 | SGLB200_F32
 *   topk_weights  [num_tokens, topk] fp32, topk_ids [num_tokens, topk] int32, both contiguous
 *   1 <= num_experts <= 1024 (any value, no power-of-two rule and no workspace), 1 <= topk <= num_experts.
 * Replaces: topk_softmax  sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:512-590
 *           (schema common_extension.cc:259-260; caller python/sglang/srt/layers/moe/topk.py fused_topk).
 */
int sglb200_topk_softmax(const void* gating_output, int dtype, float* topk_weights, int32_t* topk_ids,
                         int64_t num_tokens, int64_t num_experts, int64_t topk, int renormalize, void* stream);

/*
 * Sigmoid router with a selection bias and two-level top-k (the DeepSeek-V3 gate), always renormalised:
 *   s = sigmoid(input[t, e]); b = s + bias[e] (both rounded to the input type);
 *   score of a group (num_experts / num_expert_group consecutive experts) = sum of its two largest b;
 *   the topk_group best groups stay (ties: lower group); inside them the topk - num_fused_shared_experts best b are
 *   taken in descending order (ties: lower expert) with weight s; slots after them get the ids num_experts,
 *   num_experts + 1, ... and the weight sum / routed_scaling_factor; every weight is then divided by the sum of the
 *   routed weights and, with apply_routed_scaling_factor_on_output != 0, multiplied by routed_scaling_factor.
 *   input [num_tokens, num_experts] and bias [num_experts] share dtype (SGLB200_BF16 | F16 | F32), contiguous;
 *   topk_weights [num_tokens, topk] fp32, topk_ids [num_tokens, topk] int32.
 * Limits: num_experts <= 1024 (any value divisible by num_expert_group, no power-of-two rule), num_expert_group <= 32,
 *   at least 2 experts per group, topk <= 32.
 * Replaces: moe_fused_gate  sgl-kernel/csrc/moe/moe_fused_gate.cu:52-262,378-525 (schema common_extension.cc:268-272);
 *           torch-native twin biased_grouped_topk_impl  python/sglang/srt/layers/moe/topk.py:595-665.
 */
int sglb200_moe_fused_gate(const void* input, const void* bias, int dtype, float* topk_weights, int32_t* topk_ids,
                           int64_t num_tokens, int64_t num_experts, int64_t num_expert_group, int64_t topk_group,
                           int64_t topk, int64_t num_fused_shared_experts, float routed_scaling_factor,
                           int apply_routed_scaling_factor_on_output, void* stream);

/*
 * Block-aligned counting sort of the flattened expert ids, the routing table of the tile-gather MoE runner.
 * Bucket b (0 <= b < num_buckets) collects the slots whose id is b - 1; bucket 0 therefore holds id -1
 * (slots of experts another rank owns).  Each bucket is padded to a multiple of block_size.
 *   topk_ids            [numel] int32, values in [-1, num_buckets - 2]
 *   sorted_token_ids    [>= numel + num_buckets * (block_size - 1)] int32: slot indices bucket by bucket, inside a
 *                       bucket in ASCENDING slot order (the reference's order inside a bucket is whatever its
 *                       atomics produce); with pad_sorted_token_ids != 0 the padding entries below
 *                       num_tokens_post_pad are set to numel, otherwise the caller pre-fills the array
 *   expert_ids          [>= capacity / block_size] int32: bucket index - 1 of each block
 *   num_tokens_post_pad [1] int32: total padded length
 *   cumsum              [num_buckets + 1] int32 or NULL: padded start of every bucket, then the total (the
 *                       reference leaves its sort cursors there; no caller reads them)
 * Limits: numel <= 2^24, num_buckets <= 1024, block_size <= 4096.
 * Replaces: moe_align_block_size  sgl-kernel/csrc/moe/moe_align_kernel.cu:302-364 (kernels :28-300;
 *           schema common_extension.cc:253-257); the caller passes num_experts + 1 as num_buckets
 *           (python/sglang/srt/layers/moe/fused_moe_triton/moe_align_block_size.py:17-88).
 */
int sglb200_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int64_t num_buckets, int64_t block_size,
                                 int32_t* sorted_token_ids, int32_t* expert_ids, int32_t* num_tokens_post_pad,
                                 int32_t* cumsum, int pad_sorted_token_ids, void* stream);

/*
 * output[t, :] = cast(routed_scaling_factor * sum_j input[t, j, :]); fp32 sum in ascending j.
 *   input [num_tokens, topk, hidden], output [num_tokens, hidden], contiguous, dtype = SGLB200_BF16 | SGLB200_F16,
 *   hidden % 8 == 0, 16-byte aligned pointers.
 * Replaces: moe_sum_reduce  sgl-kernel/csrc/moe/moe_sum_reduce.cu:227-403 (schema common_extension.cc:262-263).
 */
int sglb200_moe_sum_reduce(const void* input, void* output, int64_t num_tokens, int64_t topk, int64_t hidden,
                           int dtype, float routed_scaling_factor, void* stream);

/*
 * GEMM + all-reduce over peer memory for the row-parallel linear at small M (each rank holds a K-slice and produces a
 * full [M, N] partial sum).  Two launches per rank, no collective library call:
 *   1. sglb200_fp8_blockwise_scaled_mm_push: the GEMM of sglb200_fp8_blockwise_scaled_mm whose epilogue stores every
 *      output tile straight into the receive buffer of EVERY rank (peer stores over NVLink; slot [epoch & 1][rank])
 *      and then raises that tile's flag words there, so the transfer runs tile by tile under the remaining math.
 *   2. sglb200_peer_reduce: waits (bounded) per tile until all `world` ranks' flag words reached the epoch, adds the
 *      `world` slots in fp32 in ascending rank order (every rank gets the same bits) and writes `out`.
 * Memory, per rank, mapped by every rank (sglb200_peer_alloc / sglb200_peer_open, or any peer-accessible allocation):
 *   receive buffer  sglb200_peer_recv_bytes(slot_elems) bytes = [2][8][slot_elems] 16-bit elements, M * N <= slot_elems;
 *   flag words      sglb200_peer_flag_bytes() bytes, zero before the first call; the tail holds this rank's
 *                   control words (exchanges completed, block tickets, failure mark).
 * peer_recv / peer_flags are HOST arrays of `world` device pointers, entry r = rank r's buffer as mapped in this
 * process.  The epoch of an exchange is (exchanges completed) + 1; it lives in the control words, both kernels read it
 * there and the last block of the reduce kernel advances it, so the pair of launches can be captured in a CUDA graph
 * and replayed.  Rules: all ranks issue the same sequence of exchanges, each on ONE stream per rank (the two
 * alternating slot sets are safe exactly because a rank's exchange e + 1 is enqueued after its exchange e); at most
 * 1024 output tiles of 128 x 128; world <= 8.
 * workspace / workspace_bytes: scratch for M <= 128 (size from sglb200_fp8_blockwise_scaled_mm_push_workspace_bytes; 0 for
 * larger M).  With it the few-rows weight-streaming kernel computes fp32 sums (K split over the SMs where that pays) and
 * a second small kernel adds the splits, casts and does the pushing and flagging; without it (NULL) the 128-row kernel
 * with the push epilogue runs.  Both produce the bits of the corresponding plain entry point.
 * A wait that runs out (a rank that never pushed) leaves its tile unwritten, sets device status 5
 * (sglb200_read_device_status) and does not advance the epoch, so the same exchange can be reduced again once the
 * missing rank has pushed; if only some ranks timed out the group is out of step and the buffers must be set up
 * again.  timeout_ns <= 0 selects 2 s.
 * Replaces: the one-shot path of the custom all-reduce the reference uses under its row-parallel linear at small sizes
 *           (sgl-kernel/csrc/allreduce/custom_all_reduce.cuh:203-266, python/sglang/srt/layers/linear.py:1379-1380,
 *           python/sglang/srt/distributed/device_communicators/custom_all_reduce.py), fused with the GEMM before it.
 */
int sglb200_fp8_blockwise_scaled_mm_push(const void* a, const void* b, const float* sa, const float* sb, int64_t M,
                                         int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t sa_stride_m,
                                         int64_t sa_stride_k, int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype,
                                         void* const* peer_recv, void* const* peer_flags, int rank, int world,
                                         int64_t slot_elems, void* workspace, int64_t workspace_bytes, void* stream);
int64_t sglb200_fp8_blockwise_scaled_mm_push_workspace_bytes(int64_t M, int64_t N, int64_t K);
/*
 * The same exchange in two shots, for outputs too large to send whole to every rank (three launches per rank, same
 * buffers, same rules, freely mixed with the one-shot form from one exchange to the next):
 *   1. sglb200_fp8_blockwise_scaled_mm_push_scatter: the 128-row GEMM whose epilogue stores output tile t only into the
 *      receive buffer of rank t % world (tiles numbered row-major over the 128 x 128 grid) and flags it there.
 *   2. sglb200_peer_reduce_scatter: per owned tile waits (bounded) for the `world` partial tiles, adds them in fp32 in
 *      ascending rank order (the bits the one-shot reduce produces), writes the tile to this rank's `out` and stores it
 *      into every other rank's slot [epoch & 1][this rank] at the tile's position, then flags it there.
 *   3. sglb200_peer_gather: waits (bounded) for the tiles this rank does not own and copies them into `out`; its last
 *      block advances the epoch.
 * Bytes leaving a rank per exchange: 2 (world - 1) / world x the output instead of (world - 1) x the output.  Needs at
 * least `world` output tiles (SGLB200_ERR_SHAPE otherwise); `out` is the same [M, N] tensor in 2 and 3.  A wait that
 * runs out in either kernel sets device status 5 and keeps the epoch, as above.
 * Replaces: the two-stage path of the reference's custom all-reduce (reduce-scatter, then all-gather:
 *           sgl-kernel/csrc/allreduce/custom_all_reduce.cuh:225-266, cross_device_reduce_2stage), fused with the GEMM before it.
 */
int sglb200_fp8_blockwise_scaled_mm_push_scatter(const void* a, const void* b, const float* sa, const float* sb, int64_t M,
                                                 int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t sa_stride_m,
                                                 int64_t sa_stride_k, int64_t sb_stride_n, int64_t sb_stride_k,
                                                 int out_dtype, void* const* peer_recv, void* const* peer_flags, int rank,
                                                 int world, int64_t slot_elems, void* stream);
int sglb200_peer_reduce_scatter(void* const* peer_recv, void* const* peer_flags, void* out, int64_t M, int64_t N,
                                int64_t ldc, int out_dtype, int rank, int world, int64_t slot_elems, int64_t timeout_ns,
                                void* stream);
int sglb200_peer_gather(const void* recv_local, void* flags_local, void* out, int64_t M, int64_t N, int64_t ldc,
                        int out_dtype, int rank, int world, int64_t slot_elems, int64_t timeout_ns, void* stream);
int sglb200_peer_reduce(const void* recv_local, void* flags_local, void* out, int64_t M, int64_t N, int64_t ldc,
                        int out_dtype, int world, int64_t slot_elems, int64_t timeout_ns, void* stream);
int64_t sglb200_peer_flag_bytes(void);
int64_t sglb200_peer_recv_bytes(int64_t slot_elems);
/* Exchanges this rank has completed (its control word).  SYNCHRONISES (cudaMemcpy); for tests and debugging. */
int sglb200_peer_completed(const void* flags_local, int64_t* completed);

/*
 * Expert-parallel token dispatch and combine over peer memory: the all-to-alls of the MoE layer without a collective
 * library and without a host round trip for the row counts.  Every rank owns one exchange buffer of
 * sglb200_ep_buffer_bytes(capacity, H, topk, world, m_max) bytes, zero before the first use, mapped by every rank
 * (sglb200_peer_alloc / sglb200_peer_open); peer_bases is a HOST array of `world` device pointers, entry r = rank r's
 * buffer as mapped in this process.  capacity = rows a rank can receive per exchange, m_max = tokens a rank may send.
 * Choose capacity >= world * m_max (a token goes to a rank at most once, so that always fits; the Python wrapper refuses
 * less): with a smaller one a full buffer DROPS rows (status 23) and the combine adds stale data for them.  sglb200_ep_buffer_offsets returns the byte offsets of {recv_q [capacity, H] e4m3,
 * recv_s [capacity, H/128] f32, recv_meta [capacity, 2] i32, recv_ids [capacity, topk] i32, recv_w [capacity, topk] f32,
 * comb [world, m_max, H] 16-bit, control words} inside a buffer.  One exchange = four launches on one stream per rank,
 * the same sequence on every rank; the exchange counter lives in the control words (read by all four kernels, advanced
 * by the last block of the combine-reduce kernel), so the layer can be captured in a CUDA graph and replayed:
 *   sglb200_ep_dispatch        every token of this rank (q [M, H] e4m3, scales s, topk_ids with GLOBAL expert ids, fp32
 *                              weights) is stored once into the buffer of every rank that owns one of its experts
 *                              (expert e lives on rank e / num_local_experts), in a row reserved there by a remote atomic.
 *   sglb200_ep_dispatch_quant  the same with the activation quantiser in front: x [M, H] bf16 / f16 (row stride ldx
 *                              elements) is read once, quantised per 128-wide group with the e4m3 limits and fp32 scales
 *                              (floor eps), and the codes and scales go straight into the owners' receive rows; bit-
 *                              identical to sglb200_per_token_group_quant_fp8 followed by sglb200_ep_dispatch.  Takes the
 *                              place of sglb200_ep_dispatch in the sequence.
 *   sglb200_ep_receive         waits (bounded) until every rank has finished dispatching; rows that were not received
 *                              get ids -1; count_out (device int32, may be NULL) = rows received.  The caller then runs
 *                              the expert MLP on recv_q / recv_s / recv_ids / recv_w over `capacity` rows
 *                              (sglb200 grouped GEMMs skip ids < 0) and gets one partial output row per received row.
 *   sglb200_ep_combine_push    partial [capacity, H] (bf16 / f16): row i goes back to its source token.
 *   sglb200_ep_combine_reduce  waits (bounded) until every rank has returned its rows; out[t] = sum of the partial rows of
 *                              token t over the ranks that own one of its experts, ascending rank, fp32.
 * The order of the received rows depends on timing, the result does not.  A wait that runs out sets device status 21
 * (receive) or 22 (combine); a full receive buffer drops the row and sets 23 (sglb200_read_device_status).
 * Replaces: DeepEP Buffer.dispatch / Buffer.combine as called from
 *           python/sglang/srt/layers/moe/token_dispatcher/deepep.py:398-492 (third party, not in the tree), the
 *           reorder kernels python/sglang/srt/layers/moe/ep_moe/kernels.py:435-720, and for the _quant form the
 *           quantisation the dispatcher runs before it sends (token_dispatcher/deepep.py:360-371).
 */
int64_t sglb200_ep_buffer_bytes(int64_t capacity, int64_t H, int64_t topk, int64_t world, int64_t m_max);
int sglb200_ep_buffer_offsets(int64_t capacity, int64_t H, int64_t topk, int64_t world, int64_t m_max, int64_t* offsets7);
int sglb200_ep_dispatch(const void* q, const float* s, int64_t s_stride_m, int64_t s_stride_k, const int32_t* topk_ids,
                        const float* topk_weights, int64_t M, int64_t H, int64_t topk, int64_t num_local_experts,
                        void* const* peer_bases, int rank, int world, int64_t capacity, int64_t m_max, void* stream);
int sglb200_ep_dispatch_quant(const void* x, int in_dtype, int64_t ldx, const int32_t* topk_ids, const float* topk_weights,
                              int64_t M, int64_t H, int64_t topk, int64_t num_local_experts, void* const* peer_bases,
                              int rank, int world, int64_t capacity, int64_t m_max, float eps, void* stream);
int sglb200_ep_receive(void* const* peer_bases, int rank, int world, int64_t H, int64_t topk, int64_t num_local_experts,
                       int64_t capacity, int64_t m_max, int32_t* count_out, int64_t timeout_ns, void* stream);
int sglb200_ep_combine_push(const void* partial, int dtype, void* const* peer_bases, int rank, int world, int64_t H,
                            int64_t topk, int64_t num_local_experts, int64_t capacity, int64_t m_max, void* stream);
int sglb200_ep_combine_reduce(void* const* peer_bases, int rank, int world, const int32_t* topk_ids, void* out, int dtype,
                              int64_t M, int64_t H, int64_t topk, int64_t num_local_experts, int64_t capacity,
                              int64_t m_max, int64_t timeout_ns, void* stream);
/* Exchanges this rank has completed (its control word).  SYNCHRONISES (cudaMemcpy); for tests and debugging. */
int sglb200_ep_completed(const void* local_base, int64_t capacity, int64_t H, int64_t topk, int64_t world, int64_t m_max,
                         int64_t* completed);

/*
 * Set-up calls for the buffers above; the only entry points that ALLOCATE device memory, and they synchronise.
 * sglb200_peer_alloc: cudaMalloc + zero fill on the current device, and the 64-byte CUDA IPC handle another process
 * passes to sglb200_peer_open to map the same memory (peer access is enabled on first use).  sglb200_peer_close
 * unmaps an opened pointer, sglb200_peer_free releases an allocated one.
 * Replaces: the IPC buffer set-up of custom_all_reduce.py (create_shared_buffer / free_shared_buffer) and
 *           sgl-kernel/csrc/allreduce/custom_all_reduce.cu (init_custom_ar, register_buffer).
 */
int sglb200_peer_alloc(int64_t bytes, void** dev_ptr, unsigned char* handle64);
int sglb200_peer_open(const unsigned char* handle64, void** dev_ptr);
int sglb200_peer_close(void* dev_ptr);
int sglb200_peer_free(void* dev_ptr);

/*
 * In-place sum over the ranks of one node of a bf16 / f16 buffer that every rank maps through ONE NVLink multicast
 * address (NVSwitch in-switch reduction): the all-reduce after a row-parallel linear for outputs too large for the
 * push epilogues above.  Rank r reduces the r-th slice of the buffer with multimem.ld_reduce (fp32 accumulation in the
 * switch, ONE rounding of the sum) and writes the sums into every rank's memory with multimem.st, so each GPU sends and
 * receives the buffer once.  Two bounded cross-rank barriers (flag words in peer memory, per-block epochs kept on the
 * device: graph-replayable) make the call safe after the producer kernel on every rank's stream and complete on every
 * rank when it ends.  Every rank must make the same call on its own stream, and the ranks' kernels must be able to run
 * at the same time (one GPU per rank).
 *   multicast_addr  address of element 0 of the buffer in the MULTICAST mapping (not the local one), 16-byte aligned.
 *   flag_blocks     HOST array of `world` device addresses: entry r = rank r's flag block (sglb200_nvls_flag_bytes()
 *                   bytes, zero before the first call) as mapped in this process.
 *   numel           elements, a multiple of 8.
 *   blocks          thread blocks of the kernel, 1..128, 0 = 128; THE SAME ON EVERY RANK for a given call (block b pairs
 *                   with block b of the peers).  Few blocks leave SMs to a GEMM that runs beside the all-reduce.
 * The library creates neither the multicast object nor the peer mappings; the Python side (sglang_b200.distributed.nvls)
 * takes both from torch's symmetric-memory allocator.  A wait that runs out sets status 41 / 42 (first / second barrier).
 * Replaces: the all-reduce the reference's row-parallel linear calls for large outputs, GroupCoordinator.all_reduce
 *           python/sglang/srt/distributed/parallel_state.py:513-629 (pynccl / torch.distributed route), and the
 *           symmetric-memory route device_communicators/torch_symm_mem.py (multimem_all_reduce_).
 */
int sglb200_nvls_all_reduce(uint64_t multicast_addr, const uint64_t* flag_blocks, int rank, int world, int64_t numel,
                            int dtype, int blocks, void* stream);
int64_t sglb200_nvls_flag_bytes(void);

/*
 * The dense GEMM and the multicast all-reduce of its output in ONE cooperative launch: the row-parallel linear for
 * large outputs.  The last comm_ctas CTAs of the grid compute no tiles; row block by row block (2048 rows: one raster
 * group of the tile schedule) they wait until the tile CTAs of the same grid have stored the block (a device counter per
 * row block), pair up with the same CTAs of the other ranks' kernels (flag words as in sglb200_nvls_all_reduce) and sum
 * the block through the switch (multimem.ld_reduce / multimem.st) while the tile CTAs compute the next block; only the
 * last block's reduction is exposed.  Every wait is bounded (status 6: the row block was never finished, 7 / 8: a peer
 * never arrived).
 *   out            this rank's mapping of the symmetric buffer, [M, N] contiguous; multicast_out = the multicast
 *                  address of the same element (0, 0).
 *   flag_blocks    as for sglb200_nvls_all_reduce (the two calls may share them; all ranks make the same sequence).
 *   done_counters  64 device words of scratch owned by this rank (zeroed by the call, on the stream).
 *   comm_ctas      1..64, THE SAME ON EVERY RANK; the GEMM runs on the SMs that are left.
 * One such call at a time per GPU (the kernel occupies every SM it is given; a cooperative launch fails otherwise).
 * Replaces: RowParallelLinear.forward + tensor_model_parallel_all_reduce, python/sglang/srt/layers/linear.py:1361-1386,
 *           for outputs above the custom all-reduce's size limit.
 */
int sglb200_fp8_blockwise_scaled_mm_allreduce(const void* a, const void* b, const float* sa, const float* sb, void* out,
                                              uint64_t multicast_out, const uint64_t* flag_blocks, void* done_counters,
                                              int rank, int world, int comm_ctas, int64_t M, int64_t N, int64_t K,
                                              int64_t lda, int64_t ldb, int64_t sa_stride_m, int64_t sa_stride_k,
                                              int64_t sb_stride_n, int64_t sb_stride_k, int out_dtype, void* stream);

/*
 * Device-side status word of the GEMM kernels: 0, or the code of the first bounded wait that timed out
 * (1 TMA producer, 2 or 3 MMA issuer, 4 promotion warps, 5 peer-flag wait of sglb200_peer_reduce, 6-8 the communication
 * CTAs of sglb200_fp8_blockwise_scaled_mm_allreduce, 11-18 the same
 * roles in the UE8M0 and few-rows kernels, 21-23 the expert-parallel exchange, 31-35 the CTA-pair kernel, 41-42 the multicast all-reduce).  Every
 * kernel family keeps its own word; each call reads AND clears all of them and returns the first non-zero one, so a
 * status never surfaces on a later, unrelated read.  This call SYNCHRONISES the device (cudaMemcpyFromSymbol); it is for
 * tests and debugging, not for the serving path.  Returns -1 if the read itself failed.  No counterpart in the reference (its kernels have no bounded waits).
 */
int sglb200_read_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* SGLB200_H_ */
