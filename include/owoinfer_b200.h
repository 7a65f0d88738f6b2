/* owoinfer_b200 — C ABI of the B200 (sm_100a) implementation of the quantized MOSS-Image DiT block.
 *
 * Every entry point replaces one function of the reference engine's quantized-block path and keeps its argument
 * order, preconditions and error behaviour; the reference symbol is cited above each declaration (paths inside the
 * reference project). Conventions, mirrored from include/mossinfer/mossinfer.h:5-45,94-113:
 *   - plain C: pointers, sizes, POD structs; no C++ type or exception crosses the boundary;
 *   - every function returns a b2_status; on failure b2_last_error_message() holds a thread-local description;
 *   - all data pointers are DEVICE pointers unless the name says host; row strides are in ELEMENTS;
 *   - the caller owns all memory and passes the CUDA stream (a cudaStream_t passed as void*; NULL = default stream);
 *   - no allocation and no host synchronisation on the hot path (the one-time SiTU table fill is the documented
 *     exception, as in the reference);
 *   - invalid arguments are rejected before any launch (B2_ERR_INVALID_ARGUMENT; the reference throws
 *     std::invalid_argument), m == 0 is a no-op.
 */
#ifndef OWOINFER_B200_H_
#define OWOINFER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: the numeric values of mi_status (include/mossinfer/mossinfer.h:94-108) that this path can return. */
typedef enum b2_status {
  B2_OK = 0,
  B2_ERR_INVALID_ARGUMENT = -1,
  B2_ERR_NOT_SUPPORTED = -3,
  B2_ERR_CUDA = -8,
  B2_ERR_INTERNAL = -9
} b2_status;

/* mi_last_error_message (include/mossinfer/mossinfer.h:113): thread-local text of the last failure on this thread. */
const char* b2_last_error_message(void);

/* kInt8NumericsVersion (src/kernels/quant/quant.h:38), kInt4NumericsVersion (src/kernels/quant4/quant4.h:36),
 * attention_q8::kNumericsVersion (src/kernels/attention_q8/attention_q8.h:73), kGroupedDecodeVersion
 * (src/kernels/quant/w4a8_decode.h:27): which = 0, 1, 2, 3; any other value returns 0. The INT8, INT4 and grouped-decode
 * values are the reference's (the outputs are bit-identical to its kernels). The attention value carries the
 * reference's contract version in its low half and this library's kernel revision in its high half: the output meets
 * the reference's tolerances but not its bits. */
uint32_t b2_numerics_version(int which);

/* ---------------------------------------------------------------------------------------------------------------
 * Activation quantisers (bf16 in, int8 / packed int4 + one f32 scale per token out).
 * ------------------------------------------------------------------------------------------------------------- */

/* quant::rotate_quantize (src/kernels/quant/quant.h:48). x bf16 [m,k] stride ldx; q int8 [m,k] stride ldq; scale f32 [m].
 * k % 256 == 0, k <= 32768, x and q 16-byte aligned, ldx % 8 == 0, ldq % 16 == 0. */
int b2_rotate_quantize(const void* x, int64_t ldx, int8_t* q, int64_t ldq, float* scale, int64_t m, int k,
                       void* stream);

/* b2_rotate_quantize on a column-chunked input: columns [i * chunk_cols, (i + 1) * chunk_cols) of every row are read
 * from chunk i, a bf16 [m, chunk_cols] matrix of row stride ldx that starts chunk_stride elements after chunk i - 1
 * (chunk_cols % 16 == 0, k % chunk_cols == 0). Same bits as b2_rotate_quantize on the assembled rows. The input layout
 * of the sequence-parallel block's output projection; no counterpart in the reference. */
int b2_rotate_quantize_chunked(const void* x, int64_t ldx, int chunk_cols, int64_t chunk_stride, int8_t* q, int64_t ldq,
                               float* scale, int64_t m, int k, void* stream);

/* quant::rms_norm_modulate_rotate_quantize (src/kernels/quant/quant.h:62). norm_weight, mod_scale, mod_shift bf16 [k],
 * 16-byte aligned. y (optional, may be NULL): bf16 [m,k] stride ldy receives the norm output. The mean of squares is
 * summed in the order torch uses for an [m,k] input, which depends on m: call once per tensor the reference normalises. */
int b2_rms_norm_modulate_rotate_quantize(const void* x, int64_t ldx, const void* norm_weight, const void* mod_scale,
                                         const void* mod_shift, int8_t* q, int64_t ldq, float* scale, int64_t m, int k,
                                         void* stream, void* y, int64_t ldy);

/* quant4::convrot_quantize_int4 (src/kernels/quant4/quant4.h:45). q packed int4 [m,k/2] bytes, stride ldq bytes,
 * even column in the low nibble. ldq % 16 == 0, ldq >= k/2. */
int b2_convrot_quantize_int4(const void* x, int64_t ldx, uint8_t* q, int64_t ldq, float* scale, int64_t m, int k,
                             void* stream);

/* quant4::rms_norm_modulate_convrot_quantize_int4 (src/kernels/quant4/quant4.h:51). */
int b2_rms_norm_modulate_convrot_quantize_int4(const void* x, int64_t ldx, const void* norm_weight,
                                               const void* mod_scale, const void* mod_shift, uint8_t* q, int64_t ldq,
                                               float* scale, int64_t m, int k, void* stream);

/* moss_dit::unpack_int4 (src/models/moss_dit/dit_kernels.h:32): packed signed nibbles [rows,k/2] (stride ldp bytes) ->
 * int8 [rows,k] (stride ldo). k % 32 == 0, 16-byte aligned rows. */
int b2_unpack_int4(const void* packed, int64_t ldp, int8_t* out, int64_t ldo, int64_t rows, int64_t k, void* stream);

/* quant::decode_grouped_int8 (src/kernels/quant/w4a8_decode.h:39), 4-bit codes only: packed [rows,k/2]; group scales
 * s_rel [rows,k/group] as e4m3 bytes (scale_kind 0, the reference's format) or fp16 (scale_kind 1); codebook f32 [16]
 * or NULL (level = code - 8); out int8 [rows,k]. group % 16 == 0, k % group == 0, rows < 2^31, k <= 131071.
 * Untrusted scales, as in the reference (w4a8_decode.cu:57-62): a group whose scale is NaN or negative decodes to zeros
 * and ORs 1 into the device word `invalid` (never cleared here); invalid == NULL uses a word inside the library, read
 * with b2_w4_invalid_scales. */
int b2_decode_grouped_int8(const void* packed, const void* s_rel, int scale_kind, const float* codebook, int64_t rows,
                           int64_t k, int group, int8_t* out, unsigned* invalid, void* stream);

/* The library's own "a group scale was NaN or negative" word of the current device (set by b2_decode_grouped_int8 with
 * invalid == NULL, by b2_w4a8_gemm* and by the W4A8 tier of the block): copied to *host_value, then zeroed when
 * clear != 0. Synchronises the device: for load-time checks and tests, not for the hot path. The reference hands the
 * caller's word to every decode (w4a8_decode.h:39); this is that word kept by the library. */
int b2_w4_invalid_scales(unsigned* host_value, int clear);

/* ---------------------------------------------------------------------------------------------------------------
 * INT8 x INT8 -> INT32 GEMM with fused epilogues.
 * ------------------------------------------------------------------------------------------------------------- */

/* quant::Int8Operands (src/kernels/quant/quant.h:82-89). x_q int8 [m,k] stride ldx with x_scale f32 [m]; w int8 [n,k]
 * contiguous with w_scale f32 [n]. 16-byte aligned x_q, w, w_scale; k % 16 == 0; ldx % 16 == 0; 0 < k <= 131071. */
typedef struct b2_int8_operands {
  const int8_t* x_q;
  int64_t ldx;
  const float* x_scale;
  const int8_t* w;
  const float* w_scale;
  int64_t m, n, k;
} b2_int8_operands;

/* quant::Int8Tile (src/kernels/quant/quant.h:77). The tcgen05 kernel has its own tiles; every tile gives the same
 * bits (the int32 sum is exact). 0 = auto. */
typedef enum b2_int8_tile { B2_TILE_AUTO = 0, B2_TILE_128x256 = 1, B2_TILE_128x128 = 2, B2_TILE_2CTA_256x256 = 3 } b2_int8_tile;

/* quant::int8_gemm (src/kernels/quant/quant.h:92): out = bf16((acc * x_scale[r]) * w_scale[c] + bias[c]).
 * bias bf16 [n] or NULL; out bf16 stride ldo, 16-byte aligned, ldo % 8 == 0, n % 8 == 0. */
int b2_int8_gemm(const b2_int8_operands* op, const void* bias, void* out, int64_t ldo, void* stream, int tile);

/* b2_int8_gemm with a column-chunked output: columns [i * chunk_cols, (i + 1) * chunk_cols) of every row go to chunk i,
 * a bf16 [m, chunk_cols] matrix of row stride ldo that starts chunk_stride elements after chunk i - 1
 * (chunk_cols % 8 == 0, n % chunk_cols == 0, ldo >= chunk_cols). Same values as b2_int8_gemm. The output layout of the
 * sequence-parallel block's QKV projection (one chunk per destination rank); no counterpart in the reference. */
int b2_int8_gemm_chunked(const b2_int8_operands* op, const void* bias, void* out, int64_t ldo, int chunk_cols,
                         int64_t chunk_stride, void* stream, int tile);

/* quant::int8_gemm_gated_residual (src/kernels/quant/quant.h:98): residual += bf16(bf16(y) * gate[c]) in place. */
int b2_int8_gemm_gated_residual(const b2_int8_operands* op, const void* bias, const void* gate, void* residual,
                                int64_t ldr, void* stream, int tile);

/* quant::int8_gemm_situ_glu (src/kernels/quant/quant.h:110): w is [2F,k] stored [hidden | gate], op->n = 2F;
 * out bf16 [m,F] stride ldo, 8-byte aligned, ldo % 4 == 0, F % 4 == 0. The first call on a device outside stream
 * capture fills two 128 KiB factor tables on `stream` and synchronises it once. */
int b2_int8_gemm_situ_glu(const b2_int8_operands* op, void* out, int64_t ldo, void* stream, int tile);

/* The raw int32 accumulators of the same GEMM core, acc int32 [m,n] stride ldacc (the scalar oracle kernel of
 * tests/unit/test_quant_kernels.cu:208-231 computes these; here the tensor-core kernel dumps its own). */
int b2_int8_gemm_acc(const b2_int8_operands* op, int32_t* acc, int64_t ldacc, void* stream, int tile);

/* W4A8 GEMM: 4-bit grouped weight codes decoded to the INT8 grid (b2_decode_grouped_int8's rule) and multiplied by
 * INT8 activations; bit-identical to quant::decode_grouped_int8 followed by quant::int8_gemm
 * (src/kernels/quant/w4a8_decode.h:1-39 + src/kernels/quant/quant.h:92). scratch: device int8 [n,k] for the decoded
 * weight (caller-owned; may be reused across calls). epilogue: 0 plain (aux = bias or NULL), 1 gated residual
 * (aux = gate, out = residual in place), 2 SiTU-GLU. Every argument is checked before anything is launched; m == 0
 * launches nothing. A NaN or negative group scale decodes to zeros and is reported by b2_w4_invalid_scales.
 * Two routes with identical results: the codes are expanded inside the GEMM's B-operand staging (e4m3 group scales, a
 * power-of-two group size, k % 128 == 0; chosen automatically for few rows, see b2_debug_w4a8_route; scratch is then not
 * touched and may be NULL), or decoded to `scratch` (int8 [n, k]) first and multiplied by the INT8 kernel. */
typedef struct b2_w4_weight {
  const void* packed;   /* uint8 [n, k/2] */
  const void* s_rel;    /* [n, k/group] e4m3 or fp16 */
  int scale_kind;       /* 0 e4m3, 1 fp16 */
  int group;
  const float* codebook; /* f32 [16] or NULL */
  const float* s_channel; /* f32 [n]: the GEMM's w_scale */
} b2_w4_weight;
int b2_w4a8_gemm(const int8_t* x_q, int64_t ldx, const float* x_scale, const b2_w4_weight* w, int64_t m, int64_t n,
                 int64_t k, int epilogue, const void* aux, void* out, int64_t ldo, int8_t* scratch, void* stream);

/* Which of b2_w4a8_gemm's two routes runs: -1 automatic (the default: decode inside the GEMM up to 256 rows of
 * activations, where the GEMM is bound by the weight's bytes; decode to the scratch above, where it is bound by the
 * tensor core and expanding the weight once beats expanding it per M tile), 0 always the scratch, 1 the fused kernel
 * whenever the weight's format allows. For tests and timing; B2_W4A8_FUSED=0|1 in the environment sets the start value.
 * No counterpart in the reference. */
int b2_debug_w4a8_route(int route);

/* b2_w4a8_gemm without a scratch argument, for hosts that cannot give this call any device memory of their own and
 * are not allowed to allocate: a plug-in running on a step path where the CUDA allocator is off limits (an allocation
 * can synchronise the device or fail in the middle of a step), or an embedding whose arena was sized before the W4A8
 * tier was chosen. The decoded INT8 weight is written to a 16 MiB array inside the library's own device image, so
 * n * k must not exceed 16 MiB (16777216); larger weights are refused with B2_ERR_INVALID_ARGUMENT and need
 * b2_w4a8_gemm. Nothing is allocated or freed, by this call or by anything it calls. Every GPU that loads the library
 * carries the array until the process ends. The first call on a device looks up the array's device address (the device
 * must be current); make that first call before capturing a stream. All calls on a device share the one array and it
 * keeps what the last call decoded: two calls whose kernels can overlap on the GPU (different streams) race on it, so
 * serialise them. Nothing in it needs clearing: each call overwrites the n * k bytes it then reads.
 * No counterpart in the reference, whose callers always own their buffers. */
int b2_w4a8_gemm_noalloc(const int8_t* x_q, int64_t ldx, const float* x_scale, const b2_w4_weight* w, int64_t m, int64_t n,
                         int64_t k, int epilogue, const void* aux, void* out, int64_t ldo, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * QK-norm + RoPE, RoPE table, 8-bit attention.
 * ------------------------------------------------------------------------------------------------------------- */

/* kernels::fused::qk_norm_rope_moss (src/kernels/fused/qk_norm_rope.h:17). qkv bf16 [tokens, >= 2*heads*128] stride ld
 * (q heads then k heads), rewritten in place; q_norm, k_norm bf16 [128]; table bf16 [tokens,128] = [sin64|cos64]. */
int b2_qk_norm_rope_moss(void* qkv, int64_t ld, int64_t tokens, int heads, const void* q_norm, const void* k_norm,
                         const void* table, int64_t table_ld, void* stream);

/* kernels::moss_rope_table (src/kernels/basic/rope.h:37): out bf16 [height*width + text_length, 128] stride ld. */
int b2_moss_rope_table(void* out, int64_t ld, int height, int width, int text_length, void* stream);
/* kernels::moss_rope_table_reference (src/kernels/basic/rope.h:43; rope.cu:53-71, 169-180): the rows of reference image
 * `index` (0-based) of the edit layout, bf16 [height * width, 128]: coordinates (index + 1, 0, centred row, centred
 * column) with moss_rope_table's bands and arithmetic. */
int b2_moss_rope_table_reference(void* out, int64_t ld, int height, int width, int index, void* stream);

/* attention_q8::Variant / Options (src/kernels/attention_q8/attention_q8.h:75-88), the two e4m3 P·V variants
 * (MI_ATTENTION_Q8_FP8, MI_ATTENTION_Q8_FP8_F32ACC, include/mossinfer/mossinfer.h:268-269). p_range / v_range <= 0 pick
 * the variant's defaults: 448 / 448 for int8_fp8_f32acc, 112 / 4.5 for int8_fp8. tcgen05 accumulates in fp32, so
 * int8_fp8 runs the same kernel with its own ranges: where the reference adds a 64-key tile in fp16 before flushing it
 * into fp32, this library adds in fp32 throughout (at least as close to exact attention); ranges are accepted and
 * refused by the reference's rule for fp16 accumulation all the same. The fp16 P·V variants (0, 1) are not built. */
#define B2_ATTENTION_Q8_FP8 2
#define B2_ATTENTION_Q8_FP8_F32ACC 3
typedef struct b2_attention_options {
  int variant;
  float p_range;
  float v_range;
} b2_attention_options;

/* A bf16 [tokens, heads, 128] view: element strides, head_dim contiguous (core/tensor.h:29-57 restricted to rank 3). */
typedef struct b2_view3 {
  void* data;
  int64_t tokens, heads;
  int64_t row_stride, head_stride;
} b2_view3;

/* attention_q8::QkNormRope (src/kernels/attention_q8/attention_q8.h:112-120). */
typedef struct b2_qk_norm_rope {
  const void* q_norm;
  const void* k_norm;
  const void* table;
  int64_t table_ld;
} b2_qk_norm_rope;

/* attention_q8::attention_q8_workspace_bytes (src/kernels/attention_q8/attention_q8.h:98). */
size_t b2_attention_q8_workspace_bytes(const b2_attention_options* o, int64_t total_q, int64_t total_k, int batch,
                                       int max_seqlen, int num_heads, int num_kv_heads);

/* attention_q8::attention_q8 (src/kernels/attention_q8/attention_q8.h:122). cu_seqlens_* device int32 [batch+1];
 * workspace 256-byte aligned; scale finite > 0; norm_rope NULL or the fused QK-norm + RoPE (then k is rewritten in
 * place and q's values are unspecified afterwards). Self-attention layouts only: num_heads == num_kv_heads. */
int b2_attention_q8(const b2_attention_options* o, const b2_view3* q, const b2_view3* k, const b2_view3* v,
                    const b2_view3* out, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                    int max_seqlen, float scale, void* workspace, size_t workspace_bytes, void* stream,
                    const b2_qk_norm_rope* norm_rope);

/* attention_q8::detail::preprocess (src/kernels/attention_q8/q8_preprocess.cu:389): the pre-pass of b2_attention_q8
 * alone. Fills the workspace (layout: b2_attention_q8_layout) with q_i8, k_i8, v8 and the scales; with norm_rope the
 * QK-norm + RoPE runs first and k is rewritten in place. Same argument rules as b2_attention_q8. */
int b2_attention_q8_preprocess(const b2_attention_options* o, const b2_view3* q, const b2_view3* k, const b2_view3* v,
                               const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch, int max_seqlen,
                               void* workspace, size_t workspace_bytes, void* stream, const b2_qk_norm_rope* norm_rope);

/* Test hook. b2_attention_q8 with the same arguments, which additionally stores the raw int32 Q8·K8^T accumulators that
 * the attention kernel's softmax threads read from tensor memory, for the 128 query rows of tile `tile_q` of
 * (sequence `seq`, head `head`): scores int32 [128, ld], row r = query tile_q * 128 + r of the sequence, column j = key j
 * (ld >= 64 * ceil(kv_len / 64)); rows at or past the sequence's end and columns at or past kv_len are unspecified.
 * The regular output is produced as well (by a second instantiation of the same kernel). These are the integer scores
 * of third_party/sageattention/csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:290-345; the reference has no such hook (its
 * tests compute them with a scalar kernel, tests/unit/test_attention_q8.cu). */
int b2_attention_q8_debug_scores(const b2_attention_options* o, const b2_view3* q, const b2_view3* k, const b2_view3* v,
                                 const b2_view3* out, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                                 int max_seqlen, float scale, void* workspace, size_t workspace_bytes, void* stream,
                                 const b2_qk_norm_rope* norm_rope, int seq, int head, int tile_q, int32_t* scores,
                                 int64_t ld);

/* The workspace layout of attention_q8.cu:47-73 as this library carves it (byte offsets from the 256-byte aligned base),
 * exposed so tests can compare the pre-pass outputs with the oracle: q_i8, k_i8 int8 and v8 e4m3 [total, heads, 128]
 * (V stays in its natural layout: the tensor core reads it as an MN-major operand, so there is no transposed, padded or
 * permuted copy); q_scale f32 [batch, heads, q_blocks]; k_scale f32 [batch, heads, k_blocks]; k_mean, v_scale, v_recp f32
 * [batch, heads, 128]; part_sum, part_amax f32 [batch, heads, chunks, 128]. */
typedef struct b2_attention_layout {
  size_t q_i8, k_i8, v8, q_scale, k_scale, k_mean, v_scale, v_recp, part_sum, part_amax, total;
  int64_t padded_k;
  int q_blocks, k_blocks, chunks;
} b2_attention_layout;
int b2_attention_q8_layout(const b2_attention_options* o, int64_t total_q, int64_t total_k, int batch, int max_seqlen,
                           int num_heads, int num_kv_heads, b2_attention_layout* out);

/* ---------------------------------------------------------------------------------------------------------------
 * The block and the step.
 * ------------------------------------------------------------------------------------------------------------- */

/* Int8Linear (src/models/moss_dit/dit_weights.h:75-79): w int8 [n,k] + scale f32 [n]. With tier == B2_TIER_W4A8 the
 * `w4` member describes the packed weight instead and `w` is unused. */
typedef struct b2_linear {
  const int8_t* w;
  const float* scale;
  const b2_w4_weight* w4;
} b2_linear;

/* BlockTensors restricted to the all-quantized block (src/models/moss_dit/dit_weights.h:106-136). */
typedef struct b2_block_weights {
  size_t struct_size;
  const void* norm1;   /* bf16 [D] */
  const void* norm2;   /* bf16 [D] */
  const void* q_norm;  /* bf16 [128] */
  const void* k_norm;  /* bf16 [128] */
  b2_linear qkv;       /* [3D, D] */
  b2_linear o;         /* [D, D] */
  b2_linear up_gate;   /* [2F, D], stored [hidden | gate] */
  b2_linear down;      /* [D, F] */
} b2_block_weights;

#define B2_TIER_INT8 0        /* W8A8 ConvRot, the High tier */
#define B2_TIER_W4A4_VIA_INT8 1 /* int4 weights + int4 activations in INT8 lanes (dit_block_quant.h:107-111) */
#define B2_TIER_W4A8 2        /* grouped 4-bit weights decoded to INT8, INT8 activations */

/* QuantBlockBuffers + BlockRun (src/models/moss_dit/dit_block_quant.h:77-105, dit_block_fused.h:120-165) for the
 * all-INT8 route, with an activation layout owned by this library (the reference's `big` layout constants do not fit
 * F = 12288). All buffers 256-byte aligned. */
typedef struct b2_block_buffers {
  size_t struct_size;
  void* x;            /* bf16 [L, D] residual stream, updated in place */
  const void* mod;    /* bf16 [6*D]: shift_a, scale_a, gate_a, shift_f, scale_f, gate_f */
  const void* rope;   /* bf16 [L, 128] */
  void* workspace;    /* b2_block_quant_workspace_bytes() */
  size_t workspace_bytes;
} b2_block_buffers;

typedef struct b2_block_run {
  size_t struct_size;
  int64_t tokens;            /* L: rows of x in this run */
  int D, F, heads;           /* 3072, 8192 | 12288, 24 */
  const int32_t* cu_seqlens; /* device int32 [batch+1] */
  int batch;
  int max_seqlen;
  int tier;                  /* B2_TIER_* */
  b2_attention_options attention;
  int fused_norm_rope;       /* -1 auto (in the pre-pass whenever the run has no slots or tap; same bits either way, and
                              * faster here at every size: the reference's 3072-row switch, dit_block_quant.cpp:32-35, is an
                              * sm_89 measurement), 0 separate kernel, 1 in the pre-pass */
  /* Reference keys and reference prefill (BlockRun of src/models/moss_dit/dit_block_fused.h:132-147). A caller built
   * against a header that ends at fused_norm_rope passes that struct_size and gets none of it. All zero / NULL: unused.
   * slot_rows > 0: attention reads keys and values from the region [slot A | the run's tokens | slot B], slot_rows rows
   * per slot; sequence i's keys are rows [k0 + cu_seqlens_k[i], k0 + cu_seqlens_k[i + 1]) of it, k0 <= k1 bound the rows
   * the run reads, and max_seqlen covers the key lengths. slot_kv[s]: bf16 [slot_rows, 2 D], k | v per token as
   * kv_tap wrote them (after QK-norm and RoPE), copied into slot s before attention; NULL for a slot the run does not
   * read. QK-norm + RoPE then run as their own kernel on the run's own rows. */
  int64_t slot_rows;
  const void* slot_kv[2];
  int64_t slot_kv_ld;          /* elements between rows of slot_kv; 0 = 2 D (contiguous, as kv_tap writes them) */
  const int32_t* cu_seqlens_k; /* device int32 [batch + 1] */
  int64_t k0, k1;
  /* kv_tap != NULL: after QK-norm and RoPE the run's k and v rows are copied there as bf16 [tokens, 2 D]
   * (tap_reference_kv, dit_block_fused.h:158); tap_only != 0: the block ends there, x untouched. */
  void* kv_tap;
  int tap_only;
} b2_block_run;

size_t b2_block_quant_workspace_bytes(const b2_block_run* run);

/* moss_dit::run_block_quant (src/models/moss_dit/dit_block_quant.h:145), all-quantized route with 8-bit attention. */
int b2_run_block_quant(const b2_block_weights* w, const b2_block_buffers* a, const b2_block_run* run, void* stream);

/* The block loop of MossDit::forward (src/models/moss_dit/moss_dit.cpp:1427-1460): blocks[i] applied in order to a->x.
 * Every block reads the one modulation vector a->mod, as in the reference, where the timestep embedding produces one
 * vector per step that all blocks share; a per-block modulation is not supported. */
int b2_dit_step(const b2_block_weights* blocks, int num_blocks, const b2_block_buffers* a, const b2_block_run* run,
                void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Sequence-parallel (Ulysses) block: one process per GPU, `size` ranks share every sequence. A rank owns a contiguous
 * 1/size slice of each sequence's tokens outside attention and heads/size heads of the full sequences inside it; two
 * exchanges per block over NCCL point-to-point calls on the caller's stream. The output equals the single-GPU block's
 * bit for bit. The reference engine is single-GPU (include/mossinfer/mossinfer.h:314): no counterpart there.
 * ------------------------------------------------------------------------------------------------------------- */

/* A communicator of one sequence-parallel group. Rank 0 of the group calls b2_sp_unique_id and hands the 128 bytes to
 * the other ranks by any means; then every rank of the group calls b2_sp_comm_create (a collective; the rank's device
 * must be current). size == 1 needs no id and no NCCL. NCCL is bound at run time (libnccl.so.2, preferring a copy the
 * process has already loaded); B2_ERR_NOT_SUPPORTED when none is found. */
typedef struct b2_sp_comm b2_sp_comm;
int b2_sp_unique_id(void* id, size_t id_bytes);
int b2_sp_comm_create(const void* id, size_t id_bytes, int size, int rank, b2_sp_comm** out);
int b2_sp_comm_destroy(b2_sp_comm* comm);
/* Measurement aid: with on != 0 every message of the group's exchanges becomes a device copy of the same size inside this
 * GPU (wrong results, same kernels and byte counts), so that "step with exchanges" minus "step with local copies" is the
 * communication time a step does not hide. */
int b2_sp_comm_local_exchange(b2_sp_comm* comm, int on);

/* local: the block run of this rank. tokens = sum over the sequences of seq_len / size (the rank's rows of x, sequence
 * by sequence); cu_seqlens (device int32 [batch + 1]), batch and max_seqlen describe the FULL sequences; tier must be
 * B2_TIER_INT8; heads / size must be even. seq_lens_host: host int32 [batch], the full lengths, each a multiple of size. */
typedef struct b2_sp_run {
  size_t struct_size;
  b2_block_run local;
  const int32_t* seq_lens_host;
} b2_sp_run;

size_t b2_block_quant_sp_workspace_bytes(const b2_sp_run* run, int size);

/* b2_run_block_quant on this rank's token shard. a->x: bf16 [local.tokens, D]; a->rope: the FULL table, bf16
 * [sum of seq_lens, 128] (QK-norm + RoPE run on the full sequences inside the attention pre-pass); a->workspace:
 * b2_block_quant_sp_workspace_bytes. w->qkv holds the QKV weight with its rows (and scales) reordered for the group:
 * [destination rank r][q | k | v][head r * heads/size + j][128 rows], so that the GEMM's column block r is what rank r
 * needs. Every rank of the group must make the same sequence of calls (the exchanges are collective). */
int b2_run_block_quant_sp(const b2_block_weights* w, const b2_block_buffers* a, const b2_sp_run* run, b2_sp_comm* comm,
                          void* stream);
int b2_dit_step_sp(const b2_block_weights* blocks, int num_blocks, const b2_block_buffers* a, const b2_sp_run* run,
                   b2_sp_comm* comm, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Guidance and the velocity update that follow the block loop of a denoising step (fp32 latents, device pointers).
 * Each op is one fp32 operation rounded once, in the reference's order: identical bits.
 * ------------------------------------------------------------------------------------------------------------- */

/* pipeline::cfg_combine (src/pipeline/samplers/sampler_driver.h:188; kernel sampler_kernels.cu:304):
 * out = uncond + g * (cond - uncond). */
int b2_cfg_combine(const float* cond, const float* uncond, float g, float* out, int64_t n, void* stream);
/* pipeline::slg_correct (sampler_driver.h:189; kernel sampler_kernels.cu:308): out = pred + scale * (cond - skipped). */
int b2_slg_correct(const float* pred, const float* cond, const float* skipped, float scale, float* out, int64_t n,
                   void* stream);
/* pipeline::euler_update (sampler_driver.h:202; kernel sampler_kernels.cu:209): x += h * v. */
int b2_euler_update(float* x, const float* v, float h, int64_t n, void* stream);
/* pipeline::ab2_update (sampler_driver.h:203; kernel sampler_kernels.cu:213): x += h * (a * v - b * v_prev). */
int b2_ab2_update(float* x, const float* v, const float* v_prev, float h, float a, float b, int64_t n, void* stream);

/* pipeline::guide_prediction in velocity space (src/pipeline/samplers/sampler_driver.cpp:565-577) followed by the
 * update, in ONE pass over the latent instead of up to four launches: v = cfg ? v_uncond + cfg_scale * (v_cond -
 * v_uncond) : v_cond; with slg, v = (cfg ? v : v_skip) + slg_scale * (v_cond - v_skip); v is stored to v_out when that
 * is non-NULL (the next Adams-Bashforth step's v_prev); update 1: x += h * v, update 2: x += h * (a * v - b * v_prev),
 * update 0: none (then v_out is required). Same bits as the reference's sequence of calls. */
typedef struct b2_guided_step {
  size_t struct_size;
  float* x;               /* [n] latent, updated in place */
  const float* v_cond;    /* [n] */
  const float* v_uncond;  /* [n], with cfg */
  const float* v_skip;    /* [n], with slg */
  const float* v_prev;    /* [n], update 2 */
  float* v_out;           /* [n] or NULL; must not alias v_prev */
  float cfg_scale, slg_scale, h, a, b;
  int cfg, slg, update;
  int64_t n;
} b2_guided_step;
int b2_guided_velocity_step(const b2_guided_step* step, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * The shell of MossDit::forward around the block loop (src/models/moss_dit/moss_dit.cpp:1181-1477).
 * ------------------------------------------------------------------------------------------------------------- */

/* moss_dit::latent_to_tokens (src/models/moss_dit/dit_kernels.h:16-19; dit_kernels.cu:137-158): f32 [channels, hw] ->
 * bf16 tokens [hw, channels] (row stride ld >= channels, so a wider token matrix can be filled at a column offset). */
int b2_latent_to_tokens(const float* latents, int channels, int64_t hw, void* tokens, int64_t ld, void* stream);
/* moss_dit::tokens_to_latent (dit_kernels.h:22): contiguous bf16 [hw, channels] -> f32 [channels, hw]. */
int b2_tokens_to_latent(const void* tokens, float* latents, int channels, int64_t hw, void* stream);
/* moss_dit::linear_fp32_row (dit_kernels.h:37; dit_kernels.cu:79-93): out[r] = bf16(dot(w[r, :], x) + bias[r]) with bf16
 * weights [n, k], fp32 x [k] and bias [n], the dot product in the reference kernel's order (one warp per row, 8 weights
 * per lane and step, one fma per weight, butterfly of adds): same bits. k % 8 == 0; w and x 16-byte aligned. */
int b2_linear_fp32_row(const void* w, const float* x, const float* bias, void* out, int n, int k, void* stream);
/* kernels::rms_norm_modulate_moss (src/kernels/basic/norm.h:29; bits of basic/norm.cu:67-128, the prologue of
 * b2_rms_norm_modulate_rotate_quantize without the quantiser): y = bf16(bf16(bf16(bf16(x * r) * w) * bf16(1 + scale)) +
 * shift), r from the mean of squares in torch's order for an [m, k] input. k % 256 == 0, k <= 4096. */
int b2_rms_norm_modulate(const void* x, int64_t ldx, const void* norm_weight, const void* mod_scale, const void* mod_shift,
                         void* y, int64_t ldy, int64_t m, int k, void* stream);

/* The official sinusoid of the timestep (moss_dit.cpp:979-985, distill.cpp:128-135): emb [256] = cos | sin of
 * timestep * 10000^(-i/128), computed in double and rounded to fp32. Host only. */
int b2_time_sinusoid(float timestep, float* emb);
/* TimeEmbeddingFp32 (src/models/moss_dit/distill.h): host fp32 weights of the timestep MLP. */
typedef struct b2_time_embedding {
  size_t struct_size;
  int64_t dim;      /* 3072 */
  const float* w0;  /* [dim, 256] */
  const float* b0;  /* [dim] */
  const float* w2;  /* [dim, dim] */
  const float* b2;  /* [dim] */
} b2_time_embedding;
/* moss_dit::time_vector_fp32 (distill.cpp:126-150): sinusoid -> linear -> SiLU -> linear on the host, each dot product
 * accumulated in double from the bias on. About 10 ms of one core for dim 3072; the rows are split over up to eight
 * host threads (each row summed in the same order, so no bit changes: 2-3 ms). Cache it per timestep as the reference
 * does (moss_dit.cpp:954-960). time: host [dim]. */
int b2_time_vector_fp32(const b2_time_embedding* te, float timestep, float* time);

/* kernels::silu (src/kernels/basic/elementwise.cu:92-100): out = bf16(x / (1 + expf(-x))), bf16 in and out, in place allowed. */
int b2_silu_bf16(const void* x, void* out, int64_t n, void* stream);

/* MossDit::time_modulation in its bf16 form (moss_dit.cpp:970-990, the path a model without a fp32 timestep MLP takes):
 * the sinusoid in double -> bf16 [256], linear -> SiLU -> linear (the timestep MLP), then the block and head modulation
 * linears, all bf16 with fp32 accumulation through cuBLASLt as in the reference (summation order the library's).
 * Weights and biases bf16 on the device (a bias may be NULL). mod: device bf16 [6 dim], head: [2 dim], for
 * b2_forward::mod / head. workspace: 256-byte aligned, b2_time_modulation_bf16_workspace_bytes(). */
typedef struct b2_time_mlp_bf16 {
  size_t struct_size;
  int64_t dim;                 /* 3072 */
  const void* in_w;            /* [dim, 256] */
  const void* in_bias;         /* [dim] */
  const void* out_w;           /* [dim, dim] */
  const void* out_bias;        /* [dim] */
  const void* block_mod_w;     /* [6 dim, dim] */
  const void* block_mod_bias;  /* [6 dim] */
  const void* head_mod_w;      /* [2 dim, dim] */
  const void* head_mod_bias;   /* [2 dim] */
} b2_time_mlp_bf16;
size_t b2_time_modulation_bf16_workspace_bytes(const b2_time_mlp_bf16* m);
int b2_time_modulation_bf16(const b2_time_mlp_bf16* m, float timestep, void* mod, void* head, void* workspace,
                            size_t workspace_bytes, void* stream);

/* kernels::Gemm::linear for the two bf16 linears of the shell (src/kernels/basic/gemm.h:20-63): out [m, n] = x [m, k] *
 * w [n, k]^T (+ bias [n]), bf16 in and out, fp32 accumulation, through cuBLASLt bound at run time (libcublasLt.so.12,
 * preferring a copy the process has already loaded; B2_ERR_NOT_SUPPORTED when none is found). As in the reference the
 * summation order is the library's. workspace: 256-byte aligned, b2_linear_bf16_workspace_bytes() is plenty. */
size_t b2_linear_bf16_workspace_bytes(void);
int b2_linear_bf16(const void* x, int64_t ldx, const void* w, const void* bias, void* out, int64_t ldo, int64_t m, int n,
                   int k, void* workspace, size_t workspace_bytes, void* stream);

/* The tensors of MossDit outside the blocks (src/models/moss_dit/moss_dit.h:395-440), device memory. */
typedef struct b2_dit_model {
  size_t struct_size;
  const b2_block_weights* blocks; /* host array [num_blocks] */
  int num_blocks;                 /* 42 */
  int D, F, heads, latent_channels; /* 3072, 8192 | 12288, 24, 128 */
  const void* block_mod_w;      /* bf16 [6 D, D]: the one modulation linear every block shares */
  const float* block_mod_bias;  /* f32 [6 D] */
  const void* head_mod_w;       /* bf16 [2 D, D] */
  const float* head_mod_bias;   /* f32 [2 D] */
  const void* video_w;          /* bf16 [D, 128] */
  const void* video_bias;       /* bf16 [D] or NULL */
  const void* final_norm;       /* bf16 [D] */
  const void* final_w;          /* bf16 [128, D] */
  const void* final_bias;       /* bf16 [128] or NULL */
  /* MossDit::InputExtension (moss_dit.h:215; set_input_extension, moss_dit.cpp:1118-1133): an embedder over the latent's 128
   * channels followed by ext_channels more, used instead of video_w / video_bias when ext_w is not NULL. */
  const void* ext_w;            /* bf16 [D, 128 + ext_channels] or NULL */
  const void* ext_bias;         /* bf16 [D] */
  int ext_channels;             /* > 0 and a multiple of 8 with ext_w */
} b2_dit_model;

/* MossDit::Row (src/models/moss_dit/moss_dit.h:99): one sequence of the forward = the video tokens of a latent followed by its text tokens. */
typedef struct b2_forward_row {
  const void* text;  /* device bf16 [text_len, D] */
  int64_t text_len;  /* >= 1 */
  uint64_t skip;     /* bit b set: the row skips block b (skip-layer guidance) */
  int latent;        /* which latent of the batch the row reads */
  float* out;        /* device f32 [128, height, width] */
} b2_forward_row;

typedef struct b2_forward {
  size_t struct_size;
  const float* latents;      /* device f32 [num_latents, 128, height, width] */
  int num_latents, height, width;
  const float* time_vector;  /* host f32 [D]: b2_time_vector_fp32 of the step's timestep */
  const b2_forward_row* rows;
  int num_rows;              /* 1..8 */
  int tier;                  /* B2_TIER_* */
  b2_attention_options attention;
  void* workspace;           /* b2_dit_forward_workspace_bytes(), 256-byte aligned */
  size_t workspace_bytes;
  /* With the model's input extension: device f32 [num_latents, ext_channels, height, width]. */
  const float* extra;
  /* Reference images (MossDit::set_references, moss_dit.h:383, moss_dit.cpp:1080-1090; RefKv, moss_dit.h:227): the cache b2_dit_prefill_references filled,
   * device bf16 [num_blocks, ref_tokens, 2 D]; NULL / 0 without. A forward with references takes one latent and at
   * most two rows; every sequence then attends to its own keys plus the reference keys in a slot next to it
   * (moss_dit.cpp:1283-1300). */
  const void* ref_kv;
  int64_t ref_tokens;
  /* The modulation vectors already computed (device bf16 [6 D] and [2 D]: b2_time_modulation_bf16, or a caller's own):
   * both or neither; with them time_vector is not read and the model's modulation linears are not needed. A caller
   * compiled against the struct without these two fields still works. */
  const void* mod;
  const void* head;
} b2_forward;

/* moss_dit::StepGraphs (src/models/moss_dit/dit_graph.h:14-66; runtime::GraphCache, src/runtime/graph_cache.h:20-58):
 * CUDA graphs of whole forwards, least recently used first out. b2_dit_forward_graphed enqueues what b2_dit_forward
 * would, through the graph of the call's key: replayed when cached (*replayed = 1), otherwise captured from one run of
 * the forward and launched. The key is everything but device memory contents and the time vector: the model structure
 * and its block table, grid, rows (text address and length, skip set, latent, output address), tier, attention
 * options, workspace, reference cache. The time vector is written to a buffer of the cache ahead of the graph, so
 * steps of one shape replay one graph. A key whose hash meets another cached key's runs eagerly (collisions), as does
 * a forward whose capture cannot be made (eager) or a cache of capacity 0. stream: not the default stream. Not
 * thread-safe (one cache per model and thread); the model, block table, rows' buffers and workspace of a cached
 * graph must stay where they are while it can be replayed (b2_dit_graphs_clear otherwise). */
typedef struct b2_dit_graphs b2_dit_graphs;
typedef struct b2_dit_graph_stats {
  uint64_t replays, captures, collisions, eager, evictions;
  size_t size; /* graphs cached now */
} b2_dit_graph_stats;
int b2_dit_graphs_create(size_t capacity, b2_dit_graphs** out);
int b2_dit_graphs_clear(b2_dit_graphs* graphs);
int b2_dit_graphs_destroy(b2_dit_graphs* graphs);
int b2_dit_graphs_stats(const b2_dit_graphs* graphs, b2_dit_graph_stats* stats);
int b2_dit_forward_graphed(b2_dit_graphs* graphs, const b2_dit_model* model, const b2_forward* forward, void* stream,
                           int* replayed);

/* MossDit::prefill_references (moss_dit.cpp:1479-1580): the reference latents (each device f32 [128, h_i, w_i], their
 * grids in heights / widths) run through every block as one sequence without text, under the modulation of
 * time_vector (the time vector of timestep 0 there), each with its reference RoPE table; block b's k | v rows after
 * QK-norm and RoPE land in kv_out[b] (device bf16 [num_blocks, sum h_i w_i, 2 D]). With the model's input extension
 * the extra channels are zero. workspace: b2_dit_prefill_workspace_bytes(). */
typedef struct b2_prefill {
  size_t struct_size;
  const float* const* latents; /* host array of num_refs device pointers */
  const int* heights;
  const int* widths;
  int num_refs;
  const float* time_vector;    /* host f32 [D] */
  void* kv_out;
  int tier;
  b2_attention_options attention;
  void* workspace;
  size_t workspace_bytes;
} b2_prefill;
size_t b2_dit_prefill_workspace_bytes(const b2_dit_model* model, const b2_prefill* prefill);
int b2_dit_prefill_references(const b2_dit_model* model, const b2_prefill* prefill, void* stream);

size_t b2_dit_forward_workspace_bytes(const b2_dit_model* model, const b2_forward* forward);
/* MossDit::forward (moss_dit.cpp:1181-1477) for the all-quantized block path, without reference slots, input extension,
 * step cache, LoRA or streamed weights: modulation vectors from the time vector, video embedding once per latent,
 * per-row RoPE tables, [video | text] rows, for every block the runs of contiguous rows that do not skip it as one varlen
 * batch each, then final norm + head modulation, head linear and the transpose back to [128, h, w] per row. Small host
 * arrays travel as kernel parameters: the call does not synchronise and needs no pinned memory. */
int b2_dit_forward(const b2_dit_model* model, const b2_forward* forward, void* stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Weight ingestion: a ComfyUI-layout safetensors file of the quantized MOSS-Image DiT -> device tensors.
 * What quant::read_model + to_model_index + the block upload do in the reference for this path
 * (src/weights/quant/quant_model.h:1-45, quant_model.cpp:205-285, src/models/moss_dit/dit_weights.cpp:194-300).
 * ------------------------------------------------------------------------------------------------------------- */

typedef struct b2_dit_file b2_dit_file;
typedef struct b2_dit_file_info {
  size_t struct_size;
  int num_blocks;
  int F;                  /* FFN width read from layers.0.proj.ffn_down */
  int tier;               /* B2_TIER_*: the one tier of every block linear in the file */
  int has_shell;          /* the tensors outside the blocks are there: b2_dit_file_model() can run b2_dit_forward */
  int has_time_embedding; /* time_embedding.0 / .2 are there: b2_dit_file_time_embedding() is not NULL */
  size_t device_bytes;
  int stored_tier;        /* the tier of the file's bytes; differs from `tier` after b2_dit_file_open_expanded */
} b2_dit_file_info;

/* Reads the header, checks every tensor the model needs (names, dtypes, shapes, per-module comfy_quant configs or the
 * legacy _quantization_metadata key, scales finite and > 0) before any tensor byte is read, then copies the tensors into
 * one device allocation on the current device: int8_tensorwise + convrot (group 256) as stored (a scalar scale expanded
 * to rows), convrot_w4a4 and asym_w4a8_int8 packed as stored for the tiers that decode them on the device. q / k / v
 * stored apart are stacked into the fused QKV matrix. Everything else in the file (text embedder, other models'
 * tensors) is ignored. Errors: B2_ERR_INVALID_ARGUMENT with a message that names the file and the tensor. */
int b2_dit_file_open(const char* path, b2_dit_file** out);
/* The same, for a part with memory to spare: grouped 4-bit linears (asym_w4a8_int8) are expanded to the INT8 grid
 * once, on the device, behind their upload (quant::decode_grouped_int8, a NaN or negative group scale raising the
 * library's b2_w4_invalid_scales word), and the blocks run the INT8 tier with s_channel as the weight scale
 * (info.tier == B2_TIER_INT8, info.stored_tier == B2_TIER_W4A8). The W4A8 tier does that expansion into a scratch on
 * every step, so the outputs are bit-identical and the per-step decode is gone; the price is n * k more bytes per
 * linear (a 42-block model: 6.3 GB more). The reference keeps 4-bit weights packed because its GPUs have 16-24 GB
 * (src/models/moss_dit/dit_weights.h:106-136). INT8 files, and convrot_w4a4 files (whose tier also quantises the
 * activations to 4 bits), load as with b2_dit_file_open. */
int b2_dit_file_open_expanded(const char* path, b2_dit_file** out);
int b2_dit_file_get_info(const b2_dit_file* file, b2_dit_file_info* info);
/* The loaded model; blocks[] always, the shell tensors when has_shell. Valid until b2_dit_file_close. */
const b2_dit_model* b2_dit_file_model(const b2_dit_file* file);
/* Host fp32 copy of the timestep MLP for b2_time_vector_fp32, or NULL. The file's bf16 values are exact in fp32; the
 * reference runs this MLP in bf16 through cuBLASLt (moss_dit.cpp:970-990) unless a fp32 replacement is installed
 * (distill.h), so results agree with its fp32 form, not bit for bit with its bf16 form. */
const b2_time_embedding* b2_dit_file_time_embedding(const b2_dit_file* file);
/* The same MLP and the two modulation linears as bf16 device tensors for b2_time_modulation_bf16 (the reference's default
 * form, moss_dit.cpp:970-990), or NULL when the file lacks the shell or the time embedding. */
const b2_time_mlp_bf16* b2_dit_file_time_mlp_bf16(const b2_dit_file* file);
void b2_dit_file_close(b2_dit_file* file);

/* Every mbarrier wait inside the tensor-core kernels is bounded (200 ms); a CTA whose wait expired raises a device word,
 * drains and returns instead of hanging. This reads the two words (GEMM, attention): 0 = no wait ever expired on this device.
 * Synchronises the device; for tests and post-mortems, not for the hot path. No counterpart in the reference (its
 * kernels have no device-side waits). */
int b2_kernel_status(int* gemm, int* attention);
/* Zeroes both words (after a post-mortem). Synchronises the device. */
int b2_kernel_status_clear(void);
/* Test hook of the bounded waits. wait_limit_ns != 0 sets how long a wait inside the GEMM kernel may last on the current
 * device (default 200 ms; the attention kernel's limit is fixed at 200 ms). skip_gemm_stage != 0 makes the TMA warp of
 * every GEMM CTA leave out the loads of the last K block of its first tile: that stage's barrier then never completes,
 * the waits run out after the limit, every CTA raises the status word, drains, frees its tensor memory and returns (the
 * output of that launch is garbage, nothing faults or hangs). Call again with (0-or-limit, 0) to switch it off.
 * No counterpart in the reference. */
int b2_debug_bounded_wait(uint64_t wait_limit_ns, int skip_gemm_stage);

#ifdef __cplusplus
}
#endif
#endif /* OWOINFER_B200_H_ */
