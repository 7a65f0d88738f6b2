// Host-side sequencing of one all-quantized MOSS DiT block and of the block loop of a denoising step. One stream, no
// allocation, no host synchronisation: every kernel is queued in order on the caller's stream (graph-capturable).
//
//   qkv      rms_norm_modulate_rotate_quantize(x, norm1, scale_a, shift_a) -> int8_gemm            -> qkv [L, 3D]
//   attn     attention_q8(q, k, v views of qkv; QK-norm + RoPE fused into its pre-pass or run first) -> attn [L, D]
//   o        rotate_quantize(attn) -> int8_gemm_gated_residual(gate_a)                             -> x (in place)
//   up_gate  rms_norm_modulate_rotate_quantize(x, norm2, scale_f, shift_f) -> int8_gemm_situ_glu   -> ffn [L, F]
//   down     rotate_quantize(ffn) -> int8_gemm_gated_residual(gate_f)                              -> x (in place)
// Reference: src/models/moss_dit/dit_block_quant.cpp:196-608 (all-INT8 branch lines 365-368, 432-444, 471-480, 538-542,
// 590-599; W4A4-through-INT8 branch lines 352-355, 465-466, 520-525, 584-585).
#include <algorithm>
#include <cmath>
#include <string>

#include "common.cuh"

namespace b2 {
namespace {

constexpr std::size_t kAlign = 256;
constexpr int kFusedNormRopeMinTokens = 3072;  // src/models/moss_dit/dit_block_quant.cpp:32-35

std::size_t align_up(std::size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

struct Workspace {
  std::size_t xq, x4, scale, qkv, attn, ffn, w_unpack, attn_ws, total;
  std::size_t attn_ws_bytes;
};

Workspace carve(const b2_block_run* run) {
  Workspace w{};
  const std::size_t L = static_cast<std::size_t>(run->tokens), D = static_cast<std::size_t>(run->D), F = static_cast<std::size_t>(run->F);
  const std::size_t kmax = std::max(D, F);
  std::size_t at = 0;
  const auto take = [&](std::size_t bytes) {
    const std::size_t off = at;
    at += align_up(bytes);
    return off;
  };
  w.xq = take(L * kmax);
  w.x4 = take(run->tier == B2_TIER_W4A4_VIA_INT8 ? L * kmax / 2 : 0);
  w.scale = take(L * 4);
  w.qkv = take(L * 3 * D * 2);
  w.attn = take(L * D * 2);
  w.ffn = take(L * F * 2);
  w.w_unpack = take(run->tier == B2_TIER_INT8 ? 0 : std::max({3 * D * D, 2 * F * D, D * F}));
  w.attn_ws_bytes = b2_attention_q8_workspace_bytes(&run->attention, run->tokens, run->tokens, run->batch, run->max_seqlen,
                                                    run->heads, run->heads);
  w.attn_ws = take(w.attn_ws_bytes);
  w.total = at;
  return w;
}

int check_run(const char* op, const b2_block_run* run) {
  if (run == nullptr || run->struct_size < sizeof(b2_block_run)) return fail_invalid(op, "run is null or from an older header");
  if (run->tokens < 0 || run->D <= 0 || run->F <= 0 || run->heads <= 0 || run->D != run->heads * 128) {
    return fail_invalid(op, "needs D == heads * 128, F > 0, tokens >= 0");
  }
  if (run->D % 256 != 0 || run->F % 256 != 0) return fail_invalid(op, "D and F must be multiples of 256 (rotation groups)");
  if (run->tier < B2_TIER_INT8 || run->tier > B2_TIER_W4A8) return fail_invalid(op, "unknown tier");
  if (run->batch < 1 || run->max_seqlen < 1 || run->cu_seqlens == nullptr) return fail_invalid(op, "needs cu_seqlens, batch >= 1, max_seqlen >= 1");
  return B2_OK;
}

// One linear site: operands for the INT8 GEMM from the site's weight under the run's tier.
int site_operands(const char* op, const b2_linear& lin, int tier, std::int8_t* w_unpack, std::int64_t n, std::int64_t k,
                  cudaStream_t stream, const std::int8_t** w, const float** ws) {
  if (tier == B2_TIER_INT8) {
    if (lin.w == nullptr || lin.scale == nullptr) return fail_invalid(op, "missing INT8 weight");
    *w = lin.w, *ws = lin.scale;
    return B2_OK;
  }
  if (tier == B2_TIER_W4A4_VIA_INT8) {
    if (lin.w == nullptr || lin.scale == nullptr) return fail_invalid(op, "missing INT4 weight");
    if (const int rc = b2_unpack_int4(lin.w, k / 2, w_unpack, k, n, k, stream)) return rc;
    *w = w_unpack, *ws = lin.scale;
    return B2_OK;
  }
  return fail_status(B2_ERR_INTERNAL, op, "unexpected tier");
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" {

size_t b2_block_quant_workspace_bytes(const b2_block_run* run) {
  if (check_run("block_quant_workspace_bytes", run) != B2_OK) return 0;
  return carve(run).total;
}

int b2_run_block_quant(const b2_block_weights* w, const b2_block_buffers* a, const b2_block_run* run, void* stream) {
  constexpr const char* op = "run_block_quant";
  if (const int rc = check_run(op, run)) return rc;
  if (w == nullptr || a == nullptr || w->struct_size < sizeof(b2_block_weights) || a->struct_size < sizeof(b2_block_buffers)) {
    return fail_invalid(op, "weights or buffers are null or from an older header");
  }
  const Workspace ws = carve(run);
  // Mismatched buffers are a programming error: refuse before any launch.
  if (a->x == nullptr || a->mod == nullptr || a->rope == nullptr || a->workspace == nullptr || a->workspace_bytes < ws.total) {
    return fail_invalid(op, "buffers do not match the run: workspace " + std::to_string(a->workspace_bytes) + " of " +
                                std::to_string(ws.total) + " bytes");
  }
  for (const void* p : {static_cast<const void*>(a->x), a->mod, a->rope, static_cast<const void*>(a->workspace)}) {
    if (!aligned_to(p, kAlign)) return fail_invalid(op, "operands must be 256-byte aligned");
  }
  if (w->norm1 == nullptr || w->norm2 == nullptr || w->q_norm == nullptr || w->k_norm == nullptr) return fail_invalid(op, "missing norm weights");
  const std::int64_t L = run->tokens, D = run->D, F = run->F;
  if (L == 0) return B2_OK;
  cudaStream_t st = as_stream(stream);
  auto* base = static_cast<std::uint8_t*>(a->workspace);
  auto* xq = reinterpret_cast<std::int8_t*>(base + ws.xq);
  auto* x4 = base + ws.x4;
  auto* scale = reinterpret_cast<float*>(base + ws.scale);
  auto* qkv = reinterpret_cast<__nv_bfloat16*>(base + ws.qkv);
  auto* attn = reinterpret_cast<__nv_bfloat16*>(base + ws.attn);
  auto* ffn = reinterpret_cast<__nv_bfloat16*>(base + ws.ffn);
  auto* w_unpack = reinterpret_cast<std::int8_t*>(base + ws.w_unpack);
  const auto* mod = static_cast<const __nv_bfloat16*>(a->mod);
  const bool a4 = run->tier == B2_TIER_W4A4_VIA_INT8;

  // Quantised GEMM input of a site: INT8 activations, or INT4 activations widened to INT8 lanes.
  const auto quant_norm = [&](const void* norm_w, const __nv_bfloat16* sc, const __nv_bfloat16* sh) -> int {
    if (!a4) return b2_rms_norm_modulate_rotate_quantize(a->x, D, norm_w, sc, sh, xq, D, scale, L, static_cast<int>(D), st, nullptr, 0);
    if (const int rc = b2_rms_norm_modulate_convrot_quantize_int4(a->x, D, norm_w, sc, sh, x4, D / 2, scale, L, static_cast<int>(D), st)) return rc;
    return b2_unpack_int4(x4, D / 2, xq, D, L, D, st);
  };
  const auto quant_plain = [&](const __nv_bfloat16* in, std::int64_t k) -> int {
    if (!a4) return b2_rotate_quantize(in, k, xq, k, scale, L, static_cast<int>(k), st);
    if (const int rc = b2_convrot_quantize_int4(in, k, x4, k / 2, scale, L, static_cast<int>(k), st)) return rc;
    return b2_unpack_int4(x4, k / 2, xq, k, L, k, st);
  };
  // One linear site with its epilogue (0 plain, 1 gated residual with gate `aux`, 2 SiTU-GLU) under the run's tier. The
  // grouped 4-bit tier goes through b2_w4a8_gemm, which decodes inside the GEMM where the weight's format allows and
  // through the scratch otherwise.
  const auto site = [&](const b2_linear& lin, std::int64_t n, std::int64_t k, int epilogue, const void* aux, void* out,
                        std::int64_t ldo) -> int {
    if (run->tier == B2_TIER_W4A8) {
      if (lin.w4 == nullptr) return fail_invalid(op, "missing grouped 4-bit weight");
      return b2_w4a8_gemm(xq, k, scale, lin.w4, L, n, k, epilogue, aux, out, ldo, w_unpack, st);
    }
    const std::int8_t* wq = nullptr;
    const float* wsc = nullptr;
    if (const int rc = site_operands(op, lin, run->tier, w_unpack, n, k, st, &wq, &wsc)) return rc;
    const b2_int8_operands o{xq, k, scale, wq, wsc, L, n, k};
    if (epilogue == 0) return b2_int8_gemm(&o, aux, out, ldo, st, B2_TILE_AUTO);
    if (epilogue == 1) return b2_int8_gemm_gated_residual(&o, nullptr, aux, out, ldo, st, B2_TILE_AUTO);
    return b2_int8_gemm_situ_glu(&o, out, ldo, st, B2_TILE_AUTO);
  };

  // QKV projection.
  if (const int rc = quant_norm(w->norm1, mod + 1 * D, mod + 0 * D)) return rc;
  if (const int rc = site(w->qkv, 3 * D, D, 0, nullptr, qkv, 3 * D)) return rc;

  // Attention. QK-norm + RoPE inside the pre-pass from 3072 tokens on (same bits either way).
  const bool fused = run->fused_norm_rope < 0 ? L >= kFusedNormRopeMinTokens : run->fused_norm_rope != 0;
  if (!fused) {
    if (const int rc = b2_qk_norm_rope_moss(qkv, 3 * D, L, run->heads, w->q_norm, w->k_norm, a->rope, 128, st)) return rc;
  }
  const b2_view3 vq{qkv, L, run->heads, 3 * D, 128}, vk{qkv + D, L, run->heads, 3 * D, 128}, vv{qkv + 2 * D, L, run->heads, 3 * D, 128};
  const b2_view3 vo{attn, L, run->heads, D, 128};
  const b2_qk_norm_rope nr{w->q_norm, w->k_norm, a->rope, 128};
  b2_attention_options ao = run->attention;
  if (ao.variant == 0) ao.variant = B2_ATTENTION_Q8_FP8_F32ACC;
  const float sm_scale = static_cast<float>(1.0 / std::sqrt(128.0));
  if (const int rc = b2_attention_q8(&ao, &vq, &vk, &vv, &vo, run->cu_seqlens, run->cu_seqlens, run->batch, run->max_seqlen,
                                     sm_scale, base + ws.attn_ws, ws.attn_ws_bytes, st, fused ? &nr : nullptr)) {
    return rc;
  }

  // x += o(attn) * gate_a.
  if (const int rc = quant_plain(attn, D)) return rc;
  if (const int rc = site(w->o, D, D, 1, mod + 2 * D, a->x, D)) return rc;

  // ffn = situ_glu(up_gate(rms_norm_modulate(x))).
  if (const int rc = quant_norm(w->norm2, mod + 4 * D, mod + 3 * D)) return rc;
  if (const int rc = site(w->up_gate, 2 * F, D, 2, nullptr, ffn, F)) return rc;

  // x += down(ffn) * gate_f.
  if (const int rc = quant_plain(ffn, F)) return rc;
  return site(w->down, D, F, 1, mod + 5 * D, a->x, D);
}

int b2_kernel_status(int* gemm, int* attention) {
  int g = 0, t = 0;
  if (const int rc = gemm_status_word(&g)) return rc;
  if (const int rc = attn_status_word(&t)) return rc;
  if (gemm != nullptr) *gemm = g;
  if (attention != nullptr) *attention = t;
  return B2_OK;
}

int b2_kernel_status_clear(void) {
  if (const int rc = gemm_status_clear()) return rc;
  return attn_status_clear();
}

int b2_debug_bounded_wait(uint64_t wait_limit_ns, int skip_gemm_stage) {
  return gemm_debug_set(wait_limit_ns, skip_gemm_stage != 0 ? 1 : 0);
}

int b2_dit_step(const b2_block_weights* blocks, int num_blocks, const b2_block_buffers* a, const b2_block_run* run,
                void* stream) {
  if (blocks == nullptr || num_blocks < 0) return fail_invalid("dit_step", "null blocks");
  for (int i = 0; i < num_blocks; ++i) {
    if (const int rc = b2_run_block_quant(&blocks[i], a, run, stream)) return rc;
  }
  return B2_OK;
}

}  // extern "C"
