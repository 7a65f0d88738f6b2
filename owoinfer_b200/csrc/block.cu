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
#include <cstddef>
#include <cstring>
#include <string>

#include "common.cuh"

namespace b2 {
namespace {

constexpr std::size_t kAlign = 256;

std::size_t align_up(std::size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

struct Workspace {
  std::size_t xq, x4, scale, qkv, attn, ffn, w_unpack, attn_ws, total;
  std::size_t attn_ws_bytes;
};

// The run as this file reads it: a caller's struct may end before the reference-key fields (an older header).
constexpr std::size_t kRunCoreBytes = offsetof(b2_block_run, slot_rows);
b2_block_run whole_run(const b2_block_run* run) {
  b2_block_run r{};
  std::memcpy(&r, run, std::min(run->struct_size, sizeof r));
  return r;
}

Workspace carve(const b2_block_run* run_in) {
  Workspace w{};
  const b2_block_run whole = whole_run(run_in);
  const b2_block_run* run = &whole;
  const std::size_t L = static_cast<std::size_t>(run->tokens), D = static_cast<std::size_t>(run->D), F = static_cast<std::size_t>(run->F);
  const std::size_t region = L + 2 * static_cast<std::size_t>(run->slot_rows);  // [slot A | tokens | slot B]
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
  w.qkv = take(region * 3 * D * 2);
  w.attn = take(L * D * 2);
  w.ffn = take(L * F * 2);
  w.w_unpack = take(run->tier == B2_TIER_INT8 ? 0 : std::max({3 * D * D, 2 * F * D, D * F}));
  w.attn_ws_bytes = b2_attention_q8_workspace_bytes(&run->attention, run->tokens, static_cast<std::int64_t>(region), run->batch,
                                                    run->max_seqlen, run->heads, run->heads);
  w.attn_ws = take(w.attn_ws_bytes);
  w.total = at;
  return w;
}

int check_run(const char* op, const b2_block_run* run) {
  if (run == nullptr || run->struct_size < kRunCoreBytes) return fail_invalid(op, "run is null or from an older header");
  if (run->tokens < 0 || run->D <= 0 || run->F <= 0 || run->heads <= 0 || run->D != run->heads * 128) {
    return fail_invalid(op, "needs D == heads * 128, F > 0, tokens >= 0");
  }
  if (run->D % 256 != 0 || run->F % 256 != 0) return fail_invalid(op, "D and F must be multiples of 256 (rotation groups)");
  if (run->tier < B2_TIER_INT8 || run->tier > B2_TIER_W4A8) return fail_invalid(op, "unknown tier");
  if (run->batch < 1 || run->max_seqlen < 1 || run->cu_seqlens == nullptr) return fail_invalid(op, "needs cu_seqlens, batch >= 1, max_seqlen >= 1");
  const b2_block_run r = whole_run(run);
  if (r.slot_rows < 0 || r.slot_kv_ld < 0 || (r.slot_kv_ld > 0 && r.slot_kv_ld < 2 * r.D)) return fail_invalid(op, "negative slot_rows, or slot_kv_ld below 2 D");
  if (r.slot_rows > 0) {
    if (r.cu_seqlens_k == nullptr || r.k0 < 0 || r.k1 < r.k0 || r.k1 > r.tokens + 2 * r.slot_rows) {
      return fail_invalid(op, "reference slots need cu_seqlens_k and 0 <= k0 <= k1 <= tokens + 2 * slot_rows");
    }
    if ((r.k0 < r.slot_rows && r.slot_kv[0] == nullptr) || (r.k1 > r.slot_rows + r.tokens && r.slot_kv[1] == nullptr)) {
      return fail_invalid(op, "the key rows reach into a slot that has no slot_kv");
    }
  }
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

int b2_run_block_quant(const b2_block_weights* w, const b2_block_buffers* a, const b2_block_run* run_in, void* stream) {
  constexpr const char* op = "run_block_quant";
  if (const int rc = check_run(op, run_in)) return rc;
  const b2_block_run whole = whole_run(run_in);
  const b2_block_run* run = &whole;
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

  // QKV projection, into the rows after slot A when the run reads reference keys.
  const std::int64_t slot = run->slot_rows;
  __nv_bfloat16* own = qkv + slot * 3 * D;
  if (const int rc = quant_norm(w->norm1, mod + 1 * D, mod + 0 * D)) return rc;
  if (const int rc = site(w->qkv, 3 * D, D, 0, nullptr, own, 3 * D)) return rc;

  // Attention. QK-norm + RoPE inside the pre-pass from 3072 tokens on (same bits either way); as their own kernel when
  // the keys are not the run's own rows alone or the rows are tapped after them.
  const bool plain = slot == 0 && run->kv_tap == nullptr;
  // Automatic = the pre-pass at every size: the two routes give the same bits, and on this part the fused one is the faster
  // from 2 x 320 tokens (167 against 173 us per block) to 2 x 8192 (the reference's sm_89 measurements put the switch at
  // 3072 rows, dit_block_quant.cpp:32-35).
  const bool fused = plain && (run->fused_norm_rope < 0 || run->fused_norm_rope != 0);
  if (!fused) {
    if (const int rc = b2_qk_norm_rope_moss(own, 3 * D, L, run->heads, w->q_norm, w->k_norm, a->rope, 128, st)) return rc;
  }
  const std::size_t kv_bytes = static_cast<std::size_t>(2 * D) * sizeof(__nv_bfloat16), row_bytes = static_cast<std::size_t>(3 * D) * sizeof(__nv_bfloat16);
  if (run->kv_tap != nullptr) {
    // tap_reference_kv: the k | v columns of every row, contiguous.
    if (const cudaError_t e = cudaMemcpy2DAsync(run->kv_tap, kv_bytes, own + D, row_bytes, kv_bytes, static_cast<std::size_t>(L), cudaMemcpyDeviceToDevice, st); e != cudaSuccess) {
      return fail_cuda(op, e);
    }
    if (run->tap_only != 0) return B2_OK;
  }
  std::int64_t k0 = 0, k_rows = L;
  const std::int32_t* cu_k = run->cu_seqlens;
  if (slot > 0) {
    // The cached keys and values into the k | v columns of the slots the key rows reach (moss_dit.cpp:1441-1452).
    for (int s2 = 0; s2 < 2; ++s2) {
      const bool read = s2 == 0 ? run->k0 < slot : run->k1 > slot + L;
      if (!read) continue;
      __nv_bfloat16* dst = qkv + (s2 == 0 ? 0 : slot + L) * 3 * D + D;
      const std::size_t src_pitch = run->slot_kv_ld > 0 ? static_cast<std::size_t>(run->slot_kv_ld) * sizeof(__nv_bfloat16) : kv_bytes;
      if (const cudaError_t e = cudaMemcpy2DAsync(dst, row_bytes, run->slot_kv[s2], src_pitch, kv_bytes, static_cast<std::size_t>(slot), cudaMemcpyDeviceToDevice, st); e != cudaSuccess) {
        return fail_cuda(op, e);
      }
    }
    k0 = run->k0, k_rows = run->k1 - run->k0, cu_k = run->cu_seqlens_k;
  }
  const b2_view3 vq{own, L, run->heads, 3 * D, 128};
  const b2_view3 vk{qkv + k0 * 3 * D + D, k_rows, run->heads, 3 * D, 128}, vv{qkv + k0 * 3 * D + 2 * D, k_rows, run->heads, 3 * D, 128};
  const b2_view3 vo{attn, L, run->heads, D, 128};
  const b2_qk_norm_rope nr{w->q_norm, w->k_norm, a->rope, 128};
  b2_attention_options ao = run->attention;
  if (ao.variant == 0) ao.variant = B2_ATTENTION_Q8_FP8_F32ACC;
  const float sm_scale = static_cast<float>(1.0 / std::sqrt(128.0));
  if (const int rc = b2_attention_q8(&ao, &vq, &vk, &vv, &vo, run->cu_seqlens, cu_k, run->batch, run->max_seqlen, sm_scale,
                                     base + ws.attn_ws, ws.attn_ws_bytes, st, fused ? &nr : nullptr)) {
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
