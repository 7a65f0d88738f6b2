// Header-only C++ adapter that puts libowoinfer_b200 behind the reference engine's block interface: include it from a
// translation unit of the reference (its src/ directory on the include path), next to owoinfer_b200.h.
//
//   mi::moss_dit::b200_can_run(...)          true when the block is one this library runs
//   mi::moss_dit::run_block_quant_b200(...)  moss_dit::run_block_quant's parameters, in its order
//                                            (src/models/moss_dit/dit_block_quant.h:145-146), plus the workspace
//
// It converts the reference's non-owning tensors (src/core/tensor.h:29-57) into the C ABI's plain structs and maps the
// status codes back onto the reference's exceptions: invalid argument -> std::invalid_argument (before any launch, as
// dit_block_quant.h:135-137 promises), CUDA failure -> mi::CudaError (src/core/cuda_check.h:14-16).
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "core/cuda_check.h"
#include "models/moss_dit/dit_block_quant.h"
#include "owoinfer_b200.h"

namespace mi::moss_dit {

inline void b200_check(int status) {
  if (status == B2_OK) return;
  const std::string what = b2_last_error_message();
  if (status == B2_ERR_INVALID_ARGUMENT) throw std::invalid_argument(what);
  if (status == B2_ERR_CUDA) throw mi::CudaError(what);
  if (status == B2_ERR_NOT_SUPPORTED) throw std::logic_error(what);
  throw std::runtime_error(what);
}

// The blocks this library runs: all four linears INT8 ConvRot and fused (dit_weights.h:106-111), attention in one of the
// e4m3 P.V variants (q8_fp8, the High tier's default, with its 112 / 4.5 ranges and fp32 in place of its fp16 tile
// accumulation; q8_fp8_f32acc), no LoRA side branch; reference slots and the K/V tap included. Everything else stays on
// the reference's own path.
inline bool b200_can_run(const BlockTensors& w, const QuantBlockBuffers& a, const BlockRun& /*run*/, AttentionMode attention) {
  return !w.qkv_split && !w.qkv8.empty() && !w.o8.empty() && !w.up_gate8.empty() && !w.down8.empty() && !w.int4() &&
         !w.nvfp4() && (attention == AttentionMode::kQ8Fp8F32Acc || attention == AttentionMode::kQ8Fp8) && a.lora == nullptr;
}

// The b2_block_run of a run of the reference: D and F from the weights' shapes, heads = D / 128. With reference slots the
// cached k | v rows are read where MossDit::forward put them, in the k | v columns of the slot rows of `big` (slot A
// before all tokens, slot B after them: dit_block_fused.h:136-141); this library copies them next to its own QKV rows.
inline b2_block_run b200_block_run(const BlockTensors& w, const BlockRun& run, const QuantBlockBuffers* a = nullptr) {
  b2_block_run br{};
  br.struct_size = sizeof(b2_block_run);
  br.tokens = run.t1 - run.t0;
  br.D = static_cast<int>(w.o8.w.dim(0));
  br.F = static_cast<int>(w.down8.w.dim(1));
  br.heads = br.D / 128;
  br.cu_seqlens = static_cast<const std::int32_t*>(run.cu_seqlens.data);
  br.batch = static_cast<int>(run.cu_seqlens.numel()) - 1;
  br.max_seqlen = run.max_seqlen;
  br.tier = B2_TIER_INT8;
  br.attention = b2_attention_options{B2_ATTENTION_Q8_FP8_F32ACC, 0.f, 0.f};
  br.fused_norm_rope = -1;
  br.kv_tap = run.kv_tap;
  br.tap_only = run.tap_only ? 1 : 0;
  if (run.slot_rows > 0) {
    br.slot_rows = run.slot_rows;
    br.cu_seqlens_k = static_cast<const std::int32_t*>(run.cu_seqlens_k.data);
    br.k0 = run.k0 - run.t0;  // rows of [slot A | the run's tokens | slot B]
    br.k1 = run.k1 - run.t0;
    if (a != nullptr) {
      const std::int64_t qkv_dim = 3 * static_cast<std::int64_t>(br.D), total = a->f.x.dim(0);
      const auto* big = static_cast<const std::uint16_t*>(a->f.big.data);
      br.slot_kv[0] = big + br.D;
      br.slot_kv[1] = big + (run.slot_rows + total) * qkv_dim + br.D;
      br.slot_kv_ld = qkv_dim;
    }
  }
  return br;
}

// Bytes of the workspace run_block_quant_b200 needs for this run (size it once for the largest run; 256-byte aligned,
// e.g. from the reference's device arena).
inline std::size_t b200_workspace_bytes(const BlockTensors& w, const BlockRun& run) {
  const b2_block_run br = b200_block_run(w, run);
  return b2_block_quant_workspace_bytes(&br);
}

// moss_dit::run_block_quant for a block b200_can_run() accepts. `qkv_gemm` and `route` belong to the bf16 pairs of the
// reference's mixed blocks and are not used here; `block` only names LoRA sites there. The activations of the block
// live in `workspace` (this library's own layout), not in a.f.big.
inline void run_block_quant_b200(const BlockTensors& w, const QuantBlockBuffers& a, const BlockRun& run,
                                 const QkvGemm& /*qkv_gemm*/, const FusedRouteSnapshot& /*route*/, AttentionMode attention,
                                 cudaStream_t stream, int /*block*/, void* workspace, std::size_t workspace_bytes) {
  if (!b200_can_run(w, a, run, attention)) {
    throw std::invalid_argument("run_block_quant_b200: not an all-INT8 block with q8_fp8 or q8_fp8_f32acc attention, or it uses LoRA");
  }
  const auto lin = [](const Int8Linear& l) {
    return b2_linear{static_cast<const std::int8_t*>(l.w.data), static_cast<const float*>(l.scale.data), nullptr};
  };
  b2_block_weights bw{};
  bw.struct_size = sizeof(b2_block_weights);
  bw.norm1 = w.norm1.data, bw.norm2 = w.norm2.data, bw.q_norm = w.q_norm.data, bw.k_norm = w.k_norm.data;
  bw.qkv = lin(w.qkv8), bw.o = lin(w.o8), bw.up_gate = lin(w.up_gate8), bw.down = lin(w.down8);
  b2_block_run br = b200_block_run(w, run, &a);
  if (attention == AttentionMode::kQ8Fp8) br.attention.variant = B2_ATTENTION_Q8_FP8;
  b2_block_buffers bb{};
  bb.struct_size = sizeof(b2_block_buffers);
  bb.x = static_cast<char*>(a.f.x.data) + run.t0 * a.f.x.stride[0] * 2;          // rows [t0, t1) of the residual stream
  bb.mod = a.f.mod.data;
  bb.rope = static_cast<const char*>(a.f.rope.data) + run.t0 * a.f.rope.stride[0] * 2;
  bb.workspace = workspace, bb.workspace_bytes = workspace_bytes;
  b200_check(b2_run_block_quant(&bw, &bb, &br, stream));
}

}  // namespace mi::moss_dit
