// C-ABI shim over the reference's own CUDA kernels for the quantized-block path, compiled for sm_100a from the
// reference tree where it lies (their legacy mma.sync kernels: the same-GPU, bit-level oracle and the "reference on this
// box" speed baseline). TEST INFRASTRUCTURE ONLY. Arguments mirror the reference's signatures; exceptions become -1.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <exception>
#include <stdexcept>

#include "core/tensor.h"
#include "kernels/attention_q8/attention_q8.h"
#include "kernels/attention_q8/q8_kernels.h"
#include "kernels/fused/qk_norm_rope.h"
#include "kernels/quant/quant.h"
#include "models/moss_dit/dit_kernels.h"
#include "pipeline/samplers/sampler_kernels.h"
#include "kernels/sm75/int8_sm75.h"
#include "kernels/sm75/sm75.h"

// Pieces of the reference this build leaves out (pre-Ampere paths, fp16 P·V attention): never reached on B200.
namespace mi::kernels::sm75 {
bool fp16_weights() { return false; }
void int8_gemm(const quant::Int8Operands&, const __nv_bfloat16*, __nv_bfloat16*, std::int64_t, cudaStream_t) {
  throw std::logic_error("sm75 path not built");
}
void int8_gemm_gated_residual(const quant::Int8Operands&, const __nv_bfloat16*, const __nv_bfloat16*, __nv_bfloat16*,
                              std::int64_t, cudaStream_t) {
  throw std::logic_error("sm75 path not built");
}
void int8_gemm_situ_glu(const quant::Int8Operands&, __nv_bfloat16*, std::int64_t, cudaStream_t) {
  throw std::logic_error("sm75 path not built");
}
}  // namespace mi::kernels::sm75
namespace mi::attention_q8::detail {
void run_int8_fp16(const AttnParams&, bool, cudaStream_t) { throw std::logic_error("fp16 P.V variants not built"); }
int int8_fp16_kernel_arch(bool) { return 0; }
}  // namespace mi::attention_q8::detail

namespace {
using mi::DType;
using mi::Tensor;
thread_local char g_err[512];
template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    std::snprintf(g_err, sizeof(g_err), "%s", e.what());
    return -1;
  }
}
Tensor view3(void* p, std::int64_t tokens, std::int64_t heads, std::int64_t row, std::int64_t head) {
  Tensor t = Tensor::view(p, DType::kBF16, mi::Device::kCUDA, {tokens, heads, 128});
  t.stride[0] = row, t.stride[1] = head, t.stride[2] = 1;
  return t;
}
mi::kernels::quant::Int8Operands ops(const std::int8_t* xq, std::int64_t ldx, const float* xs, const std::int8_t* w,
                                     const float* ws, std::int64_t m, std::int64_t n, std::int64_t k) {
  mi::kernels::quant::Int8Operands o;
  o.x_q = xq, o.ldx = ldx, o.x_scale = xs, o.w = w, o.w_scale = ws, o.m = m, o.n = n, o.k = k;
  return o;
}
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err; }

int ref_rotate_quantize(const void* x, std::int64_t ldx, std::int8_t* q, std::int64_t ldq, float* scale, std::int64_t m,
                        int k, void* stream) {
  return guarded([&] {
    mi::kernels::quant::rotate_quantize(static_cast<const __nv_bfloat16*>(x), ldx, q, ldq, scale, m, k,
                                        static_cast<cudaStream_t>(stream));
  });
}

int ref_rms_norm_modulate_rotate_quantize(const void* x, std::int64_t ldx, const void* w, const void* sc, const void* sh,
                                          std::int8_t* q, std::int64_t ldq, float* scale, std::int64_t m, int k,
                                          void* stream) {
  using bf = __nv_bfloat16;
  return guarded([&] {
    mi::kernels::quant::rms_norm_modulate_rotate_quantize(static_cast<const bf*>(x), ldx, static_cast<const bf*>(w),
                                                          static_cast<const bf*>(sc), static_cast<const bf*>(sh), q, ldq,
                                                          scale, m, k, static_cast<cudaStream_t>(stream));
  });
}

int ref_int8_gemm(const std::int8_t* xq, std::int64_t ldx, const float* xs, const std::int8_t* w, const float* ws,
                  std::int64_t m, std::int64_t n, std::int64_t k, const void* bias, void* out, std::int64_t ldo,
                  void* stream) {
  using bf = __nv_bfloat16;
  return guarded([&] {
    mi::kernels::quant::int8_gemm(ops(xq, ldx, xs, w, ws, m, n, k), static_cast<const bf*>(bias), static_cast<bf*>(out),
                                  ldo, static_cast<cudaStream_t>(stream));
  });
}

int ref_int8_gemm_gated_residual(const std::int8_t* xq, std::int64_t ldx, const float* xs, const std::int8_t* w,
                                 const float* ws, std::int64_t m, std::int64_t n, std::int64_t k, const void* bias,
                                 const void* gate, void* residual, std::int64_t ldr, void* stream) {
  using bf = __nv_bfloat16;
  return guarded([&] {
    mi::kernels::quant::int8_gemm_gated_residual(ops(xq, ldx, xs, w, ws, m, n, k), static_cast<const bf*>(bias),
                                                 static_cast<const bf*>(gate), static_cast<bf*>(residual), ldr,
                                                 static_cast<cudaStream_t>(stream));
  });
}

int ref_int8_gemm_situ_glu(const std::int8_t* xq, std::int64_t ldx, const float* xs, const std::int8_t* w, const float* ws,
                           std::int64_t m, std::int64_t n, std::int64_t k, void* out, std::int64_t ldo, void* stream) {
  return guarded([&] {
    mi::kernels::quant::int8_gemm_situ_glu(ops(xq, ldx, xs, w, ws, m, n, k), static_cast<__nv_bfloat16*>(out), ldo,
                                           static_cast<cudaStream_t>(stream));
  });
}

int ref_qk_norm_rope(void* qkv, std::int64_t ld, std::int64_t tokens, int heads, void* q_norm, void* k_norm, void* table,
                     std::int64_t table_ld, void* stream) {
  return guarded([&] {
    Tensor t = Tensor::view(qkv, DType::kBF16, mi::Device::kCUDA, {tokens, ld});
    Tensor qn = Tensor::view(q_norm, DType::kBF16, mi::Device::kCUDA, {128});
    Tensor kn = Tensor::view(k_norm, DType::kBF16, mi::Device::kCUDA, {128});
    Tensor tab = Tensor::view(table, DType::kBF16, mi::Device::kCUDA, {tokens, 128});
    tab.stride[0] = table_ld;
    mi::kernels::fused::qk_norm_rope_moss(t, heads, qn, kn, tab, static_cast<cudaStream_t>(stream));
  });
}

std::size_t ref_attention_q8_workspace_bytes(std::int64_t total, int batch, int max_seqlen, int heads) {
  mi::attention_q8::Options o;
  o.variant = mi::attention_q8::Variant::kInt8Fp8F32Acc;
  return mi::attention_q8::attention_q8_workspace_bytes(o, total, total, batch, max_seqlen, heads, heads);
}

// Self-attention over a fused qkv buffer [total, 3 * heads * 128] (row stride ld); variant 2 = int8_fp8 (fp16 tile
// accumulation), 3 = int8_fp8_f32acc; p_range / v_range <= 0 pick the variant's defaults; norm_rope != 0 runs the fused
// QK-norm + RoPE pre-pass.
int ref_attention_q8_variant(int variant, float p_range, float v_range, void* qkv, std::int64_t ld, std::int64_t total,
                             int heads, void* out, std::int64_t out_ld, int* cu, int batch, int max_seqlen, float scale,
                             void* workspace, std::size_t workspace_bytes, int norm_rope, void* q_norm, void* k_norm,
                             void* table, void* stream) {
  return guarded([&] {
    auto* base = static_cast<__nv_bfloat16*>(qkv);
    const Tensor q = view3(base, total, heads, ld, 128), k = view3(base + heads * 128, total, heads, ld, 128);
    const Tensor v = view3(base + 2 * heads * 128, total, heads, ld, 128), o = view3(out, total, heads, out_ld, 128);
    const Tensor cuq = Tensor::view(cu, DType::kI32, mi::Device::kCUDA, {batch + 1});
    mi::attention_q8::Options opt;
    opt.variant = variant == 2 ? mi::attention_q8::Variant::kInt8Fp8 : mi::attention_q8::Variant::kInt8Fp8F32Acc;
    opt.p_range = p_range, opt.v_range = v_range;
    mi::attention_q8::QkNormRope nr;
    if (norm_rope) {
      nr.q_norm = Tensor::view(q_norm, DType::kBF16, mi::Device::kCUDA, {128});
      nr.k_norm = Tensor::view(k_norm, DType::kBF16, mi::Device::kCUDA, {128});
      nr.table = Tensor::view(table, DType::kBF16, mi::Device::kCUDA, {total, 128});
    }
    mi::attention_q8::attention_q8(opt, q, k, v, o, cuq, cuq, max_seqlen, scale, workspace, workspace_bytes,
                                   static_cast<cudaStream_t>(stream), norm_rope ? &nr : nullptr);
  });
}

int ref_attention_q8(void* qkv, std::int64_t ld, std::int64_t total, int heads, void* out, std::int64_t out_ld, int* cu,
                     int batch, int max_seqlen, float scale, void* workspace, std::size_t workspace_bytes, int norm_rope,
                     void* q_norm, void* k_norm, void* table, void* stream) {
  return ref_attention_q8_variant(3, 0.f, 0.f, qkv, ld, total, heads, out, out_ld, cu, batch, max_seqlen, scale, workspace,
                                  workspace_bytes, norm_rope, q_norm, k_norm, table, stream);
}

// The guidance and velocity-update kernels of the sampler driver (src/pipeline/samplers/sampler_kernels.cu).
int ref_cfg_velocity(const float* c, const float* u, float g, float* out, std::int64_t n, cudaStream_t st) {
  return guarded([&] { mi::pipeline::sampler_kernels::cfg_velocity(c, u, g, out, n, st); });
}

int ref_slg_velocity(const float* p, const float* c, const float* k, float s, float* out, std::int64_t n, cudaStream_t st) {
  return guarded([&] { mi::pipeline::sampler_kernels::slg_velocity(p, c, k, s, out, n, st); });
}
int ref_velocity_euler(float* x, const float* v, float h, std::int64_t n, cudaStream_t st) {
  return guarded([&] { mi::pipeline::sampler_kernels::velocity_euler(x, v, h, n, st); });
}
int ref_ab2(float* x, const float* v, const float* vp, float h, float a, float b, std::int64_t n, cudaStream_t st) {
  return guarded([&] { mi::pipeline::sampler_kernels::ab2(x, v, vp, h, a, b, n, st); });
}

// The shell's exactly specified kernels (src/models/moss_dit/dit_kernels.cu): the two transposes and linear_fp32_row.
int ref_latent_to_tokens(float* latents, std::int64_t channels, std::int64_t h, std::int64_t w, void* tokens, cudaStream_t st) {
  return guarded([&] {
    mi::moss_dit::latent_to_tokens(Tensor::view(latents, DType::kF32, mi::Device::kCUDA, {channels, h, w}),
                                   Tensor::view(tokens, DType::kBF16, mi::Device::kCUDA, {h * w, channels}), st);
  });
}
int ref_tokens_to_latent(void* tokens, std::int64_t channels, std::int64_t h, std::int64_t w, float* latents, cudaStream_t st) {
  return guarded([&] {
    mi::moss_dit::tokens_to_latent(Tensor::view(tokens, DType::kBF16, mi::Device::kCUDA, {h * w, channels}),
                                   Tensor::view(latents, DType::kF32, mi::Device::kCUDA, {channels, h, w}), st);
  });
}
int ref_linear_fp32_row(void* w, std::int64_t n, std::int64_t k, const float* x, const float* bias, void* out, cudaStream_t st) {
  return guarded([&] {
    mi::moss_dit::linear_fp32_row(Tensor::view(w, DType::kBF16, mi::Device::kCUDA, {n, k}), x, bias,
                                  Tensor::view(out, DType::kBF16, mi::Device::kCUDA, {n}), st);
  });
}

}  // extern "C"
