// Guidance and the velocity update of one denoising step, on fp32 latents. What follows the block loop of a step in the
// reference: the classifier-free-guidance combine of the cond / uncond velocities, the skip-layer-guidance correction and
// the Euler or Adams-Bashforth-2 update of the latent (pipeline::guide_prediction in velocity space,
// src/pipeline/samplers/sampler_driver.cpp:565-577; kernels src/pipeline/samplers/sampler_kernels.cu:209-218, 304-310).
// Every op is one fp32 operation rounded once, in the reference's order, so the fused kernel gives the bits of the
// reference's sequence of launches:
//   cfg   v = u + g * (c - u)
//   slg   v = p + s * (c - k),  p = the cfg result, or k itself when cfg is off
//   none  v = c
//   euler x = x + h * v          ab2  x = x + h * (a * v - b * v_prev)
// HBM-bound (up to six streams of 2 MB at 1024^2): one pass with 128-bit accesses instead of up to four launches.
#include <algorithm>
#include <string>

#include "common.cuh"

namespace b2 {
namespace {

struct StepArgs {
  float* x;
  const float* v_cond;
  const float* v_uncond;
  const float* v_skip;
  const float* slg_base;  // the p of the slg line; null: the cfg result, or v_skip when cfg is off
  const float* v_prev;
  float* v_out;
  float g, slg_scale, h, a, b;
  int cfg, slg, update;  // update: 0 none, 1 Euler, 2 Adams-Bashforth 2
  std::int64_t n;
};

__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }

__device__ __forceinline__ float guided(const StepArgs& s, float c, float u, float k, float base) {
  float v = c;
  if (s.cfg) v = fadd(u, fmul(s.g, fsub(c, u)));
  if (s.slg) v = fadd(s.slg_base != nullptr ? base : s.cfg ? v : k, fmul(s.slg_scale, fsub(c, k)));
  return v;
}
__device__ __forceinline__ float updated(const StepArgs& s, float x, float v, float vp) {
  if (s.update == 1) return fadd(x, fmul(s.h, v));
  if (s.update == 2) return fadd(x, fmul(s.h, fsub(fmul(s.a, v), fmul(s.b, vp))));
  return x;
}

// kVec: every pointer in use is 16-byte aligned and n % 4 == 0.
template <bool kVec>
__global__ void __launch_bounds__(256) guided_step_kernel(const StepArgs s) {
  const std::int64_t stride = static_cast<std::int64_t>(gridDim.x) * blockDim.x;
  const std::int64_t first = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if constexpr (kVec) {
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const auto ld = [&](const float* p, std::int64_t i, bool on) { return on ? reinterpret_cast<const float4*>(p)[i] : zero; };
    for (std::int64_t i = first; i < s.n / 4; i += stride) {
      const float4 c = ld(s.v_cond, i, true), u = ld(s.v_uncond, i, s.cfg != 0), k = ld(s.v_skip, i, s.slg != 0);
      const float4 p = ld(s.slg_base, i, s.slg != 0 && s.slg_base != nullptr);
      const float4 v = make_float4(guided(s, c.x, u.x, k.x, p.x), guided(s, c.y, u.y, k.y, p.y), guided(s, c.z, u.z, k.z, p.z),
                                   guided(s, c.w, u.w, k.w, p.w));
      if (s.v_out != nullptr) reinterpret_cast<float4*>(s.v_out)[i] = v;
      if (s.update != 0) {
        const float4 x = ld(s.x, i, true), q = ld(s.v_prev, i, s.update == 2);
        reinterpret_cast<float4*>(s.x)[i] =
            make_float4(updated(s, x.x, v.x, q.x), updated(s, x.y, v.y, q.y), updated(s, x.z, v.z, q.z), updated(s, x.w, v.w, q.w));
      }
    }
  } else {
    for (std::int64_t i = first; i < s.n; i += stride) {
      const float v = guided(s, s.v_cond[i], s.cfg ? s.v_uncond[i] : 0.f, s.slg ? s.v_skip[i] : 0.f,
                             s.slg && s.slg_base != nullptr ? s.slg_base[i] : 0.f);
      if (s.v_out != nullptr) s.v_out[i] = v;
      if (s.update != 0) s.x[i] = updated(s, s.x[i], v, s.update == 2 ? s.v_prev[i] : 0.f);
    }
  }
}

int launch_step(const char* op, const StepArgs& s, cudaStream_t stream) {
  if (s.n == 0) return B2_OK;
  bool vec = s.n % 4 == 0;
  for (const void* p : {static_cast<const void*>(s.x), static_cast<const void*>(s.v_cond), static_cast<const void*>(s.v_uncond),
                        static_cast<const void*>(s.v_skip), static_cast<const void*>(s.slg_base), static_cast<const void*>(s.v_prev),
                        static_cast<const void*>(s.v_out)}) {
    vec = vec && (p == nullptr || aligned_to(p, 16));
  }
  const std::int64_t items = vec ? s.n / 4 : s.n;
  const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((items + 255) / 256, static_cast<std::int64_t>(sm_count()) * 8));
  if (vec) guided_step_kernel<true><<<blocks, 256, 0, stream>>>(s);
  else guided_step_kernel<false><<<blocks, 256, 0, stream>>>(s);
  return check_launch(op);
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" {

int b2_cfg_combine(const float* cond, const float* uncond, float g, float* out, int64_t n, void* stream) {
  constexpr const char* op = "cfg_combine";
  if (n < 0 || (n > 0 && (cond == nullptr || uncond == nullptr || out == nullptr))) return fail_invalid(op, "null operand or negative n");
  StepArgs s{};
  s.v_cond = cond, s.v_uncond = uncond, s.v_out = out, s.g = g, s.cfg = 1, s.n = n;
  return launch_step(op, s, as_stream(stream));
}

int b2_slg_correct(const float* pred, const float* cond, const float* skipped, float scale, float* out, int64_t n, void* stream) {
  constexpr const char* op = "slg_correct";
  if (n < 0 || (n > 0 && (pred == nullptr || cond == nullptr || skipped == nullptr || out == nullptr))) {
    return fail_invalid(op, "null operand or negative n");
  }
  StepArgs s{};
  s.v_cond = cond, s.v_skip = skipped, s.slg_base = pred, s.v_out = out, s.slg_scale = scale, s.slg = 1, s.n = n;
  return launch_step(op, s, as_stream(stream));
}

int b2_euler_update(float* x, const float* v, float h, int64_t n, void* stream) {
  constexpr const char* op = "euler_update";
  if (n < 0 || (n > 0 && (x == nullptr || v == nullptr))) return fail_invalid(op, "null operand or negative n");
  StepArgs s{};
  s.x = x, s.v_cond = v, s.h = h, s.update = 1, s.n = n;
  return launch_step(op, s, as_stream(stream));
}

int b2_ab2_update(float* x, const float* v, const float* v_prev, float h, float a, float b, int64_t n, void* stream) {
  constexpr const char* op = "ab2_update";
  if (n < 0 || (n > 0 && (x == nullptr || v == nullptr || v_prev == nullptr))) return fail_invalid(op, "null operand or negative n");
  StepArgs s{};
  s.x = x, s.v_cond = v, s.v_prev = v_prev, s.h = h, s.a = a, s.b = b, s.update = 2, s.n = n;
  return launch_step(op, s, as_stream(stream));
}

int b2_guided_velocity_step(const b2_guided_step* g, void* stream) {
  constexpr const char* op = "guided_velocity_step";
  if (g == nullptr || g->struct_size < sizeof(b2_guided_step)) return fail_invalid(op, "null step or from an older header");
  if (g->n < 0 || g->update < 0 || g->update > 2) return fail_invalid(op, "negative n or unknown update (0 none, 1 Euler, 2 AB2)");
  if (g->n > 0) {
    if (g->v_cond == nullptr || (g->cfg && g->v_uncond == nullptr) || (g->slg && g->v_skip == nullptr)) {
      return fail_invalid(op, "missing velocity (v_cond always, v_uncond with cfg, v_skip with slg)");
    }
    if (g->update != 0 && g->x == nullptr) return fail_invalid(op, "an update needs x");
    if (g->update == 2 && g->v_prev == nullptr) return fail_invalid(op, "the Adams-Bashforth update needs v_prev");
    if (g->update == 0 && g->v_out == nullptr) return fail_invalid(op, "nothing to write: no update and no v_out");
    if (g->update == 2 && g->v_out == g->v_prev && g->v_out != nullptr) {
      return fail_invalid(op, "v_out must not alias v_prev (the update reads v_prev after v_out is written)");
    }
  }
  StepArgs s{};
  s.x = g->x, s.v_cond = g->v_cond, s.v_uncond = g->v_uncond, s.v_skip = g->v_skip, s.v_prev = g->v_prev, s.v_out = g->v_out;
  s.g = g->cfg_scale, s.slg_scale = g->slg_scale, s.h = g->h, s.a = g->a, s.b = g->b;
  s.cfg = g->cfg != 0, s.slg = g->slg != 0, s.update = g->update, s.n = g->n;
  return launch_step(op, s, as_stream(stream));
}

}  // extern "C"
