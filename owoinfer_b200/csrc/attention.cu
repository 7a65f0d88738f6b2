// SageAttention-style 8-bit attention for sm_100a, plus the MOSS QK-norm + RoPE and RoPE-table kernels that feed it.
//
//   pre-pass (HBM-bound, 128-bit accesses)
//     prologue   (fused QK-norm + RoPE only) per (32 tokens, head): RMS-norm + RoPE of q and k, k written back,
//                Q quantised
//     stats      per (512-key chunk, head, sequence): partial per-channel K sums and V |max| in a fixed order
//     finalize   k_mean = bf16(sum / len); v_scale = amax / v_range; v_recp = v_range / amax
//     quantise   Q per (32 tokens, head) [when not fused]; K - k_mean per (64 keys, head) -> int8; V * v_recp -> e4m3
//   attention: one CTA per (128 query rows, head, sequence), two CTAs per SM; K/V in 128-key tiles, the tensor work in
//   64-key sub-tiles with the score accumulator double-buffered in TMEM
//     S = Q8 · K8^T   tcgen05.mma kind::i8 (N = 64), int32 accumulator in TMEM (exact)
//     softmax         4 warps, one thread per query row: S -> fp32 (exact: |S| < 2^22), scaled by
//                     sm_scale * log2e * q_scale * k_scale[64-key block], P = exp2(.) against a reference maximum that
//                     is raised only when its headroom runs out (which makes rescaling O rare), denominator in fp32
//                     from the unrounded P, P rounded to e4m3 into a swizzled shared tile
//     O += P8 · V8    tcgen05.mma kind::f8f6f4, fp32 accumulator in TMEM; V is read in its natural [key, channel]
//                     layout as an MN-major operand, so the pre-pass needs no transpose
//     out = O / d * v_scale[channel] -> bf16
// Reference semantics: src/kernels/attention_q8/attention_q8.h:1-127, q8_preprocess.cu:67-385,
// third_party/sageattention/csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:54-743 (variant kInt8Fp8F32Acc);
// src/kernels/fused/qk_norm_rope.cu:43-89; src/kernels/basic/rope.cu:30-51.
#include <algorithm>
#include <climits>
#include <cmath>
#include <string>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int kHeadDim = 128;
constexpr int kStatsChunk = 512;
constexpr std::size_t kAlign = 256;

__device__ int g_attn_status = 0;
#ifdef B2_ATTN_TRACE
__device__ long long g_attn_trace[8192];
#define TRACE(slot) do { if (tracing) a.trace[u * 16 + (slot)] = clock64(); } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif

__device__ __forceinline__ std::uint64_t global_ns() {
  std::uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool wait_bar(std::uint32_t bar, std::uint32_t parity, volatile int* abort_word) {
  if (mbar_try_wait(bar, parity)) return true;
  const std::uint64_t t0 = global_ns();
  for (;;) {
    // A tight inner loop (test, branch); the abort word and the clock are looked at once per 256 tests.
#pragma unroll 1
    for (int i = 0; i < 256; ++i) {
      if (mbar_try_wait_hint(bar, parity)) return true;
    }
    if (*abort_word != 0) return false;
    if (global_ns() - t0 > 200000000ull) {
      *abort_word = 1;
      return false;
    }
  }
}

// The same for a role with slack (the TMA and MMA warps share their scheduler with softmax warps): sleeps between tests so
// that waiting costs next to no issue slots.
template <int kSleepNs>
__device__ __forceinline__ bool wait_bar_relaxed(std::uint32_t bar, std::uint32_t parity, volatile int* abort_word) {
  if (mbar_try_wait(bar, parity)) return true;
  const std::uint64_t t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      __nanosleep(kSleepNs);
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_word != 0) return false;
    if (global_ns() - t0 > 200000000ull) {
      *abort_word = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* x) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const std::uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* x) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  x[0] = __uint_as_float(raw.x << 16), x[1] = __uint_as_float(raw.x & 0xFFFF0000u);
  x[2] = __uint_as_float(raw.y << 16), x[3] = __uint_as_float(raw.y & 0xFFFF0000u);
}
__device__ __forceinline__ std::uint32_t pack_bf2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const std::uint32_t*>(&h);
}
__device__ __forceinline__ std::int32_t f2i8(float v) {
  std::int32_t r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ std::uint32_t pack_i8x4(float a, float b, float c, float d) {
  return (static_cast<std::uint32_t>(f2i8(a)) & 0xFF) | ((static_cast<std::uint32_t>(f2i8(b)) & 0xFF) << 8) |
         ((static_cast<std::uint32_t>(f2i8(c)) & 0xFF) << 16) | ((static_cast<std::uint32_t>(f2i8(d)) & 0xFF) << 24);
}
// Four floats -> four e4m3 bytes (round to nearest even, saturate to +-448): `a` in the low byte.
__device__ __forceinline__ std::uint32_t e4m3x4(float a, float b, float c, float d) {
  std::uint32_t w;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(w)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return w;
}
// Packed fp32 pairs (one instruction for two lanes of work): d = a * b + c and d = a + b on (x, y) pairs.
__device__ __forceinline__ std::uint64_t pack2(float x, float y) {
  std::uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
  return r;
}
__device__ __forceinline__ void unpack2(std::uint64_t v, float& x, float& y) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ std::uint64_t fma2(std::uint64_t a, std::uint64_t b, std::uint64_t c) {
  std::uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ std::uint64_t add2(std::uint64_t a, std::uint64_t b) {
  std::uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
#ifndef B2_TRACE_WARP
#define B2_TRACE_WARP 2
#endif
#ifndef B2_MMA_SLEEP_NS
#define B2_MMA_SLEEP_NS 100
#endif
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------------------------------------------
// QK-norm + RoPE (standalone) and the RoPE table.
// ---------------------------------------------------------------------------------------------------------------
struct NormRopeArgs {
  __nv_bfloat16* qkv;
  std::int64_t ld;
  const __nv_bfloat16* q_norm;
  const __nv_bfloat16* k_norm;
  const __nv_bfloat16* table;
  std::int64_t table_ld;
  std::int64_t tokens;
  int heads;
  float factor;
};

// One warp per (token, q-or-k head), lane l holding channels 4l..4l+3: the quad sum then the shuffle-down tree are the
// order of torch's reduce for a 128-wide row. RoPE pairs channel d with d + 64, i.e. lane l with lane l ^ 16.
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(const NormRopeArgs a) {
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const std::int64_t items = a.tokens * 2 * a.heads;
  const std::int64_t stride = static_cast<std::int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (std::int64_t item = static_cast<std::int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); item < items;
       item += stride) {
    const std::int64_t token = item / (2 * a.heads);
    const int head = static_cast<int>(item % (2 * a.heads));
    __nv_bfloat16* p = a.qkv + token * a.ld + static_cast<std::int64_t>(head) * kHeadDim + 4 * lane;
    float x[4], w[4], si[4], co[4];
    load4(p, x);
    load4((head < a.heads ? a.q_norm : a.k_norm) + 4 * lane, w);
    const __nv_bfloat16* tab = a.table + token * a.table_ld + 4 * (lane & 15);
    load4(tab, si);
    load4(tab + 64, co);
    float v = fadd(fadd(fadd(fmul(x[0], x[0]), fmul(x[1], x[1])), fmul(x[2], x[2])), fmul(x[3], x[3]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fadd(v, __shfl_down_sync(0xffffffffu, v, off));
    const float r = rsqrtf(fadd(fmul(__shfl_sync(0xffffffffu, v, 0), a.factor), 1e-6f));
    const bool lo_half = lane < 16;
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float y = rbf(fmul(rbf(fmul(x[i], r)), w[i]));
      const float other = __shfl_xor_sync(0xffffffffu, y, 16);
      const float lo = lo_half ? y : other, hi = lo_half ? other : y;
      o[i] = lo_half ? fadd(rbf(fmul(lo, co[i])), rbf(fmul(-hi, si[i]))) : fadd(rbf(fmul(hi, co[i])), rbf(fmul(lo, si[i])));
    }
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf2(o[0], o[1]), pack_bf2(o[2], o[3]));
  }
}

struct RopeBands {
  float v[16];
};
// 1 / 1e4^(i/16), i = 0..15, as fp32 (fp32 pow, then fp32 reciprocal).
constexpr RopeBands kBands = {{1.f, 0.562341332f, 0.316227764f, 0.177827939f, 0.100000001f, 0.0562341288f, 0.0316227786f,
                               0.0177827943f, 0.00999999978f, 0.00562341325f, 0.00316227786f, 0.00177827943f,
                               0.00100000005f, 0.000562341302f, 0.000316227786f, 0.00017782794f}};

// One thread per table element: row r, column c; columns 0..63 hold sin, 64..127 cos, over (axis, band) = (c % 64 / 16,
// c % 16); image tokens (r < height * width) have coordinates (0, text_length, row - (H-1)/2, col - (W-1)/2), text token i
// has (0, i, 0, 0).
// Reference tokens of the edit layout (image_r, image_f = reference index + 1, 0; no text rows) use the same arithmetic.
__global__ void rope_table_kernel(__nv_bfloat16* out, std::int64_t ld, std::int64_t n, int height, int width,
                                  float image_r, float image_f, const RopeBands bands) {
  const std::int64_t hw = static_cast<std::int64_t>(height) * width;
  const float h_mid = static_cast<float>((height - 1) / 2.0), w_mid = static_cast<float>((width - 1) / 2.0);
  const std::int64_t total = n * 128;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const std::int64_t r = i >> 7;
    const int c = static_cast<int>(i & 127), pz = c & 63, axis = pz >> 4, band = pz & 15;
    float coord = 0.f;
    if (r < hw) {
      if (axis == 0) coord = image_r;
      if (axis == 1) coord = image_f;
      if (axis == 2) coord = __fsub_rn(static_cast<float>(r / width), h_mid);
      if (axis == 3) coord = __fsub_rn(static_cast<float>(r % width), w_mid);
    } else if (axis == 1) {
      coord = static_cast<float>(r - hw);
    }
    const float phase = fmul(coord, bands.v[band]);
    out[r * ld + c] = __float2bfloat16_rn(c < 64 ? sinf(phase) : cosf(phase));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Pre-pass.
// ---------------------------------------------------------------------------------------------------------------
struct PrepArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* k;
  const __nv_bfloat16* v;
  std::int64_t q_row, q_head, k_row, k_head, v_row, v_head;
  const int* cu;
  int batch, heads, max_seqlen, chunks, q_blocks, k_blocks;
  float v_range;
  // fused prologue
  const __nv_bfloat16* q_norm;
  const __nv_bfloat16* k_norm;
  const __nv_bfloat16* table;
  std::int64_t table_row;
  float norm_factor;
  // outputs
  std::int8_t* q_i8;
  std::int8_t* k_i8;
  std::uint8_t* v8;
  float* q_scale;
  float* k_scale;
  float* k_mean;
  float* v_scale;
  float* v_recp;
  float* part_sum;
  float* part_amax;
};

// Packed bf16 pairs: a * b and a + b, each result rounded once to bf16. For bf16 operands these equal the fp32 operation
// followed by a rounding to bf16 (the fp32 product of two bf16 values is exact; an fp32 sum of two bf16 values is either
// exact or, when the exponents are more than 16 apart, lands nowhere near a bf16 rounding boundary).
__device__ __forceinline__ std::uint32_t bmul2(std::uint32_t a, std::uint32_t b) {
  std::uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ std::uint32_t badd2(std::uint32_t a, std::uint32_t b) {
  std::uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// RMS-norm + RoPE of one (token, head) row held by 16 lanes x 8 channels (two of the 32 quads of the standalone kernel
// per lane: its shuffle tree 16, 8, 4, 2, 1 becomes 8, 4, 2, 1 per quad and a final add of the two at lane 0).
// x: the row's eight raw bf16 values as four packed pairs; w, co: weight and cosine pairs; si: sine pairs, already negated
// for the lanes of the low half (lo' = bf16(lo*cos) + bf16(-hi*sin), hi' = bf16(hi*cos) + bf16(lo*sin)). After the first
// rounding (x * r, with the fp32 r) every step works on bf16 values and is done on packed pairs. y: four packed pairs.
__device__ __forceinline__ void norm_rope_row(const std::uint32_t (&x)[4], const std::uint32_t (&w)[4],
                                              const std::uint32_t (&si)[4], const std::uint32_t (&co)[4], float factor,
                                              std::uint32_t (&y)[4]) {
  float f[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(x[i] << 16);
    f[2 * i + 1] = __uint_as_float(x[i] & 0xFFFF0000u);
  }
  float quad[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float* e = f + 4 * h;
    quad[h] = fadd(fadd(fadd(fmul(e[0], e[0]), fmul(e[1], e[1])), fmul(e[2], e[2])), fmul(e[3], e[3]));
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) {
#pragma unroll
    for (int h = 0; h < 2; ++h) quad[h] = fadd(quad[h], __shfl_down_sync(0xffffffffu, quad[h], off, 16));
  }
  const float total = __shfl_sync(0xffffffffu, fadd(quad[0], quad[1]), 0, 16);
  const float r = rsqrtf(fadd(fmul(total, factor), 1e-6f));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const std::uint32_t n = bmul2(pack_bf2(fmul(f[2 * i], r), fmul(f[2 * i + 1], r)), w[i]);
    const std::uint32_t o = __shfl_xor_sync(0xffffffffu, n, 8, 16);  // the channel pair 64 further (or back)
    y[i] = badd2(bmul2(n, co[i]), bmul2(o, si[i]));
  }
}

// Fused prologue, one CTA per (32-token Q block, head, sequence): 32 token rows x 16 lanes x 8 channels. RMS-norm + RoPE
// of q and k; Q quantised with the block's scale; k written back in place for the statistics and K/V quantisation
// passes. Every load of a row is issued before the first use.
__global__ void __launch_bounds__(512, 2) norm_rope_quant_q_kernel(const PrepArgs p) {
  const int bx = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int lane = static_cast<int>(threadIdx.x) & 15, row = static_cast<int>(threadIdx.x) >> 4;
  const int start = p.cu[b], len = p.cu[b + 1] - start;
  const std::int64_t scale_at = (static_cast<std::int64_t>(b) * p.heads + h) * p.q_blocks + bx;
  if (bx * 32 >= len) {
    // A block at or past the sequence end holds no tokens: its scale is the empty block's.
    if (threadIdx.x == 0) p.q_scale[scale_at] = 0.0000001f / 127.0f;
    return;
  }
  const int t = bx * 32 + row;
  const bool valid = t < len;
  const std::int64_t tok = static_cast<std::int64_t>(start) + t;
  const int pair = (lane & 7) * 8;
  const auto quad = [](uint4 v, std::uint32_t (&o)[4]) { o[0] = v.x, o[1] = v.y, o[2] = v.z, o[3] = v.w; };
  uint4 xr = make_uint4(0, 0, 0, 0), kr = xr, sr = xr, cr = xr;
  __nv_bfloat16* k_at = p.k + tok * p.k_row + h * p.k_head + lane * 8;
  if (valid) {
    xr = *reinterpret_cast<const uint4*>(p.q + tok * p.q_row + h * p.q_head + lane * 8);
    kr = *reinterpret_cast<const uint4*>(k_at);
    sr = *reinterpret_cast<const uint4*>(p.table + tok * p.table_row + pair);
    cr = *reinterpret_cast<const uint4*>(p.table + tok * p.table_row + 64 + pair);
  }
  std::uint32_t x[4], kx[4], si[4], co[4], w[4], qy[4], ky[4];
  quad(xr, x), quad(kr, kx), quad(sr, si), quad(cr, co);
  if (lane < 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) si[i] ^= 0x80008000u;
  }
  quad(*reinterpret_cast<const uint4*>(p.q_norm + lane * 8), w);
  norm_rope_row(x, w, si, co, p.norm_factor, qy);
  quad(*reinterpret_cast<const uint4*>(p.k_norm + lane * 8), w);
  norm_rope_row(kx, w, si, co, p.norm_factor, ky);
  if (valid) *reinterpret_cast<uint4*>(k_at) = make_uint4(ky[0], ky[1], ky[2], ky[3]);
  float q[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    q[2 * i] = __uint_as_float(qy[i] << 16);
    q[2 * i + 1] = __uint_as_float(qy[i] & 0xFFFF0000u);
  }
  float qmax = 0.0000001f;
#pragma unroll
  for (int j = 0; j < 8; ++j) qmax = fmaxf(qmax, fabsf(q[j]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) qmax = fmaxf(qmax, __shfl_xor_sync(0xffffffffu, qmax, off));
  __shared__ float s_w[16];
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = qmax;
  __syncthreads();
  qmax = s_w[0];
#pragma unroll
  for (int i = 1; i < 16; ++i) qmax = fmaxf(qmax, s_w[i]);
  if (threadIdx.x == 0) p.q_scale[scale_at] = qmax / 127.0f;
  if (!valid) return;
  const float qs = 127.0f / qmax;
  *reinterpret_cast<uint2*>(p.q_i8 + (tok * p.heads + h) * kHeadDim + lane * 8) =
      make_uint2(pack_i8x4(q[0] * qs, q[1] * qs, q[2] * qs, q[3] * qs), pack_i8x4(q[4] * qs, q[5] * qs, q[6] * qs, q[7] * qs));
}

// Statistics, one CTA per (512-key chunk, head, sequence): 16 token rows x 16 lanes x 8 channels. Row-thread `row` adds
// tokens row, row + 16, ... of the chunk in order; the 16 partials are then added in order, and the finalize kernel adds
// the chunks in order: the K mean is reproducible and independent of the launch shape. Loads run four tokens ahead.
__global__ void __launch_bounds__(256) stats_kernel(const PrepArgs p) {
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int lane = static_cast<int>(threadIdx.x) & 15, row = static_cast<int>(threadIdx.x) >> 4;
  const int start = p.cu[b], len = p.cu[b + 1] - start;
  float sum[8] = {}, amax[8] = {};
  __shared__ float s_red[16][kHeadDim];

  const int t_end = min(len, (c + 1) * kStatsChunk);
  constexpr int kAhead = 4;
  for (int t0 = c * kStatsChunk + row; t0 < t_end; t0 += 16 * kAhead) {
    uint4 kr[kAhead], vr[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int t = t0 + 16 * u;
      const std::int64_t tok = static_cast<std::int64_t>(start) + t;
      if (t < t_end) {
        kr[u] = *reinterpret_cast<const uint4*>(p.k + tok * p.k_row + h * p.k_head + lane * 8);
        vr[u] = *reinterpret_cast<const uint4*>(p.v + tok * p.v_row + h * p.v_head + lane * 8);
      } else {
        kr[u] = vr[u] = make_uint4(0, 0, 0, 0);  // +0 leaves the sum and the maximum as they are
      }
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (t0 + 16 * u >= t_end) break;
      const std::uint32_t kw[4] = {kr[u].x, kr[u].y, kr[u].z, kr[u].w}, vw[4] = {vr[u].x, vr[u].y, vr[u].z, vr[u].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        sum[2 * i] += __uint_as_float(kw[i] << 16);
        sum[2 * i + 1] += __uint_as_float(kw[i] & 0xFFFF0000u);
        amax[2 * i] = fmaxf(amax[2 * i], fabsf(__uint_as_float(vw[i] << 16)));
        amax[2 * i + 1] = fmaxf(amax[2 * i + 1], fabsf(__uint_as_float(vw[i] & 0xFFFF0000u)));
      }
    }
  }

  const std::int64_t at = ((static_cast<std::int64_t>(b) * p.heads + h) * p.chunks + c) * kHeadDim + threadIdx.x;
#pragma unroll
  for (int j = 0; j < 8; ++j) s_red[row][lane * 8 + j] = sum[j];
  __syncthreads();
  if (threadIdx.x < kHeadDim) {
    float s = 0.f;
    for (int r = 0; r < 16; ++r) s += s_red[r][threadIdx.x];
    p.part_sum[at] = s;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 8; ++j) s_red[row][lane * 8 + j] = amax[j];
  __syncthreads();
  if (threadIdx.x < kHeadDim) {
    float m = 0.f;
    for (int r = 0; r < 16; ++r) m = fmaxf(m, s_red[r][threadIdx.x]);
    p.part_amax[at] = m;
  }
}

__global__ void __launch_bounds__(kHeadDim) finalize_kernel(const PrepArgs p) {
  const int h = blockIdx.x, b = blockIdx.y, ch = threadIdx.x;
  const int len = p.cu[b + 1] - p.cu[b];
  const std::int64_t base = (static_cast<std::int64_t>(b) * p.heads + h) * p.chunks * kHeadDim + ch;
  float s = 0.f, a = 0.f;
  for (int c = 0; c < p.chunks; ++c) {
    s += p.part_sum[base + static_cast<std::int64_t>(c) * kHeadDim];
    a = fmaxf(a, p.part_amax[base + static_cast<std::int64_t>(c) * kHeadDim]);
  }
  const std::int64_t at = (static_cast<std::int64_t>(b) * p.heads + h) * kHeadDim + ch;
  p.k_mean[at] = len > 0 ? rbf(s / static_cast<float>(len)) : 0.f;
  p.v_scale[at] = a > 0.f ? a / p.v_range : 1.f;
  p.v_recp[at] = a > 0.f ? p.v_range / a : 1.f;
}

// Q per (32 tokens, head): amax floored at 1e-7, scale = amax / 127, q = rni(x * (127 / amax)). CTA = 32 rows x 16 lanes.
__global__ void __launch_bounds__(512) quant_q_kernel(const PrepArgs p) {
  const int bx = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int lane = static_cast<int>(threadIdx.x) & 15, row = static_cast<int>(threadIdx.x) >> 4;
  const int start = p.cu[b], len = p.cu[b + 1] - start;
  const int t = bx * 32 + row;
  const bool valid = t < len;
  float x[8] = {};
  const std::int64_t tok = static_cast<std::int64_t>(start) + t;
  if (valid) load8(p.q + tok * p.q_row + h * p.q_head + lane * 8, x);
  float amax = 0.0000001f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(x[j]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  __shared__ float s_w[16];
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = s_w[0];
#pragma unroll
  for (int i = 1; i < 16; ++i) amax = fmaxf(amax, s_w[i]);
  if (threadIdx.x == 0) p.q_scale[(static_cast<std::int64_t>(b) * p.heads + h) * p.q_blocks + bx] = amax / 127.0f;
  if (!valid) return;
  const float qs = 127.0f / amax;
  *reinterpret_cast<uint2*>(p.q_i8 + (tok * p.heads + h) * kHeadDim + lane * 8) =
      make_uint2(pack_i8x4(x[0] * qs, x[1] * qs, x[2] * qs, x[3] * qs), pack_i8x4(x[4] * qs, x[5] * qs, x[6] * qs, x[7] * qs));
}

// K and V of one (64 keys, head): K - mean -> int8 with one scale; V * v_recp -> e4m3. CTA = 16 rows x 16 lanes, each
// thread taking keys row, row + 16, row + 32, row + 48 (eight loads in flight per thread, one block-wide maximum).
__global__ void __launch_bounds__(256) quant_kv_kernel(const PrepArgs p) {
  const int bx = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int lane = static_cast<int>(threadIdx.x) & 15, row = static_cast<int>(threadIdx.x) >> 4;
  const int start = p.cu[b], len = p.cu[b + 1] - start;
  const std::int64_t stat = (static_cast<std::int64_t>(b) * p.heads + h) * kHeadDim + lane * 8;
  uint4 kr[4], vr[4];
  bool valid[4];
  std::int64_t tok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = bx * 64 + row + 16 * i;
    valid[i] = t < len;
    tok[i] = static_cast<std::int64_t>(start) + t;
    kr[i] = vr[i] = make_uint4(0, 0, 0, 0);
    if (valid[i]) {
      kr[i] = *reinterpret_cast<const uint4*>(p.k + tok[i] * p.k_row + h * p.k_head + lane * 8);
      vr[i] = *reinterpret_cast<const uint4*>(p.v + tok[i] * p.v_row + h * p.v_head + lane * 8);
    }
  }
  float mean[8], recp[8];
  *reinterpret_cast<float4*>(mean) = *reinterpret_cast<const float4*>(p.k_mean + stat);
  *reinterpret_cast<float4*>(mean + 4) = *reinterpret_cast<const float4*>(p.k_mean + stat + 4);
  *reinterpret_cast<float4*>(recp) = *reinterpret_cast<const float4*>(p.v_recp + stat);
  *reinterpret_cast<float4*>(recp + 4) = *reinterpret_cast<const float4*>(p.v_recp + stat + 4);
  float x[4][8];
  float amax = 0.0000001f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const std::uint32_t w[4] = {kr[i].x, kr[i].y, kr[i].z, kr[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // An absent key contributes 0 (not 0 - mean) to the block maximum.
      x[i][2 * j] = valid[i] ? __uint_as_float(w[j] << 16) - mean[2 * j] : 0.f;
      x[i][2 * j + 1] = valid[i] ? __uint_as_float(w[j] & 0xFFFF0000u) - mean[2 * j + 1] : 0.f;
      amax = fmaxf(amax, fmaxf(fabsf(x[i][2 * j]), fabsf(x[i][2 * j + 1])));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  __shared__ float s_w[8];
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = s_w[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, s_w[i]);
  if (threadIdx.x == 0) p.k_scale[(static_cast<std::int64_t>(b) * p.heads + h) * p.k_blocks + bx] = amax / 127.0f;
  const float ks = 127.0f / amax;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (!valid[i]) continue;
    const std::int64_t o = (tok[i] * p.heads + h) * kHeadDim + lane * 8;
    *reinterpret_cast<uint2*>(p.k_i8 + o) =
        make_uint2(pack_i8x4(x[i][0] * ks, x[i][1] * ks, x[i][2] * ks, x[i][3] * ks),
                   pack_i8x4(x[i][4] * ks, x[i][5] * ks, x[i][6] * ks, x[i][7] * ks));
    const std::uint32_t w[4] = {vr[i].x, vr[i].y, vr[i].z, vr[i].w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __uint_as_float(w[j] << 16) * recp[2 * j];
      v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u) * recp[2 * j + 1];
    }
    *reinterpret_cast<uint2*>(p.v8 + o) = make_uint2(e4m3x4(v[0], v[1], v[2], v[3]), e4m3x4(v[4], v[5], v[6], v[7]));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The attention kernel.
// ---------------------------------------------------------------------------------------------------------------
// The score accumulator as the softmax threads see it. |S| < 2^22, so the integer S + 0x4B400000 is the bit pattern of
// the fp32 number 12582912 + S: the order of those floats is the order of the integers and the constant folds into the
// softmax bias. B2_ATTN_CONST_BIAS = 1 (default) lets the tensor core add the constant: each score accumulator is first
// written by a K = 16 bf16 MMA of two constant operands whose dot product is exactly 12582912.0f (bit pattern
// 0x4B400000), and the INT8 MMAs of Q·K^T then accumulate their exact integers on top of those bits, so a score read
// back from tensor memory already is the float. With 0 the softmax threads add the constant with one integer add per
// score.
#ifndef B2_ATTN_CONST_BIAS
#define B2_ATTN_CONST_BIAS 1
#endif
constexpr std::uint32_t kScoreBits = 0x4B400000u;                       // 12582912.0f
constexpr std::uint32_t kScoreBias = B2_ATTN_CONST_BIAS ? 0u : kScoreBits;  // what a thread still has to add
// Of every 8 scores (4 pairs) this many pairs take 2^x from a polynomial on the FMA pipe instead of the special-function
// unit (0 = none).
#ifndef B2_ATTN_POLY_PAIRS
#define B2_ATTN_POLY_PAIRS 0
#endif

__device__ __forceinline__ std::uint64_t add2_rm(std::uint64_t a, std::uint64_t b) {
  std::uint64_t d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ std::uint64_t sub2(std::uint64_t a, std::uint64_t b) {
  std::uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for a pair without the special-function unit: x = floor(x) + r by a round-down add of 1.5 * 2^23 (whose low
// mantissa bits then hold floor(x)), a cubic for 2^r on [0, 1) (relative error below 1e-4, far inside the e4m3 rounding
// of P), and the integer part added into the exponent field. Inputs below -125 give the result for -125 (< 2^-124: zero
// for every use here).
__device__ __forceinline__ void exp2_poly2(float x0, float x1, float& p0, float& p1) {
  const std::uint64_t magic = pack2(12582912.f, 12582912.f);
  const std::uint64_t x = pack2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const std::uint64_t fl_m = add2_rm(x, magic);
  const std::uint64_t r = sub2(x, sub2(fl_m, magic));
  std::uint64_t p = fma2(pack2(0.0555054f, 0.0555054f), r, pack2(0.2402265f, 0.2402265f));
  p = fma2(p, r, pack2(0.6931472f, 0.6931472f));
  p = fma2(p, r, pack2(1.f, 1.f));
  float q0, q1, f0, f1;
  unpack2(p, q0, q1);
  unpack2(fl_m, f0, f1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(f0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(f1) << 23));
}

// One thread's 64 scores of a sub-tile, as read from tensor memory (four 16-column loads).
struct ScoreRegs {
  std::uint32_t a[16], b[16], c[16], d[16];
};
__device__ __forceinline__ void load_scores(std::uint32_t s_cols, ScoreRegs& r) {  // asynchronous: tmem_ld_wait() before use
  tmem_ld_32x16(s_cols, r.a);
  tmem_ld_32x16(s_cols + 16, r.b);
  tmem_ld_32x16(s_cols + 32, r.c);
  tmem_ld_32x16(s_cols + 48, r.d);
}

// One softmax pass of one thread over its row's 64 scores of a sub-tile, already in registers. P = exp2(f * c + bias)
// with packed fp32 pairs for the FMA and the denominator (f the biased score, the constant folded into `bias`); e4m3 P goes
// into the swizzled P tile (row = 128 bytes, 16-byte chunk n of row r stored at chunk n ^ (r % 8); this sub-tile owns
// chunks chunk0 .. chunk0 + 3). Returns the largest biased score (0 if none) and the sum of the unrounded P.
template <bool kFull>
__device__ __forceinline__ void softmax_pass(const ScoreRegs& s, float c, float bias, int valid, std::uint8_t* prow,
                                             int chunk0, int row_xor, float& bmax_out, float& sum_out) {
  const std::uint64_t c2 = pack2(c, c), bias2 = pack2(bias, bias);
  std::uint64_t dA = pack2(0.f, 0.f), dB = dA;
  float bmax = 0.f;
  const auto chunk = [&](const std::uint32_t (&r)[16], int n) {  // keys 16 n .. 16 n + 15 = one 16-byte chunk of the P row
    float pv[16];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float f0 = __uint_as_float(r[i] + kScoreBias), f1 = __uint_as_float(r[i + 1] + kScoreBias);
      float e0, e1;
      unpack2(fma2(pack2(f0, f1), c2, bias2), e0, e1);
      if (((i >> 1) & 3) < B2_ATTN_POLY_PAIRS) {
        exp2_poly2(e0, e1, pv[i], pv[i + 1]);
      } else {
        pv[i] = ex2(e0);
        pv[i + 1] = ex2(e1);
      }
      if constexpr (kFull) {
        bmax = fmax3(bmax, f0, f1);
      } else {
        const bool in0 = 16 * n + i < valid, in1 = 16 * n + i + 1 < valid;
        bmax = fmax3(bmax, in0 ? f0 : 0.f, in1 ? f1 : 0.f);
        pv[i] = in0 ? pv[i] : 0.f;
        pv[i + 1] = in1 ? pv[i + 1] : 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      dA = add2(dA, pack2(pv[i], pv[i + 1]));
      dB = add2(dB, pack2(pv[i + 2], pv[i + 3]));
    }
    *reinterpret_cast<uint4*>(prow + ((chunk0 + n) ^ row_xor) * 16) =
        make_uint4(e4m3x4(pv[0], pv[1], pv[2], pv[3]), e4m3x4(pv[4], pv[5], pv[6], pv[7]),
                   e4m3x4(pv[8], pv[9], pv[10], pv[11]), e4m3x4(pv[12], pv[13], pv[14], pv[15]));
  };
  chunk(s.a, 0);
  chunk(s.b, 1);
  chunk(s.c, 2);
  chunk(s.d, 3);
  float d0, d1, d2, d3;
  unpack2(dA, d0, d1);
  unpack2(dB, d2, d3);
  bmax_out = bmax;
  sum_out = (d0 + d1) + (d2 + d3);
}

// The largest biased score among the first `valid` of the 64 (0 if none).
__device__ __forceinline__ float max_score(const ScoreRegs& s, int valid) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    m = fmaxf(m, i < valid ? __uint_as_float(s.a[i] + kScoreBias) : 0.f);
    m = fmaxf(m, 16 + i < valid ? __uint_as_float(s.b[i] + kScoreBias) : 0.f);
    m = fmaxf(m, 32 + i < valid ? __uint_as_float(s.c[i] + kScoreBias) : 0.f);
    m = fmaxf(m, 48 + i < valid ? __uint_as_float(s.d[i] + kScoreBias) : 0.f);
  }
  return m;
}

constexpr int kTileQ = 128, kTileK = 128, kSubK = 64;
constexpr int kKvStages = 2;
constexpr int kTileBytes = 128 * 128;
constexpr int kConstBytes = B2_ATTN_CONST_BIAS ? 128 * 32 : 0;  // the constant operand of the score bias: 128 rows of 16 bf16
constexpr int kAttnSmem = kTileBytes * (1 + 2 * kKvStages + 1) + kConstBytes + 1024;  // Q, K/V stages, P, constant, alignment slack
constexpr int kAttnThreads = 192;  // TMA warp, MMA warp, 4 softmax warps
constexpr std::uint32_t kTmemCols = 256;  // S(u % 2): columns [64 (u % 2), +64); O: columns [128, 256)
// Softmax reference maximum: set kHeadroom binades above what the largest P needs, raised again once fewer than kRaise
// binades are left. e4m3 keeps full relative precision over 14 binades below p_range, so three binades of headroom cost
// nothing measurable.
constexpr float kHeadroom = 3.0f, kRaise = 1.0f;

struct AttnArgs {
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  const int* cu_q;
  const int* cu_k;
  __nv_bfloat16* out;
  std::int64_t out_row, out_head;
  int heads, q_blocks, k_blocks;
  float scale_log2;  // sm_scale * log2(e)
  float p_offset;
  // Test hook (kDump instantiation only): the raw integer scores of one (sequence, head, query tile).
  std::int32_t* dump;
  std::int64_t dump_ld;
  int dump_seq, dump_head, dump_tile;
#ifdef B2_ATTN_TRACE
  long long* trace;  // [sub-tile][8] clock64 stamps of CTA (0,0,0), softmax warp 2 lane 0 and the MMA warp
#endif
};

// Shared-memory matrix descriptor of a K-major operand stored as 32-byte rows with the 32-byte swizzle: 8-row groups are
// 256 bytes apart; layout type 6.
__device__ __forceinline__ std::uint64_t umma_desc_sw32(std::uint32_t smem_addr) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<std::uint64_t>(1) << 16;
  d |= static_cast<std::uint64_t>(256 >> 4) << 32;
  d |= static_cast<std::uint64_t>(1) << 46;
  d |= static_cast<std::uint64_t>(6) << 61;
  return d;
}
__device__ __forceinline__ void umma_bf16(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                          std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One CTA per (128 query rows, head, sequence), two CTAs per SM. K and V arrive in 128-key tiles; the tensor work runs in
// 64-key sub-tiles u = 0, 1, ... (one K scale block each) with the score accumulator double-buffered in TMEM, so the MMA
// warp computes S(u + 1) while the softmax warps turn S(u) into P(u):
//   MMA warp      S(u % 2) = [bias constant +] Q · K(u)^T (N = 64), O += P(u % 2) · V(u) (K = 64)
//   softmax warps one thread per query row (TMEM lane), 64 scores per sub-tile: no exchange between threads. A warp's
//                 loop is a chain of latencies (barrier test, tensor-memory load, votes, fences), so it is software
//                 pipelined: the loads of S(u + 1) are issued right after P(u) is handed over and land during the
//                 bookkeeping in between, and the K scale of the next sub-tile is fetched a whole pass ahead.
//   P             e4m3, the two buffers interleaved in one swizzled [128 x 128 B] tile: buffer i = bytes [64 i, +64) of
//                 each row
// kDump: the instantiation behind b2_attention_q8_debug_scores, which also stores one tile's raw integer scores.
template <bool kDump>
__global__ void __launch_bounds__(kAttnThreads, 2)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const AttnArgs a) {
  const int bq = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q_start = a.cu_q[b], qo_len = a.cu_q[b + 1] - q_start;
  const int k_start = a.cu_k[b], kv_len = a.cu_k[b + 1] - k_start;
  const int q0 = bq * kTileQ;
  if (q0 >= qo_len) return;  // uniform per CTA, before any barrier or allocation
  const int warp = static_cast<int>(threadIdx.x) >> 5, lane = static_cast<int>(threadIdx.x) & 31;
  if (kv_len == 0) {
    // No keys: zero output rows.
    const int rows = min(kTileQ, qo_len - q0);
    for (int i = threadIdx.x; i < rows * 16; i += blockDim.x) {
      __nv_bfloat16* o = a.out + static_cast<std::int64_t>(q_start + q0 + i / 16) * a.out_row + h * a.out_head + (i % 16) * 8;
      *reinterpret_cast<uint4*>(o) = make_uint4(0, 0, 0, 0);
    }
    return;
  }

  extern __shared__ std::uint8_t smem_raw[];
  __shared__ __align__(8) std::uint64_t s_q_full, s_k_full[kKvStages], s_k_empty[kKvStages], s_v_full[kKvStages],
      s_v_empty[kKvStages], s_step[2], s_p_full[2], s_s_ready;
  __shared__ std::uint32_t s_tmem_base;
  __shared__ int s_abort;
  const std::uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const std::uint32_t q_smem = base;
  const auto k_smem = [&](int s) { return base + kTileBytes * (1 + s); };
  const auto v_smem = [&](int s) { return base + kTileBytes * (1 + kKvStages + s); };
  const std::uint32_t p_smem = base + kTileBytes * (1 + 2 * kKvStages);
  const std::uint32_t const_smem = p_smem + kTileBytes;
  std::uint8_t* p_generic = smem_raw + (p_smem - smem_u32(smem_raw));

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&s_q_full), 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(smem_u32(&s_k_full[s]), 1);
      mbar_init(smem_u32(&s_k_empty[s]), 1);
      mbar_init(smem_u32(&s_v_full[s]), 1);
      mbar_init(smem_u32(&s_v_empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_step[i]), 1);
      mbar_init(smem_u32(&s_p_full[i]), 4);
    }
    mbar_init(smem_u32(&s_s_ready), 4);
    s_abort = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const std::uint32_t tmem_s = s_tmem_base, tmem_o = s_tmem_base + 128;
  volatile int* abort_word = &s_abort;
  const int n_tiles = (kv_len + kTileK - 1) / kTileK;  // 128-key K/V tiles
  const int n_sub = (kv_len + kSubK - 1) / kSubK;      // 64-key sub-tiles

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&s_q_full), kTileBytes);
      tma_load_2d(q_smem, &map_q, smem_u32(&s_q_full), h * kHeadDim, q_start + q0);
      for (int t = 0; t < n_tiles && *abort_word == 0; ++t) {
        const int s = t % kKvStages;
        const std::uint32_t ph = (t / kKvStages) & 1u;
        if (!wait_bar_relaxed<400>(smem_u32(&s_k_empty[s]), ph ^ 1u, abort_word)) break;
        mbar_expect_tx(smem_u32(&s_k_full[s]), kTileBytes);
        tma_load_2d(k_smem(s), &map_k, smem_u32(&s_k_full[s]), h * kHeadDim, k_start + t * kTileK);
        if (!wait_bar_relaxed<400>(smem_u32(&s_v_empty[s]), ph ^ 1u, abort_word)) break;
        mbar_expect_tx(smem_u32(&s_v_full[s]), kTileBytes);
        tma_load_2d(v_smem(s), &map_v, smem_u32(&s_v_full[s]), h * kHeadDim, k_start + t * kTileK);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // The whole warp walks the loop (uniform control flow, every lane takes the waits); one elected lane issues.
#ifdef B2_ATTN_TRACE
    const bool tracing = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0;
#endif
    constexpr std::uint32_t idesc_qk = umma_idesc(/*s32*/ 2, /*s8*/ 1, /*s8*/ 1, 0, 0, 128, kSubK);
    constexpr std::uint32_t idesc_pv = umma_idesc(/*f32*/ 1, /*e4m3*/ 0, /*e4m3*/ 0, 0, /*B MN-major*/ 1, 128, 128);
    constexpr std::uint32_t idesc_bias = umma_idesc(/*f32*/ 1, /*bf16*/ 1, /*bf16*/ 1, 0, 0, 128, kSubK);
    const std::uint64_t dq = umma_desc_sw128(q_smem), dp = umma_desc_sw128(p_smem);
    const std::uint64_t dconst = umma_desc_sw32(const_smem);
    static_assert(kKvStages == 2, "the descriptors below are selected, not indexed");
    const std::uint64_t dk0 = umma_desc_sw128(k_smem(0)), dk1 = umma_desc_sw128(k_smem(1));
    const std::uint64_t dv0 = umma_desc_sw128(v_smem(0)), dv1 = umma_desc_sw128(v_smem(1));
    // 64 keys = 64 rows of 128 bytes of a K or V tile: 8192 bytes, 512 in the descriptors' 16-byte units.
    constexpr std::uint32_t kHalfTile = 64 * 128 / 16;
    // S(u % 2) = [12582912.0f +] Q · K(u)^T. The K tile goes back to the TMA warp after its second half.
    const auto issue_qk = [&](int u) -> bool {
      const int s = (u >> 1) % kKvStages;
      bool got = true;
      if ((u & 1) == 0) got = wait_bar(smem_u32(&s_k_full[s]), ((u >> 1) / kKvStages) & 1u, abort_word);
      if (__any_sync(0xffffffffu, !got)) return false;
      tc_fence_after();
      if (elect_one()) {
        const std::uint32_t d_s = tmem_s + static_cast<std::uint32_t>(u & 1) * kSubK;
        // The constant operand serves as A (128 rows) and as B (its first 64 rows): every row holds the same 16 values.
        if (B2_ATTN_CONST_BIAS) umma_bf16(d_s, dconst, dconst, idesc_bias, 0u);
        const std::uint64_t d = (s != 0 ? dk1 : dk0) + (u & 1) * kHalfTile;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          umma_i8(d_s, dq + 2u * k4, d + 2u * k4, idesc_qk, (B2_ATTN_CONST_BIAS || k4 != 0) ? 1u : 0u);
        }
        if ((u & 1) != 0 || u + 1 >= n_sub) tc_commit(smem_u32(&s_k_empty[s]));
        if (u < 2) tc_commit(smem_u32(&s_step[u]));  // start-up: S(0) and S(1) are the first completions of the two barriers
      }
      __syncwarp();
      return true;
    };
    bool ok = wait_bar(smem_u32(&s_q_full), 0, abort_word) && wait_bar(smem_u32(&s_s_ready), 0, abort_word);
    ok = !__any_sync(0xffffffffu, !ok);
    tc_fence_after();
#ifdef B2_ATTN_TRACE
    // Tracing only: wait for both K halves' tile first, then time the two start-up issues (the softmax warps are idle).
    if (tracing) a.trace[200 * 16 + 0] = clock64();
#endif
    ok = ok && issue_qk(0);
#ifdef B2_ATTN_TRACE
    if (tracing) a.trace[200 * 16 + 1] = clock64();
#endif
    if (ok && n_sub > 1) ok = issue_qk(1);
#ifdef B2_ATTN_TRACE
    if (tracing) a.trace[200 * 16 + 2] = clock64();
#endif
    for (int u = 0; ok && u < n_sub; ++u) {
      const int s = (u >> 1) % kKvStages;
      bool got = true;
      if ((u & 1) == 0) got = wait_bar(smem_u32(&s_v_full[s]), ((u >> 1) / kKvStages) & 1u, abort_word);
      // The softmax warps have consumed S(u) and written P(u).
      got = got && wait_bar_relaxed<B2_MMA_SLEEP_NS>(smem_u32(&s_p_full[u & 1]), (u >> 1) & 1u, abort_word);
      if (__any_sync(0xffffffffu, !got)) break;
      tc_fence_after();
      TRACE(5);
      if (elect_one()) {
#pragma unroll
        for (int k2 = 0; k2 < 2; ++k2) {
          // P buffer u % 2: bytes [64 (u % 2), +64) of each row, 32 keys = 32 bytes along K inside the swizzle atom (+2);
          // V (MN-major): 32 key rows of 128 bytes (+256 per step), second half of the tile at +kHalfTile.
          umma_f8(tmem_o, dp + 2u * (2 * (u & 1) + k2), (s != 0 ? dv1 : dv0) + (u & 1) * kHalfTile + 256u * k2, idesc_pv,
                  (u | k2) != 0 ? 1u : 0u);
        }
        if ((u & 1) != 0 || u + 1 >= n_sub) tc_commit(smem_u32(&s_v_empty[s]));
      }
      __syncwarp();
      TRACE(6);
      if (u + 2 < n_sub && !issue_qk(u + 2)) break;
      // One completion per step: P·V(u) has landed (its P buffer and O are free again) and S(u + 2) is computed.
      if (elect_one()) tc_commit(smem_u32(&s_step[u & 1]));
      __syncwarp();
      TRACE(7);
#ifdef B2_ATTN_TRACE
      // Tracing only: when the step's MMAs have completed (the warp has nothing else to do until P(u + 1) arrives).
      if (tracing) {
        for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&s_step[u & 1]), ((u >> 1) + 1) & 1u); ++spin) {
        }
        TRACE(15);
      }
#endif
    }
  } else {
    // Softmax: 4 warps, one thread per query row; warp w may touch TMEM lanes [32 (w % 4), +32). One pass per sub-tile:
    // P = exp2(S * c - m) against the reference maximum m carried over from the earlier sub-tiles, while the sub-tile's
    // own maximum is tracked on the side. m is kept kHeadroom binades above what the largest P would need, so scores
    // above everything seen so far still fit; when they do not (P would pass p_range), the warp raises m for those
    // rows, rescales O and the denominator and runs the pass again on the same S.
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;  // row of the tile == TMEM lane
    const std::uint32_t lane_off = static_cast<std::uint32_t>(quarter * 32) << 16;
    const std::int64_t sc_base = static_cast<std::int64_t>(b) * a.heads + h;
    const float qs = a.q_scale[sc_base * a.q_blocks + (q0 + quarter * 32) / 32] * a.scale_log2;
    const float* k_scale = a.k_scale + sc_base * a.k_blocks;
    const int n_scales = min(n_sub, a.k_blocks);
#ifdef B2_ATTN_TRACE
    const bool tracing = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == B2_TRACE_WARP && lane == 0;
#endif
    const bool dumping = kDump && b == a.dump_seq && h == a.dump_head && bq == a.dump_tile;
    constexpr float kNone = -5000000.0f;  // "no score": below every scaled score
    float m_run = kNone, d_run = 0.f;
    float mx_run = kNone;  // the row's largest scaled score so far
    // Rows past the sequence's end hold whatever the tile load brought (the next sequence's queries, or zeros): they follow
    // the warp's raises but never ask for one, so a sequence's output does not depend on its neighbours in the batch.
    const bool row_live = q0 + r_local < qo_len;
    float o_scale = 1.0f;  // factor O still has to be multiplied by (applied once the P·V before it have landed)
    // Bounded wait with one answer for the whole warp (the TMEM accesses that follow are warp-wide).
    const auto warp_wait = [&](std::uint32_t bar, std::uint32_t parity) {
      const bool ok = wait_bar(bar, parity, abort_word);
      return !__any_sync(0xffffffffu, !ok);
    };
    // O (this thread's row, 128 channels) times `factor`, in place.
    const auto rescale_o = [&](float factor) {
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        std::uint32_t r[32];
        tmem_ld_32x32(tmem_o + lane_off + cc * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
        tmem_st_32x32(tmem_o + lane_off + cc * 32, r);
      }
      tmem_st_wait();
    };
    if (B2_ATTN_CONST_BIAS) {
      // This thread's row of the constant operand: 16 bf16 = two identical 16-byte halves (so the 32-byte swizzle, which
      // only swaps the halves, cannot matter) of 2048, 1024, 1024, 0 ...: 2 (2^22 + 2^20 + 2^20) = 12582912 exactly.
      std::uint8_t* crow = smem_raw + (const_smem - smem_u32(smem_raw)) + r_local * 32;
      const uint4 half = make_uint4(0x44804500u, 0x00004480u, 0u, 0u);
      *reinterpret_cast<uint4*>(crow) = half;
      *reinterpret_cast<uint4*>(crow + 16) = half;
      fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&s_s_ready));
    std::uint8_t* prow = p_generic + r_local * 128;
    bool dead = false;  // a bounded wait expired: leave without touching anything else
    ScoreRegs sr;
    float ks_cur = n_scales > 0 ? k_scale[0] : 0.f, ks_next = 0.f;
    // S(0): completion 0 of s_step[0] (the start-up Q·K^T).
    if (!warp_wait(smem_u32(&s_step[0]), 0u)) dead = true;
    if (!dead) {
      tc_fence_after();
      load_scores(tmem_s + lane_off, sr);
    }
    for (int u = 0; !dead && u < n_sub; ++u) {
      // Here S(u) is computed, P·V(u - 2) (which read this sub-tile's P buffer) has landed and the loads of S(u) are in
      // flight.
      const std::uint32_t s_cols = tmem_s + lane_off + static_cast<std::uint32_t>(u & 1) * kSubK;
      TRACE(4);
      const float c = u < n_scales ? qs * ks_cur : 0.f;
      if (u + 1 < n_scales) ks_next = k_scale[u + 1];  // used a whole pass from now
      const int valid = min(kSubK, kv_len - u * kSubK);  // valid keys of this sub-tile (>= 1)
      TRACE(8);
      tmem_ld_wait();
      TRACE(0);
      if constexpr (kDump) {
        if (dumping) {
          std::int32_t* drow = a.dump + static_cast<std::int64_t>(r_local) * a.dump_ld + u * kSubK;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            drow[i] = static_cast<std::int32_t>(sr.a[i] + kScoreBias - kScoreBits);
            drow[16 + i] = static_cast<std::int32_t>(sr.b[i] + kScoreBias - kScoreBits);
            drow[32 + i] = static_cast<std::int32_t>(sr.c[i] + kScoreBias - kScoreBits);
            drow[48 + i] = static_cast<std::int32_t>(sr.d[i] + kScoreBias - kScoreBits);
          }
        }
      }
      if (u == 0) m_run = (max_score(sr, valid) - 12582912.0f) * c - (a.p_offset - kHeadroom);
      bool o_idle = u < 1;  // every P·V up to u - 1 has to land before O is rescaled
      float mx, d_tile;
      for (;;) {
        const float bias = -fmaf(12582912.0f, c, m_run);
        float bmax;
        if (valid == kSubK) {
          softmax_pass<true>(sr, c, bias, valid, prow, 4 * (u & 1), r_local & 7, bmax, d_tile);
        } else {
          softmax_pass<false>(sr, c, bias, valid, prow, 4 * (u & 1), r_local & 7, bmax, d_tile);
        }
        TRACE(1);
        mx = bmax != 0.f ? (bmax - 12582912.0f) * c : kNone;
        const bool over = mx - m_run > a.p_offset;  // some P of this row passed p_range: the pass has to run again
        const bool act = __any_sync(0xffffffffu, over || o_scale != 1.0f);
        TRACE(9);
        if (!act) break;
        // O is about to be rescaled: every P·V issued so far (the last one is u - 1) has to have landed.
        if (!o_idle) {
          o_idle = true;
          if (!warp_wait(smem_u32(&s_step[(u - 1) & 1]), (((u - 1) >> 1) + 1) & 1u)) {  // the MMA warp's step u - 1
            dead = true;
            break;
          }
          tc_fence_after();
        }
        float alpha = o_scale;
        o_scale = 1.0f;
        if (over) {
          const float m_new = mx - (a.p_offset - kHeadroom);
          const float grow = ex2(m_run - m_new);
          m_run = m_new;
          d_run *= grow;
          alpha *= grow;
        }
        if (u > 0) rescale_o(alpha);
        if (!__any_sync(0xffffffffu, over)) break;
        load_scores(s_cols, sr);  // the pass consumed its registers: the scores are still in tensor memory
        tmem_ld_wait();
      }
      if (dead) break;
      d_run += d_tile;
      TRACE(2);
      // S is consumed and P written: both go to the MMA warp.
      fence_proxy_async_smem();
      TRACE(10);
      tc_fence_before();
      __syncwarp();
      TRACE(11);
      if (lane == 0) mbar_arrive(smem_u32(&s_p_full[u & 1]));
      TRACE(3);
      if (u + 1 < n_sub) {
        // Completion (u + 1) / 2 of s_step[(u + 1) % 2]: S(u + 1) computed and P·V(u - 1) landed (the MMA warp's step u - 1;
        // for u + 1 < 2 the start-up Q·K^T). Its loads fly while the bookkeeping below runs.
        if (!warp_wait(smem_u32(&s_step[(u + 1) & 1]), ((u + 1) >> 1) & 1u)) {
          dead = true;
          break;
        }
        TRACE(12);
        tc_fence_after();
        load_scores(tmem_s + lane_off + static_cast<std::uint32_t>((u + 1) & 1) * kSubK, sr);
        TRACE(13);
        // Less than kRaise binades of headroom left: raise the reference for the sub-tiles to come. P·V of this one was
        // computed against the old reference, so O is rescaled after it lands (at the end of the next pass).
        // One row short of headroom raises the reference of every row of the warp whose scores have grown since its last
        // raise: the rescale that follows is the whole warp's anyway (it stalls the CTA's pipeline for about a pass), and
        // rows raised together do not ask for one each later.
        mx_run = fmaxf(mx_run, mx);
        if (__any_sync(0xffffffffu, row_live && mx - m_run > a.p_offset - kRaise)) {
          const float m_new = mx_run - (a.p_offset - kHeadroom);
          if (m_new > m_run) {
            const float grow = ex2(m_run - m_new);
            m_run = m_new;
            d_run *= grow;
            o_scale = grow;
          }
        }
        ks_cur = ks_next;
      }
      TRACE(14);
    }
    if (!dead && warp_wait(smem_u32(&s_step[(n_sub - 1) & 1]), (((n_sub - 1) >> 1) + 1) & 1u)) {  // the last step
      tc_fence_after();
      const float inv_d = rcp_approx(d_run);
      const int row = q0 + r_local;
      __nv_bfloat16* orow = a.out + static_cast<std::int64_t>(q_start + row) * a.out_row + h * a.out_head;
      const float* vs = a.v_scale + sc_base * kHeadDim;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        std::uint32_t r[32];
        tmem_ld_32x32(tmem_o + lane_off + cc * 32, r);
        tmem_ld_wait();
        if (row < qo_len) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[8 * v + i]) * inv_d * __ldg(vs + cc * 32 + 8 * v + i);
            *reinterpret_cast<uint4*>(orow + cc * 32 + 8 * v) =
                make_uint4(pack_bf2(o[0], o[1]), pack_bf2(o[2], o[3]), pack_bf2(o[4], o[5]), pack_bf2(o[6], o[7]));
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (s_abort != 0) {
    if (threadIdx.x == 0) atomicExch(&g_attn_status, 1);
    const std::uint64_t t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(s_tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Host.
// ---------------------------------------------------------------------------------------------------------------
std::size_t align_up(std::size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

b2_attention_layout make_layout(std::int64_t total_q, std::int64_t total_k, int batch, int max_seqlen, int heads, int kv_heads) {
  b2_attention_layout l{};
  const auto n = [](std::int64_t v) { return static_cast<std::size_t>(v); };
  l.padded_k = total_k;
  l.q_blocks = (max_seqlen + 127) / 128 * 4;
  l.k_blocks = (max_seqlen + 63) / 64;
  l.chunks = (max_seqlen + kStatsChunk - 1) / kStatsChunk;
  std::size_t at = 0;
  const auto take = [&](std::size_t bytes) {
    const std::size_t off = at;
    at += align_up(bytes);
    return off;
  };
  l.q_i8 = take(n(total_q) * n(heads) * kHeadDim);
  l.k_i8 = take(n(total_k) * n(kv_heads) * kHeadDim);
  l.v8 = take(n(total_k) * n(kv_heads) * kHeadDim);
  l.q_scale = take(n(batch) * n(heads) * n(l.q_blocks) * 4);
  l.k_scale = take(n(batch) * n(kv_heads) * n(l.k_blocks) * 4);
  l.k_mean = take(n(batch) * n(kv_heads) * kHeadDim * 4);
  l.v_scale = take(n(batch) * n(kv_heads) * kHeadDim * 4);
  l.v_recp = take(n(batch) * n(kv_heads) * kHeadDim * 4);
  l.part_sum = take(n(batch) * n(kv_heads) * n(l.chunks) * kHeadDim * 4);
  l.part_amax = take(n(batch) * n(kv_heads) * n(l.chunks) * kHeadDim * 4);
  l.total = at;
  return l;
}

int check_view(const char* op, const b2_view3* t, const char* name) {
  if (t == nullptr || t->tokens < 0 || t->heads <= 0) return fail_invalid(op, std::string(name) + " must be a bf16 [tokens, heads, 128] view");
  if (t->row_stride % 8 != 0 || t->head_stride % 8 != 0 || !aligned_to(t->data, 16) || (t->tokens > 0 && t->data == nullptr)) {
    return fail_invalid(op, std::string(name) + " needs a 16-byte aligned base and row/head strides that are multiples of 8");
  }
  return B2_OK;
}

// attention_q8::effective_p_range / effective_v_range (attention_q8.cu:184-194): <= 0 picks the variant's default.
float resolve_p(const b2_attention_options& o) { return o.p_range > 0 ? o.p_range : o.variant == B2_ATTENTION_Q8_FP8 ? 112.f : 448.f; }
float resolve_v(const b2_attention_options& o) { return o.v_range > 0 ? o.v_range : o.variant == B2_ATTENTION_Q8_FP8 ? 4.5f : 448.f; }
float p_offset_of(float p_range) { return static_cast<float>(std::floor(std::log2(static_cast<double>(p_range)) * 1000.0) / 1000.0); }
// The nearest e4m3 value (ties to even) of a positive number up to 448.
double e4m3_nearest(double v) {
  if (v <= 0) return 0;
  int e = 0;
  std::frexp(v, &e);                                   // v = f * 2^e, f in [0.5, 1)
  const int exp = std::max(e - 1, -6);                 // normal exponents -6 .. 8; below: subnormal steps of 2^-9
  const double step = std::ldexp(1.0, exp - 3);
  return std::min(448.0, std::nearbyint(v / step) * step);
}

}  // namespace

int attn_status_word(int* host_value) {
  const cudaError_t e = cudaMemcpyFromSymbol(host_value, g_attn_status, sizeof(int));
  return e == cudaSuccess ? B2_OK : fail_cuda("attention_status", e);
}
int attn_status_clear() {
  const int zero = 0;
  const cudaError_t e = cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
  return e == cudaSuccess ? B2_OK : fail_cuda("attention_status", e);
}

}  // namespace b2

using namespace b2;

extern "C" {

int b2_qk_norm_rope_moss(void* qkv, int64_t ld, int64_t tokens, int heads, const void* q_norm, const void* k_norm,
                         const void* table, int64_t table_ld, void* stream) {
  constexpr const char* op = "qk_norm_rope_moss";
  if (tokens < 0 || heads < 1 || ld < 2LL * heads * kHeadDim || table_ld < kHeadDim) {
    return fail_invalid(op, "expected qkv [L, >= 2*heads*128] and table [L, 128]");
  }
  if (tokens == 0) return B2_OK;
  if (qkv == nullptr || table == nullptr || q_norm == nullptr || k_norm == nullptr || !aligned_to(qkv, 16) ||
      !aligned_to(table, 16) || !aligned_to(q_norm, 16) || !aligned_to(k_norm, 16) || ld % 8 != 0 || table_ld % 8 != 0) {
    return fail_invalid(op, "needs 16-byte aligned rows and weights");
  }
  const std::int64_t rows = tokens * heads;
  const NormRopeArgs a{static_cast<__nv_bfloat16*>(qkv), ld, static_cast<const __nv_bfloat16*>(q_norm),
                       static_cast<const __nv_bfloat16*>(k_norm), static_cast<const __nv_bfloat16*>(table), table_ld,
                       tokens, heads, static_cast<float>(rows) / static_cast<float>(rows * kHeadDim)};
  const std::int64_t items = tokens * 2 * heads;
  const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((items + 7) / 8, 148 * 64));
  qk_norm_rope_kernel<<<blocks, 256, 0, as_stream(stream)>>>(a);
  return check_launch(op);
}

int b2_moss_rope_table(void* out, int64_t ld, int height, int width, int text_length, void* stream) {
  constexpr const char* op = "moss_rope_table";
  if (height < 0 || width < 0 || text_length < 0 || ld < 128) return fail_invalid(op, "negative extent or ld < 128");
  const std::int64_t n = static_cast<std::int64_t>(height) * width + text_length;
  if (n == 0) return B2_OK;
  if (out == nullptr) return fail_invalid(op, "null table");
  const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((n * 128 + 255) / 256, 148 * 32));
  rope_table_kernel<<<blocks, 256, 0, as_stream(stream)>>>(static_cast<__nv_bfloat16*>(out), ld, n, height, width, 0.f,
                                                           static_cast<float>(text_length), kBands);
  return check_launch(op);
}

int b2_moss_rope_table_reference(void* out, int64_t ld, int height, int width, int index, void* stream) {
  constexpr const char* op = "moss_rope_table_reference";
  if (height < 1 || width < 1 || index < 0 || index >= (1 << 24) || ld < 128) {
    return fail_invalid(op, "needs a grid of at least 1 x 1, 0 <= index < 2^24 and ld >= 128");
  }
  if (out == nullptr) return fail_invalid(op, "null table");
  const std::int64_t n = static_cast<std::int64_t>(height) * width;
  const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((n * 128 + 255) / 256, 148 * 32));
  rope_table_kernel<<<blocks, 256, 0, as_stream(stream)>>>(static_cast<__nv_bfloat16*>(out), ld, n, height, width,
                                                           static_cast<float>(index + 1), 0.f, kBands);
  return check_launch(op);
}

size_t b2_attention_q8_workspace_bytes(const b2_attention_options* o, int64_t total_q, int64_t total_k, int batch,
                                       int max_seqlen, int num_heads, int num_kv_heads) {
  (void)o;
  return make_layout(total_q, total_k, batch, max_seqlen, num_heads, num_kv_heads).total;
}

int b2_attention_q8_layout(const b2_attention_options* o, int64_t total_q, int64_t total_k, int batch, int max_seqlen,
                           int num_heads, int num_kv_heads, b2_attention_layout* out) {
  (void)o;
  if (out == nullptr) return fail_invalid("attention_q8_layout", "null output");
  *out = make_layout(total_q, total_k, batch, max_seqlen, num_heads, num_kv_heads);
  return B2_OK;
}

namespace {
struct ScoreDump {
  std::int32_t* scores = nullptr;
  std::int64_t ld = 0;
  int seq = 0, head = 0, tile = 0;
};

int attention_impl(const char* op, const b2_attention_options* o, const b2_view3* q, const b2_view3* k, const b2_view3* v,
                   const b2_view3* out, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                   int max_seqlen, float scale, void* workspace, size_t workspace_bytes, void* stream,
                   const b2_qk_norm_rope* norm_rope, const ScoreDump* dump, bool prepass_only = false) {
  if (o == nullptr) return fail_invalid(op, "null options");
  if (const int rc = check_view(op, q, "q")) return rc;
  if (const int rc = check_view(op, k, "k")) return rc;
  if (const int rc = check_view(op, v, "v")) return rc;
  if (!prepass_only) {
    if (const int rc = check_view(op, out, "out")) return rc;
  }
  if (o->variant != B2_ATTENTION_Q8_FP8_F32ACC && o->variant != B2_ATTENTION_Q8_FP8) {
    return fail_status(B2_ERR_NOT_SUPPORTED, op, "only the e4m3 P·V variants (int8_fp8, int8_fp8_f32acc) are built for sm_100a");
  }
  const std::int64_t total_q = q->tokens, heads = q->heads, total_k = k->tokens, kv_heads = k->heads;
  if (v->tokens != total_k || v->heads != kv_heads) return fail_invalid(op, "k and v must both be [total_k, num_kv_heads, 128]");
  if (!prepass_only && (out->tokens != total_q || out->heads != heads)) return fail_invalid(op, "out must have q's shape");
  if (kv_heads != heads) return fail_status(B2_ERR_NOT_SUPPORTED, op, "num_heads must equal num_kv_heads (the DiT's joint attention)");
  if (heads > 65535 || batch > 65535 || batch < 1) return fail_invalid(op, "batch and num_heads must be in [1, 65535]");
  if (cu_seqlens_q == nullptr || cu_seqlens_k == nullptr) return fail_invalid(op, "null cu_seqlens");
  if (max_seqlen <= 0) return fail_invalid(op, "max_seqlen must be positive");
  if (!(std::isfinite(scale) && scale > 0)) return fail_invalid(op, "scale must be finite and positive");
  const float p_range = resolve_p(*o), v_range = resolve_v(*o);
  if (!(std::isfinite(p_range) && p_range <= 448.f && std::isfinite(v_range) && v_range <= 448.f)) {
    return fail_invalid(op, "p_range and v_range must be in (0, 448] (e4m3 max)");
  }
  if (o->variant == B2_ATTENTION_Q8_FP8) {
    // The variant's own rule (attention_q8.cu:255-261): a 64-key partial sum of the largest P and V must stay finite in
    // fp16. Accumulation here is fp32, but a caller's ranges are accepted and refused exactly as the reference does.
    const double p_max = e4m3_nearest(std::exp2(static_cast<double>(p_offset_of(p_range)))), v_max = e4m3_nearest(v_range);
    if (64.0 * p_max * v_max > 65504.0) {
      return fail_invalid(op, "int8_fp8: 64 * e4m3(2^p_offset) * e4m3(v_range) must be <= 65504 with fp16 accumulation");
    }
  }
  if (norm_rope != nullptr) {
    if (norm_rope->q_norm == nullptr || norm_rope->k_norm == nullptr || norm_rope->table == nullptr ||
        !aligned_to(norm_rope->q_norm, 16) || !aligned_to(norm_rope->k_norm, 16) || !aligned_to(norm_rope->table, 16) ||
        norm_rope->table_ld % 8 != 0 || norm_rope->table_ld < kHeadDim) {
      return fail_invalid(op, "norm_rope: q_norm, k_norm and table must be 16-byte aligned bf16 device tensors");
    }
    if (cu_seqlens_k != cu_seqlens_q || k->row_stride != q->row_stride || total_k != total_q) {
      return fail_invalid(op, "norm_rope needs one cu_seqlens tensor and q and k rows of one stride");
    }
  }
  const b2_attention_layout l = make_layout(total_q, total_k, batch, max_seqlen, static_cast<int>(heads), static_cast<int>(kv_heads));
  if (total_q * heads * kHeadDim >= (1LL << 32) || total_k * heads * kHeadDim >= (1LL << 32)) return fail_invalid(op, "too many tokens");
  if (total_q == 0) return B2_OK;
  if (workspace == nullptr || !aligned_to(workspace, kAlign) || workspace_bytes < l.total) {
    return fail_invalid(op, "workspace too small or not 256-byte aligned (need " + std::to_string(l.total) + " bytes)");
  }
  cudaStream_t st = as_stream(stream);
  auto* base = static_cast<std::uint8_t*>(workspace);
  PrepArgs p{};
  p.q = static_cast<const __nv_bfloat16*>(q->data), p.k = static_cast<__nv_bfloat16*>(k->data);
  p.v = static_cast<const __nv_bfloat16*>(v->data);
  p.q_row = q->row_stride, p.q_head = q->head_stride, p.k_row = k->row_stride, p.k_head = k->head_stride;
  p.v_row = v->row_stride, p.v_head = v->head_stride;
  p.cu = cu_seqlens_k;
  p.batch = batch, p.heads = static_cast<int>(heads), p.max_seqlen = max_seqlen;
  p.chunks = l.chunks, p.q_blocks = l.q_blocks, p.k_blocks = l.k_blocks;
  p.v_range = v_range;
  p.q_i8 = reinterpret_cast<std::int8_t*>(base + l.q_i8);
  p.k_i8 = reinterpret_cast<std::int8_t*>(base + l.k_i8);
  p.v8 = base + l.v8;
  p.q_scale = reinterpret_cast<float*>(base + l.q_scale);
  p.k_scale = reinterpret_cast<float*>(base + l.k_scale);
  p.k_mean = reinterpret_cast<float*>(base + l.k_mean);
  p.v_scale = reinterpret_cast<float*>(base + l.v_scale);
  p.v_recp = reinterpret_cast<float*>(base + l.v_recp);
  p.part_sum = reinterpret_cast<float*>(base + l.part_sum);
  p.part_amax = reinterpret_cast<float*>(base + l.part_amax);
  const dim3 stats_grid(l.chunks, static_cast<unsigned>(heads), batch);
  if (norm_rope != nullptr) {
    const std::int64_t rows = total_q * heads;
    p.q_norm = static_cast<const __nv_bfloat16*>(norm_rope->q_norm);
    p.k_norm = static_cast<const __nv_bfloat16*>(norm_rope->k_norm);
    p.table = static_cast<const __nv_bfloat16*>(norm_rope->table);
    p.table_row = norm_rope->table_ld;
    p.norm_factor = static_cast<float>(rows) / static_cast<float>(rows * kHeadDim);
    norm_rope_quant_q_kernel<<<dim3(l.q_blocks, static_cast<unsigned>(heads), batch), 512, 0, st>>>(p);
    if (const int rc = check_launch(op)) return rc;
  }
  stats_kernel<<<stats_grid, 256, 0, st>>>(p);
  if (const int rc = check_launch(op)) return rc;
  finalize_kernel<<<dim3(static_cast<unsigned>(heads), batch), kHeadDim, 0, st>>>(p);
  if (const int rc = check_launch(op)) return rc;
  if (norm_rope == nullptr) {
    PrepArgs pq = p;
    pq.cu = cu_seqlens_q;
    quant_q_kernel<<<dim3(l.q_blocks, static_cast<unsigned>(heads), batch), 512, 0, st>>>(pq);
    if (const int rc = check_launch(op)) return rc;
  }
  quant_kv_kernel<<<dim3(l.k_blocks, static_cast<unsigned>(heads), batch), 256, 0, st>>>(p);
  if (const int rc = check_launch(op)) return rc;
  if (prepass_only) return B2_OK;

  CUtensorMap map_q, map_k, map_v;
  const std::uint64_t row_bytes = static_cast<std::uint64_t>(heads) * kHeadDim;
  if (!make_tensor_map_2d(&map_q, p.q_i8, row_bytes, static_cast<std::uint64_t>(total_q), row_bytes, 128, 128, op) ||
      !make_tensor_map_2d(&map_k, p.k_i8, row_bytes, static_cast<std::uint64_t>(total_k), row_bytes, 128, 128, op) ||
      !make_tensor_map_2d(&map_v, p.v8, row_bytes, static_cast<std::uint64_t>(total_k), row_bytes, 128, 128, op)) {
    return B2_ERR_CUDA;
  }
  AttnArgs a{};
  a.q_scale = p.q_scale, a.k_scale = p.k_scale, a.v_scale = p.v_scale;
  a.cu_q = cu_seqlens_q, a.cu_k = cu_seqlens_k;
  a.out = static_cast<__nv_bfloat16*>(out->data), a.out_row = out->row_stride, a.out_head = out->head_stride;
  a.heads = static_cast<int>(heads), a.q_blocks = l.q_blocks, a.k_blocks = l.k_blocks;
  a.scale_log2 = scale * 1.44269504088896340736f;
  a.p_offset = p_offset_of(p_range);
  if (dump != nullptr) {
    a.dump = dump->scores, a.dump_ld = dump->ld;
    a.dump_seq = dump->seq, a.dump_head = dump->head, a.dump_tile = dump->tile;
  }
#ifdef B2_ATTN_TRACE
  {
    void* tp = nullptr;
    cudaGetSymbolAddress(&tp, g_attn_trace);
    a.trace = static_cast<long long*>(tp);
  }
#endif
  const auto kernel = dump != nullptr ? attention_kernel<true> : attention_kernel<false>;
  if (const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
      e != cudaSuccess) {
    return fail_cuda(op, e);
  }
  const dim3 grid((max_seqlen + kTileQ - 1) / kTileQ, static_cast<unsigned>(heads), batch);
  kernel<<<grid, kAttnThreads, kAttnSmem, st>>>(map_q, map_k, map_v, a);
  return check_launch(op);
}
}  // namespace

int b2_attention_q8(const b2_attention_options* o, const b2_view3* q, const b2_view3* k, const b2_view3* v,
                    const b2_view3* out, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                    int max_seqlen, float scale, void* workspace, size_t workspace_bytes, void* stream,
                    const b2_qk_norm_rope* norm_rope) {
  return attention_impl("attention_q8", o, q, k, v, out, cu_seqlens_q, cu_seqlens_k, batch, max_seqlen, scale, workspace,
                        workspace_bytes, stream, norm_rope, nullptr);
}

int b2_attention_q8_preprocess(const b2_attention_options* o, const b2_view3* q, const b2_view3* k, const b2_view3* v,
                               const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch, int max_seqlen,
                               void* workspace, size_t workspace_bytes, void* stream, const b2_qk_norm_rope* norm_rope) {
  return attention_impl("attention_q8_preprocess", o, q, k, v, nullptr, cu_seqlens_q, cu_seqlens_k, batch, max_seqlen, 1.0f,
                        workspace, workspace_bytes, stream, norm_rope, nullptr, true);
}

int b2_attention_q8_debug_scores(const b2_attention_options* o, const b2_view3* q, const b2_view3* k, const b2_view3* v,
                                 const b2_view3* out, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int batch,
                                 int max_seqlen, float scale, void* workspace, size_t workspace_bytes, void* stream,
                                 const b2_qk_norm_rope* norm_rope, int seq, int head, int tile_q, int32_t* scores,
                                 int64_t ld) {
  constexpr const char* op = "attention_q8_debug_scores";
  if (scores == nullptr || seq < 0 || seq >= batch || head < 0 || tile_q < 0 || ld < (static_cast<std::int64_t>(max_seqlen) + 63) / 64 * 64) {
    return fail_invalid(op, "needs a scores buffer with ld >= 64 * ceil(max_seqlen / 64) and a (seq, head, tile_q) inside the problem");
  }
  const ScoreDump dump{scores, ld, seq, head, tile_q};
  return attention_impl(op, o, q, k, v, out, cu_seqlens_q, cu_seqlens_k, batch, max_seqlen, scale, workspace, workspace_bytes,
                        stream, norm_rope, &dump);
}

#ifdef B2_ATTN_TRACE
int b2_attention_trace(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_attn_trace, sizeof(long long) * n) == cudaSuccess ? 0 : -8;
}
#endif

}  // extern "C"
