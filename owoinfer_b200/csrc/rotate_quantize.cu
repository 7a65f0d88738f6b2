// Activation quantisers of the quantized DiT block: ConvRot rotation (x · H256 per 256-column group) + per-token INT8 or
// INT4 quantisation, optionally preceded by the MOSS RMSNorm + adaLN modulate, plus the small int4 -> int8 helpers
// (unpack, grouped decode). HBM-bound element-wise work: 128-bit global accesses, rows held in registers between the
// absmax pass and the quantise pass, shared memory only for the 16 x 16 digit transpose.
//
// Numerics (bit for bit those of the reference engine, src/kernels/quant/quant.h:4-23, src/kernels/quant4/quant4.h:1-24):
//   rotation     four radix-4 stages over the base-4 digits of the in-group index, each output
//                0.5 * (((m0' + m1') + m2') + m3') with operand 3 - d negated, single-rounded fp32; then rounded to bf16
//   INT8         s = max(min(amax, bf16max) * fp32(1/127), 1e-30); q = clamp(rne(bf16(x_rot / bf16(s))), -128, 127)
//   INT4         amax_bf = bf16(max(min(amax, bf16max), 1e-10)); s = bf16(amax_bf * fp32(1/7));
//                q = clamp(rne(bf16(x_rot / s)), -7, 7), two per byte, even column in the low nibble
//   norm         r = rsqrtf(mean(x^2) + 1e-6) with the mean summed in torch's reduce order for an [m, k] input;
//                y = bf16(bf16(bf16(bf16(x*r)*w) * bf16(1+scale)) + shift)
// The rotation first runs without its four factors 0.5 (results 16 x the reference's, bit for bit, while nothing
// overflows; the power of two is folded into the quantisation multiplier); a row whose scaled maximum is not a finite
// number below 2^126 is read again and rotated with the factors in place, so overflow, inf and NaN rows follow the
// reference exactly.
// The division x_rot / s of two bf16 values is computed as x_rot * (1/s): the exact quotient of two 8-bit significands
// is never within 2^-17 (relative) of a bf16 rounding boundary, so the bf16 rounding of the product equals the
// bf16 rounding of the correctly rounded fp32 quotient; infinities, NaN and zeros propagate identically.
#include <algorithm>
#include <string>
#include <type_traits>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int kGroup = 256;
constexpr int kMaxK = 32768;
constexpr int kTileStride = 17;                  // floats per row of the 16 x 16 transpose tile (conflict-free)
constexpr int kTileFloats = 16 * kTileStride;
constexpr float kBf16Max = 3.38953139e38f;

struct Args {
  const __nv_bfloat16* x;
  std::int64_t ldx;
  void* q;            // int8 [m, k] or packed int4 [m, k/2]
  std::int64_t ldq;   // bytes
  float* scale;
  int k;
  const __nv_bfloat16* weight;
  const __nv_bfloat16* mod_scale;
  const __nv_bfloat16* mod_shift;
  __nv_bfloat16* y;
  std::int64_t ldy;
  float factor;  // float(m) / float(m * k)
  int bw;        // torch's threads per row for this (m, k)
  // Column-chunked input (0 = off): columns [i * chunk_w, (i + 1) * chunk_w) of every row live in chunk i, a [m, chunk_w]
  // matrix of row stride ldx that starts chunk_stride elements after chunk i - 1. chunk_w % 16 == 0 (a lane's 16
  // elements stay inside one chunk).
  int chunk_w;
  std::int64_t chunk_stride;
};

// Radix-4 butterfly on four operands in digit order. kHalve = false leaves the factor 0.5 out: the outputs are then twice
// the reference's, exactly (a power-of-two factor commutes with every fp32 rounding as long as nothing overflows or goes
// subnormal), and a whole rotation comes out 16 times too large.
template <bool kHalve>
__device__ __forceinline__ void butterfly4(float& a, float& b, float& c, float& d) {
  const float s = fadd(a, b), t = fadd(a, -b);
  float y0 = fadd(fadd(s, c), -d), y1 = fadd(fadd(s, -c), d), y2 = fadd(fadd(t, c), d), y3 = fadd(fadd(-t, c), d);
  if constexpr (kHalve) y0 = fmul(0.5f, y0), y1 = fmul(0.5f, y1), y2 = fmul(0.5f, y2), y3 = fmul(0.5f, y3);
  a = y0, b = y1, c = y2, d = y3;
}
// The two stages whose digits are the low and high 2 bits of the register index.
template <bool kHalve>
__device__ __forceinline__ void stages_on_registers(float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 16; i += 4) butterfly4<kHalve>(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
  for (int i = 0; i < 4; ++i) butterfly4<kHalve>(v[i], v[i + 4], v[i + 8], v[i + 12]);
}
// max(a, |b|, |c|) that returns NaN when any operand is NaN.
__device__ __forceinline__ float max3_abs_nan(float a, float b, float c) {
  float r;
  asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c)));
  return r;
}
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 lo = reinterpret_cast<const uint4*>(p)[0], hi = reinterpret_cast<const uint4*>(p)[1];
  const std::uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
// Sixteen bf16 values as eight packed pairs (element 2i in the low half of word i).
__device__ __forceinline__ void load16_packed(const __nv_bfloat16* p, std::uint32_t (&w)[8]) {
  const uint4 lo = reinterpret_cast<const uint4*>(p)[0], hi = reinterpret_cast<const uint4*>(p)[1];
  w[0] = lo.x, w[1] = lo.y, w[2] = lo.z, w[3] = lo.w, w[4] = hi.x, w[5] = hi.y, w[6] = hi.z, w[7] = hi.w;
}
// Packed bf16 pairs: a * b and a + b, each result rounded once to bf16.
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
__device__ __forceinline__ void store16_bf16(__nv_bfloat16* p, const float (&v)[16]) {
  std::uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const std::uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Sum of squares of one row in the order of torch's reduce kernel with `bw` cooperating threads (a power of two,
// 32..512), executed by one warp: lane l plays torch threads l, l + 32, ...; `part` is bw floats of shared memory.
__device__ float torch_order_sum_squares(const __nv_bfloat16* xr, int k, int bw, float* part, int lane) {
  for (int t = lane; t < bw; t += 32) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int idx = t; idx * 4 + 3 < k; idx += bw) {
      const uint2 raw = *reinterpret_cast<const uint2*>(xr + idx * 4);
      const float e0 = __uint_as_float(raw.x << 16), e1 = __uint_as_float(raw.x & 0xFFFF0000u);
      const float e2 = __uint_as_float(raw.y << 16), e3 = __uint_as_float(raw.y & 0xFFFF0000u);
      a0 = fadd(a0, fmul(e0, e0));
      a1 = fadd(a1, fmul(e1, e1));
      a2 = fadd(a2, fmul(e2, e2));
      a3 = fadd(a3, fmul(e3, e3));
    }
    part[t] = fadd(fadd(fadd(a0, a1), a2), a3);
  }
  __syncwarp();
  for (int off = bw / 2; off >= 32; off >>= 1) {
    for (int t = lane; t < off; t += 32) part[t] = fadd(part[t], part[t + off]);
    __syncwarp();
  }
  float s = part[lane];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s = fadd(s, __shfl_down_sync(0xffffffffu, s, off));
  return __shfl_sync(0xffffffffu, s, 0);
}

// One thread block per row. A half-warp owns one 256-group at a time, 16 elements per lane; half-warp i takes groups
// i, i + halves, ... (kSlots of them, kept in registers across the row-wide absmax).
//   load layout  : lane h holds elements 16 h + j  -> register index j carries digits d0, d1
//   after the 16 x 16 transpose: element h + 16 j  -> register index j carries digits d2, d3
// The quantised bytes are scattered into a 256-byte shared tile in natural order, so each lane stores 16 (INT8) or 8
// (INT4) contiguous bytes.
template <int kSlots, bool kNorm, bool kInt4>
__global__ void __launch_bounds__(kSlots == 1 ? 256 : 512, kSlots == 1 ? (kNorm ? 8 : 6) : 1) rotate_quantize_kernel(const Args a) {
  extern __shared__ float smem_f[];
  __shared__ float s_warp_max[2][16];
  __shared__ float s_inv_rms;
  __shared__ float s_part[512];
  const int tid = static_cast<int>(threadIdx.x), lane = tid & 31, warp = tid >> 5;
  const int halves = static_cast<int>(blockDim.x) >> 4, half_id = tid >> 4, h = tid & 15;
  const int groups = a.k / kGroup;
  const std::int64_t row = blockIdx.x;
  const __nv_bfloat16* xr = a.x + row * a.ldx;
  float* tile = smem_f + half_id * kTileFloats;
  std::uint8_t* qtile = reinterpret_cast<std::uint8_t*>(smem_f + halves * kTileFloats) + half_id * kGroup;

  float v[kSlots][16];
  const auto load_row = [&] {
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      const int g = half_id + s * halves;
      if (g < groups) {
        const int col = g * kGroup + 16 * h;
        const __nv_bfloat16* src = a.chunk_w == 0 ? xr + col
                                                  : a.x + (col / a.chunk_w) * a.chunk_stride + row * a.ldx + col % a.chunk_w;
        load16_bf16(src, v[s]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[s][j] = 0.f;
      }
    }
  };
  load_row();

  if constexpr (kNorm) {
    if constexpr (kSlots == 1) {
      // The squares go through shared memory (the transpose tiles, not yet in use, hold a whole row when every half-warp
      // has one group), so that torch's 4 * bw accumulator chains run on as many threads instead of on one warp.
      float* sq = smem_f;
      if (half_id < groups) {
        float4* dst = reinterpret_cast<float4*>(sq + half_id * kGroup + 16 * h);
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          dst[j >> 2] = make_float4(fmul(v[0][j], v[0][j]), fmul(v[0][j + 1], v[0][j + 1]), fmul(v[0][j + 2], v[0][j + 2]),
                                    fmul(v[0][j + 3], v[0][j + 3]));
        }
      }
      __syncthreads();
      // Chain (t, c) = torch thread t's accumulator c: elements 4 * (t + bw * i) + c, i = 0, 1, ... in order.
      for (int ct = tid; ct < 4 * a.bw; ct += static_cast<int>(blockDim.x)) {
        float acc = 0.f;
        for (int e = ct; e < a.k; e += 4 * a.bw) acc = fadd(acc, sq[e]);
        const float a1 = __shfl_down_sync(0xffffffffu, acc, 1), a2 = __shfl_down_sync(0xffffffffu, acc, 2);
        const float a3 = __shfl_down_sync(0xffffffffu, acc, 3);
        if ((ct & 3) == 0) s_part[ct >> 2] = fadd(fadd(fadd(acc, a1), a2), a3);
      }
      __syncthreads();
      if (warp == 0) {
        for (int off = a.bw / 2; off >= 32; off >>= 1) {
          for (int t = lane; t < off; t += 32) s_part[t] = fadd(s_part[t], s_part[t + off]);
          __syncwarp();
        }
        float ss = s_part[lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss = fadd(ss, __shfl_down_sync(0xffffffffu, ss, off));
        if (lane == 0) s_inv_rms = rsqrtf(fadd(fmul(ss, a.factor), 1e-6f));
      }
    } else if (warp == 0) {
      const float ss = torch_order_sum_squares(xr, a.k, a.bw, s_part, lane);
      if (lane == 0) s_inv_rms = rsqrtf(fadd(fmul(ss, a.factor), 1e-6f));
    }
    __syncthreads();
  }
  // The norm + modulate prologue on the registers (a no-op without it); `store_y` also writes the optional bf16 copy.
  const auto prologue = [&](bool store_y) {
    if constexpr (!kNorm) return;
    const float r = s_inv_rms;
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      const int g = half_id + s * halves;
      if (g >= groups) continue;
      const int c0 = g * kGroup + 16 * h;
      // bf16(bf16(bf16(bf16(x*r)*w) * bf16(1+scale)) + shift). After the first rounding every operand is a bf16 value, so
      // the three remaining steps run on packed pairs (mul.rn / add.rn.bf16x2 round once, exactly as the fp32 operation
      // followed by a rounding to bf16 does for bf16 operands).
      std::uint32_t w[8], sc[8], sh[8];
      load16_packed(a.weight + c0, w);
      load16_packed(a.mod_scale + c0, sc);
      load16_packed(a.mod_shift + c0, sh);
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const __nv_bfloat162 n0 = __floats2bfloat162_rn(fmul(v[s][j], r), fmul(v[s][j + 1], r));
        std::uint32_t n = *reinterpret_cast<const std::uint32_t*>(&n0);
        n = bmul2(n, w[j >> 1]);
        n = bmul2(n, badd2(0x3F803F80u, sc[j >> 1]));  // 1.0 in both halves
        n = badd2(n, sh[j >> 1]);
        v[s][j] = __uint_as_float(n << 16);
        v[s][j + 1] = __uint_as_float(n & 0xFFFF0000u);
      }
      if (store_y && a.y != nullptr) store16_bf16(a.y + row * a.ldy + c0, v[s]);
    }
  };
  prologue(true);

  // The rotation, the rounding to bf16 and the row's absolute maximum. kExact = false is the fast form: no factor 0.5 in
  // the butterflies, so the rotated values (and the maximum) are 16 times the reference's, bit for bit, provided nothing
  // overflowed on the way; its maximum propagates NaN, so that an overflow (which always ends in an inf or a NaN) or a
  // non-finite input shows in it. kExact = true follows the reference literally (fmaxf, which skips NaN).
  const auto rotate = [&](auto exact_tag, int slot) -> float {
    constexpr bool kExact = decltype(exact_tag)::value;
    float amax = 0.f;
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      // Warp-uniform: both halves of a warp transpose together (an idle half runs on zeros).
      if ((half_id & ~1) + s * halves >= groups) continue;
      stages_on_registers<kExact>(v[s]);
#pragma unroll
      for (int j = 0; j < 16; ++j) tile[h * kTileStride + j] = v[s][j];
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 16; ++j) v[s][j] = tile[j * kTileStride + h];
      __syncwarp();
      stages_on_registers<kExact>(v[s]);
      if (half_id + s * halves < groups) {
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          rbf2(v[s][j], v[s][j + 1]);
          if constexpr (kExact) amax = fmaxf(amax, fmaxf(fabsf(v[s][j]), fabsf(v[s][j + 1])));
          else amax = max3_abs_nan(amax, v[s][j], v[s][j + 1]);
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float o = __shfl_xor_sync(0xffffffffu, amax, off);
      amax = kExact ? fmaxf(amax, o) : max_nan(amax, o);
    }
    if (lane == 0) s_warp_max[slot][warp] = amax;
    __syncthreads();
    amax = s_warp_max[slot][0];
    for (int w = 1; w < (static_cast<int>(blockDim.x) >> 5); ++w) {
      amax = kExact ? fmaxf(amax, s_warp_max[slot][w]) : max_nan(amax, s_warp_max[slot][w]);
    }
    return amax;
  };
  float amax = rotate(std::false_type{}, 0);
  float unscale = 0.0625f;  // the rotated values in registers are 16 x the reference's
  if (!(amax < 8.5e37f)) {  // 2^126: an overflow, a NaN or an inf somewhere (same answer in every thread of the row)
    load_row();
    prologue(false);
    amax = rotate(std::true_type{}, 1);
    unscale = 1.0f;
  } else {
    amax = fmul(amax, 0.0625f);
  }

  float s_bf;
  if constexpr (kInt4) {
    const float amax_bf = rbf(fmaxf(fminf(amax, kBf16Max), 1e-10f));
    s_bf = rbf(fmul(amax_bf, 1.0f / 7.0f));
    if (tid == 0) a.scale[row] = s_bf;
  } else {
    const float s = fmaxf(fmul(fminf(amax, kBf16Max), 1.0f / 127.0f), 1e-30f);
    if (tid == 0) a.scale[row] = s;
    s_bf = rbf(s);
  }
  // x_rot * (1 / s) with x_rot = unscale * (register value): the power of two moves into the reciprocal, exactly.
  const float inv_s = fmul(__frcp_rn(s_bf), unscale);
  constexpr float kLo = kInt4 ? -7.f : -128.f, kHi = kInt4 ? 7.f : 127.f;
  std::uint8_t* qr = static_cast<std::uint8_t*>(a.q) + row * a.ldq;
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
    if ((half_id & ~1) + s * halves >= groups) continue;
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      // Clamp, then round to nearest even: the bounds are integers, so this equals rounding first. fmaxf sends NaN to
      // the lower bound, infinities saturate. Adding 1.5 * 2^23 rounds to an integer (ties to even) and leaves its two's
      // complement in the low mantissa bits, whose low byte is the int8 code.
      float a = fmul(v[s][j], inv_s), b = fmul(v[s][j + 1], inv_s);
      rbf2(a, b);
      a = fadd(fminf(kHi, fmaxf(kLo, a)), 12582912.0f);
      b = fadd(fminf(kHi, fmaxf(kLo, b)), 12582912.0f);
      qtile[h + 16 * j] = static_cast<std::uint8_t>(__float_as_uint(a));
      qtile[h + 16 * (j + 1)] = static_cast<std::uint8_t>(__float_as_uint(b));
    }
    __syncwarp();
    const uint4 bytes = *reinterpret_cast<const uint4*>(qtile + 16 * h);
    __syncwarp();
    const int g = half_id + s * halves;
    if (g < groups) {
      if constexpr (kInt4) {
        const std::uint32_t w[4] = {bytes.x, bytes.y, bytes.z, bytes.w};
        std::uint32_t out[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const std::uint32_t lo = w[2 * i], hi = w[2 * i + 1];
          // bytes b0..b3 -> nibbles (b0 | b1 << 4), (b2 | b3 << 4)
          const std::uint32_t p0 = (lo & 0xF) | ((lo >> 4) & 0xF0), p1 = ((lo >> 16) & 0xF) | ((lo >> 20) & 0xF0);
          const std::uint32_t p2 = (hi & 0xF) | ((hi >> 4) & 0xF0), p3 = ((hi >> 16) & 0xF) | ((hi >> 20) & 0xF0);
          out[i] = p0 | (p1 << 8) | (p2 << 16) | (p3 << 24);
        }
        *reinterpret_cast<uint2*>(qr + g * (kGroup / 2) + 8 * h) = make_uint2(out[0], out[1]);
      } else {
        *reinterpret_cast<uint4*>(qr + g * kGroup + 16 * h) = bytes;
      }
    }
  }
}

int torch_reduce_threads(std::int64_t rows, std::int64_t d) {
  const auto last_pow2 = [](std::int64_t n) {
    std::int64_t p = 1;
    while (p * 2 <= n) p *= 2;
    return p;
  };
  constexpr std::int64_t kMax = 512;
  const std::int64_t dim0 = d / 4 < kMax ? last_pow2(d / 4) : kMax;
  const std::int64_t dim1 = rows < kMax ? last_pow2(rows) : kMax;
  std::int64_t bw = std::min<std::int64_t>(dim0, 32);
  const std::int64_t bh = std::min(dim1, kMax / bw);
  bw = std::min(dim0, kMax / bh);
  if ((d + bw - 1) / bw >= std::min<std::int64_t>(bh * 16, 256)) return 0;
  return static_cast<int>(bw);
}

template <bool kNorm, bool kInt4>
int launch(const char* op, const Args& a, std::int64_t m, cudaStream_t stream) {
  const int groups = a.k / kGroup;
  // Groups per half-warp so that a row needs at most 16 half-warps when one slot suffices, else up to 32.
  int slots = 1;
  while (slots < 4 && (groups + slots - 1) / slots > (slots == 1 ? 16 : 32)) slots *= 2;
  if (groups == 48) slots = 3;  // k = 12288: 16 half-warps x 3
  int halves = (groups + slots - 1) / slots;
  halves = (halves + 1) & ~1;
  const unsigned threads = static_cast<unsigned>(halves * 16);
  const std::size_t smem = static_cast<std::size_t>(halves) * (kTileFloats * sizeof(float) + kGroup);
  const dim3 grid(static_cast<unsigned>(m));
  switch (slots) {
    case 1: rotate_quantize_kernel<1, kNorm, kInt4><<<grid, threads, smem, stream>>>(a); break;
    case 2: rotate_quantize_kernel<2, kNorm, kInt4><<<grid, threads, smem, stream>>>(a); break;
    case 3: rotate_quantize_kernel<3, kNorm, kInt4><<<grid, threads, smem, stream>>>(a); break;
    default: rotate_quantize_kernel<4, kNorm, kInt4><<<grid, threads, smem, stream>>>(a); break;
  }
  return check_launch(op);
}

int check_common(const char* op, const void* x, std::int64_t ldx, const void* q, std::int64_t ldq, const float* scale,
                 std::int64_t m, int k, bool int4) {
  if (k <= 0 || k % kGroup != 0 || k > kMaxK) {
    return fail_invalid(op, "k must be a positive multiple of 256 up to 32768, got " + std::to_string(k));
  }
  if (m < 0) return fail_invalid(op, "negative row count");
  if (m > 0x7fffffff) return fail_invalid(op, "too many rows");
  if (m > 0 && (x == nullptr || q == nullptr || scale == nullptr)) return fail_invalid(op, "null operand");
  const std::int64_t qcols = int4 ? k / 2 : k;
  if (ldx < k || ldq < qcols || ldx % 8 != 0 || ldq % 16 != 0 || !aligned_to(x, 16) || !aligned_to(q, 16)) {
    return fail_invalid(op, "needs 16-byte aligned x and q with ldx >= k, ldq >= row bytes, ldx % 8 == 0 and ldq % 16 == 0 (k " +
                                std::to_string(k) + ", ldx " + std::to_string(ldx) + ", ldq " + std::to_string(ldq) + ")");
  }
  return B2_OK;
}

int check_norm(const char* op, const void* w, const void* sc, const void* sh, std::int64_t m, int k, int* bw) {
  if (w == nullptr || sc == nullptr || sh == nullptr || !aligned_to(w, 16) || !aligned_to(sc, 16) || !aligned_to(sh, 16)) {
    return fail_invalid(op, "norm_weight, mod_scale and mod_shift must be 16-byte aligned device vectors");
  }
  *bw = 32;
  if (m > 0) {
    *bw = torch_reduce_threads(m, k);
    if (*bw == 0) return fail_invalid(op, "row length " + std::to_string(k) + " needs torch's cross-warp split, not supported");
  }
  return B2_OK;
}

// ------------------------------------------------------------------------------------------------ int4 helpers

// 32 values per thread: 16 packed bytes in, 32 bytes out. Signed nibbles, even column in the low nibble.
__global__ void unpack_int4_kernel(const std::uint8_t* packed, std::int64_t ldp, std::int8_t* out, std::int64_t ldo,
                                   std::int64_t rows, int chunks_per_row) {
  const std::int64_t total = rows * chunks_per_row;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const std::int64_t r = i / chunks_per_row;
    const int c = static_cast<int>(i % chunks_per_row);
    const uint4 in = *reinterpret_cast<const uint4*>(packed + r * ldp + 16 * c);
    const std::uint32_t w[4] = {in.x, in.y, in.z, in.w};
    std::uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // Sign-extend each nibble into its own byte: shift to the top of the byte, arithmetic shift back (per byte).
      const std::uint32_t lo = (w[j] << 4) & 0xF0F0F0F0u, hi = w[j] & 0xF0F0F0F0u;
      // bytes of lo/hi hold nibble << 4; __vshr-like per-byte arithmetic shift via sign mask.
      const std::uint32_t lo_s = ((lo >> 4) & 0x0F0F0F0Fu) | (((lo >> 7) & 0x01010101u) * 0xF0u);
      const std::uint32_t hi_s = ((hi >> 4) & 0x0F0F0F0Fu) | (((hi >> 7) & 0x01010101u) * 0xF0u);
      // interleave: out bytes = lo0, hi0, lo1, hi1 | lo2, hi2, lo3, hi3
      o[2 * j] = __byte_perm(lo_s, hi_s, 0x5140);
      o[2 * j + 1] = __byte_perm(lo_s, hi_s, 0x7362);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + r * ldo + 32 * c);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

__device__ __forceinline__ float e4m3_bits_to_float(std::uint32_t b) {
  const std::uint32_t e = (b >> 3) & 0xF, mant = b & 7;
  float mag;
  if (e == 0xF && mant == 7) mag = __int_as_float(0x7FC00000);
  else if (e == 0) mag = static_cast<float>(mant) * 0.001953125f;  // 2^-9
  else mag = __uint_as_float(((e + 120u) << 23) | (mant << 20));
  return (b & 0x80) ? -mag : mag;
}

// Raised (OR 1) by a decode that met a NaN or negative group scale and was given no word of the caller's.
__device__ unsigned g_w4_invalid = 0;

// 16 columns per thread (8 packed bytes): level * group scale, rne, clamp to +-127. A group whose scale is NaN or
// negative decodes to zeros and raises *invalid (src/kernels/quant/w4a8_decode.cu:57-62).
__global__ void decode_grouped_kernel(const std::uint8_t* packed, const void* s_rel, int scale_kind, const float* codebook,
                                      std::int64_t rows, std::int64_t k, int group, std::int8_t* out, unsigned* invalid) {
  __shared__ float s_cb[16];
  if (threadIdx.x < 16) s_cb[threadIdx.x] = codebook != nullptr ? codebook[threadIdx.x] : static_cast<float>(threadIdx.x) - 8.0f;
  __syncthreads();
  const std::int64_t per_row = k / 16, total = rows * per_row, groups = k / group;
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const std::int64_t r = i / per_row, c0 = (i % per_row) * 16;
    const std::int64_t gi = r * groups + c0 / group;
    float s;
    if (scale_kind == 0) s = e4m3_bits_to_float(static_cast<const std::uint8_t*>(s_rel)[gi]);
    else s = __half2float(__ushort_as_half(static_cast<const unsigned short*>(s_rel)[gi]));
    const bool ok = !(isnan(s) || s < 0.0f);
    const uint2 in = *reinterpret_cast<const uint2*>(packed + r * (k / 2) + c0 / 2);
    const std::uint32_t w[2] = {in.x, in.y};
    std::uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      std::uint32_t word = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int col = 4 * j + b;
        const std::uint32_t code = (w[col / 8] >> (4 * (col % 8))) & 0xF;
        const float vq = fminf(127.f, fmaxf(-127.f, rintf(fmul(s_cb[code], s))));
        word |= (static_cast<std::uint32_t>(static_cast<int>(vq)) & 0xFF) << (8 * b);
      }
      o[j] = ok ? word : 0u;
    }
    *reinterpret_cast<uint4*>(out + r * k + c0) = make_uint4(o[0], o[1], o[2], o[3]);
    if (!ok) atomicOr(invalid, 1u);
  }
}

}  // namespace
}  // namespace b2

namespace b2 {
int w4_invalid_word(void** out) {
  const cudaError_t e = cudaGetSymbolAddress(out, g_w4_invalid);
  return e == cudaSuccess ? B2_OK : fail_cuda("w4_invalid_word", e);
}
}  // namespace b2

using namespace b2;

extern "C" {

int b2_rotate_quantize(const void* x, int64_t ldx, int8_t* q, int64_t ldq, float* scale, int64_t m, int k, void* stream) {
  constexpr const char* op = "rotate_quantize";
  if (const int rc = check_common(op, x, ldx, q, ldq, scale, m, k, false)) return rc;
  if (m == 0) return B2_OK;
  Args a{};
  a.x = static_cast<const __nv_bfloat16*>(x), a.ldx = ldx, a.q = q, a.ldq = ldq, a.scale = scale, a.k = k;
  return launch<false, false>(op, a, m, as_stream(stream));
}

int b2_rotate_quantize_chunked(const void* x, int64_t ldx, int chunk_cols, int64_t chunk_stride, int8_t* q, int64_t ldq,
                               float* scale, int64_t m, int k, void* stream) {
  constexpr const char* op = "rotate_quantize_chunked";
  if (chunk_cols <= 0 || chunk_cols % 16 != 0 || k % chunk_cols != 0 || chunk_stride % 8 != 0 || ldx < chunk_cols) {
    return fail_invalid(op, "needs chunk_cols % 16 == 0, k % chunk_cols == 0, ldx >= chunk_cols and chunk_stride % 8 == 0");
  }
  if (const int rc = check_common(op, x, std::max<std::int64_t>(ldx, k), q, ldq, scale, m, k, false)) return rc;
  if (ldx % 8 != 0) return fail_invalid(op, "ldx % 8 != 0");
  if (m == 0) return B2_OK;
  Args a{};
  a.x = static_cast<const __nv_bfloat16*>(x), a.ldx = ldx, a.q = q, a.ldq = ldq, a.scale = scale, a.k = k;
  a.chunk_w = chunk_cols, a.chunk_stride = chunk_stride;
  return launch<false, false>(op, a, m, as_stream(stream));
}

int b2_rms_norm_modulate_rotate_quantize(const void* x, int64_t ldx, const void* norm_weight, const void* mod_scale,
                                         const void* mod_shift, int8_t* q, int64_t ldq, float* scale, int64_t m, int k,
                                         void* stream, void* y, int64_t ldy) {
  constexpr const char* op = "rms_norm_modulate_rotate_quantize";
  if (const int rc = check_common(op, x, ldx, q, ldq, scale, m, k, false)) return rc;
  int bw = 32;
  if (const int rc = check_norm(op, norm_weight, mod_scale, mod_shift, m, k, &bw)) return rc;
  if (y != nullptr && (!aligned_to(y, 16) || ldy < k || ldy % 8 != 0)) {
    return fail_invalid(op, "y must be 16-byte aligned with ldy >= k and ldy % 8 == 0 (ldy " + std::to_string(ldy) + ")");
  }
  if (m == 0) return B2_OK;
  Args a{};
  a.x = static_cast<const __nv_bfloat16*>(x), a.ldx = ldx, a.q = q, a.ldq = ldq, a.scale = scale, a.k = k;
  a.weight = static_cast<const __nv_bfloat16*>(norm_weight);
  a.mod_scale = static_cast<const __nv_bfloat16*>(mod_scale);
  a.mod_shift = static_cast<const __nv_bfloat16*>(mod_shift);
  a.y = static_cast<__nv_bfloat16*>(y), a.ldy = ldy;
  a.factor = static_cast<float>(m) / static_cast<float>(m * k);
  a.bw = bw;
  return launch<true, false>(op, a, m, as_stream(stream));
}

int b2_convrot_quantize_int4(const void* x, int64_t ldx, uint8_t* q, int64_t ldq, float* scale, int64_t m, int k,
                             void* stream) {
  constexpr const char* op = "convrot_quantize_int4";
  if (const int rc = check_common(op, x, ldx, q, ldq, scale, m, k, true)) return rc;
  if (m == 0) return B2_OK;
  Args a{};
  a.x = static_cast<const __nv_bfloat16*>(x), a.ldx = ldx, a.q = q, a.ldq = ldq, a.scale = scale, a.k = k;
  return launch<false, true>(op, a, m, as_stream(stream));
}

int b2_rms_norm_modulate_convrot_quantize_int4(const void* x, int64_t ldx, const void* norm_weight,
                                               const void* mod_scale, const void* mod_shift, uint8_t* q, int64_t ldq,
                                               float* scale, int64_t m, int k, void* stream) {
  constexpr const char* op = "rms_norm_modulate_convrot_quantize_int4";
  if (const int rc = check_common(op, x, ldx, q, ldq, scale, m, k, true)) return rc;
  int bw = 32;
  if (const int rc = check_norm(op, norm_weight, mod_scale, mod_shift, m, k, &bw)) return rc;
  if (m == 0) return B2_OK;
  Args a{};
  a.x = static_cast<const __nv_bfloat16*>(x), a.ldx = ldx, a.q = q, a.ldq = ldq, a.scale = scale, a.k = k;
  a.weight = static_cast<const __nv_bfloat16*>(norm_weight);
  a.mod_scale = static_cast<const __nv_bfloat16*>(mod_scale);
  a.mod_shift = static_cast<const __nv_bfloat16*>(mod_shift);
  a.factor = static_cast<float>(m) / static_cast<float>(m * k);
  a.bw = bw;
  return launch<true, true>(op, a, m, as_stream(stream));
}

int b2_unpack_int4(const void* packed, int64_t ldp, int8_t* out, int64_t ldo, int64_t rows, int64_t k, void* stream) {
  constexpr const char* op = "unpack_int4";
  if (rows < 0 || k <= 0 || k % 32 != 0) return fail_invalid(op, "k must be a positive multiple of 32");
  if (rows == 0) return B2_OK;
  if (packed == nullptr || out == nullptr || !aligned_to(packed, 16) || !aligned_to(out, 16) || ldp % 16 != 0 ||
      ldo % 16 != 0 || ldp < k / 2 || ldo < k) {
    return fail_invalid(op, "needs 16-byte aligned rows (ldp % 16 == 0, ldo % 16 == 0)");
  }
  const int chunks = static_cast<int>(k / 32);
  const std::int64_t total = rows * chunks;
  const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((total + 255) / 256, 148 * 16));
  unpack_int4_kernel<<<blocks, 256, 0, as_stream(stream)>>>(static_cast<const std::uint8_t*>(packed), ldp, out, ldo, rows, chunks);
  return check_launch(op);
}

int b2_decode_grouped_int8(const void* packed, const void* s_rel, int scale_kind, const float* codebook, int64_t rows,
                           int64_t k, int group, int8_t* out, unsigned* invalid, void* stream) {
  constexpr const char* op = "decode_grouped_int8";
  if (rows < 0 || k <= 0 || group <= 0 || group % 16 != 0 || k % group != 0 || (scale_kind != 0 && scale_kind != 1)) {
    return fail_invalid(op, "needs group % 16 == 0, k % group == 0 and scale_kind 0 (e4m3) or 1 (fp16)");
  }
  // The extents of a GEMM weight: the kernel's index arithmetic (rows * k / 16 work items) cannot wrap inside them.
  if (rows > 0x7fffffff || k > 131071) return fail_invalid(op, "needs rows < 2^31 and k <= 131071");
  if (rows == 0) return B2_OK;
  if (packed == nullptr || s_rel == nullptr || out == nullptr || !aligned_to(packed, 8) || !aligned_to(out, 16)) {
    return fail_invalid(op, "null or misaligned operand");
  }
  if (invalid == nullptr) {
    void* word = nullptr;
    if (const cudaError_t e = cudaGetSymbolAddress(&word, g_w4_invalid); e != cudaSuccess) return fail_cuda(op, e);
    invalid = static_cast<unsigned*>(word);
  }
  const std::int64_t total = rows * (k / 16);
  const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((total + 255) / 256, 148 * 16));
  decode_grouped_kernel<<<blocks, 256, 0, as_stream(stream)>>>(static_cast<const std::uint8_t*>(packed), s_rel, scale_kind,
                                                              codebook, rows, k, group, out, invalid);
  return check_launch(op);
}

int b2_w4_invalid_scales(unsigned* host_value, int clear) {
  constexpr const char* op = "w4_invalid_scales";
  if (host_value == nullptr) return fail_invalid(op, "null output");
  if (const cudaError_t e = cudaMemcpyFromSymbol(host_value, g_w4_invalid, sizeof(unsigned)); e != cudaSuccess) return fail_cuda(op, e);
  if (clear != 0) {
    const unsigned zero = 0;
    if (const cudaError_t e = cudaMemcpyToSymbol(g_w4_invalid, &zero, sizeof(unsigned)); e != cudaSuccess) return fail_cuda(op, e);
  }
  return B2_OK;
}

}  // extern "C"
