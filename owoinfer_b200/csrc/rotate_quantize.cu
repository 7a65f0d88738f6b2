// Activation quantisers of the quantized DiT block: ConvRot rotation (x · H256 per 256-column group) + per-token INT8 or
// INT4 quantisation, optionally preceded by the MOSS RMSNorm + adaLN modulate, plus the small int4 -> int8 helpers
// (unpack, grouped decode). Element-wise work bound by instruction issue first (four stages of exact-order fp32 adds per
// element) and HBM second: persistent thread blocks, the next row prefetched into shared memory (cp.async) under the
// current one, the butterflies on packed fp32 pairs (add.rn.f32x2), rows held in registers as packed bf16 between the
// absmax pass and the quantise pass, shared memory for the 16 x 16 digit transpose and the byte scatter.
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
#include <atomic>
#include <string>
#include <type_traits>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int kGroup = 256;
constexpr int kMaxK = 32768;
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

using u32 = std::uint32_t;
using u64 = std::uint64_t;

// Two fp32 values in one 64-bit register; add / sub / mul round each half on its own (add.rn.f32x2 and friends), so a
// packed butterfly gives the bits of two scalar ones for half the issue slots.
__device__ __forceinline__ u64 pack2(float lo, float hi) {
  u64 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpack2(u64 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
  u64 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ u64 sub2(u64 a, u64 b) {
  u64 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
  u64 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Radix-4 butterfly on four operands in digit order, each operand a pair (the same element of two 256-groups):
// y_d = 0.5 * (((m0' + m1') + m2') + m3') with operand 3 - d negated. kHalve = false leaves the factor 0.5 out: the
// outputs are then twice the reference's, exactly (a power-of-two factor commutes with every fp32 rounding as long as
// nothing overflows or goes subnormal), and a whole rotation comes out 16 times too large.
template <bool kHalve>
__device__ __forceinline__ void butterfly4(u64& a, u64& b, u64& c, u64& d) {
  const u64 s = add2(a, b), t = sub2(a, b);
  u64 y0 = sub2(add2(s, c), d), y1 = add2(sub2(s, c), d), y2 = add2(add2(t, c), d), y3 = add2(sub2(c, t), d);
  if constexpr (kHalve) {
    const u64 half = pack2(0.5f, 0.5f);
    y0 = mul2(half, y0), y1 = mul2(half, y1), y2 = mul2(half, y2), y3 = mul2(half, y3);
  }
  a = y0, b = y1, c = y2, d = y3;
}
// The two stages whose digits are the low and high 2 bits of the register index.
template <bool kHalve>
__device__ __forceinline__ void stages_on_registers(u64 (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 16; i += 4) butterfly4<kHalve>(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
  for (int i = 0; i < 4; ++i) butterfly4<kHalve>(v[i], v[i + 4], v[i + 8], v[i + 12]);
}

// Sixteen bf16 values as eight packed pairs (element 2i in the low half of word i).
__device__ __forceinline__ void load16_packed(const __nv_bfloat16* p, u32 (&w)[8]) {
  const uint4 lo = reinterpret_cast<const uint4*>(p)[0], hi = reinterpret_cast<const uint4*>(p)[1];
  w[0] = lo.x, w[1] = lo.y, w[2] = lo.z, w[3] = lo.w, w[4] = hi.x, w[5] = hi.y, w[6] = hi.z, w[7] = hi.w;
}
// Packed bf16 pairs: a * b and a + b, each result rounded once to bf16.
__device__ __forceinline__ u32 bmul2(u32 a, u32 b) {
  u32 d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ u32 badd2(u32 a, u32 b) {
  u32 d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Two floats rounded to bf16: lo in the low half.
__device__ __forceinline__ u32 pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const u32*>(&h);
}
__device__ __forceinline__ float bf_lo(u32 w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(u32 w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// Sum of squares of one row in the order of torch's reduce kernel with `bw` cooperating threads (a power of two,
// 32..512), executed by one warp: lane l plays torch threads l, l + 32, ...; `part` is bw floats of shared memory.
__device__ float torch_order_sum_squares(const __nv_bfloat16* xr, int k, int bw, float* part, int lane) {
  for (int t = lane; t < bw; t += 32) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int idx = t; idx * 4 + 3 < k; idx += bw) {
      const uint2 raw = *reinterpret_cast<const uint2*>(xr + idx * 4);
      const float e0 = bf_lo(raw.x), e1 = bf_hi(raw.x), e2 = bf_lo(raw.y), e3 = bf_hi(raw.y);
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

constexpr int kTileStride = 17;  // 64-bit words per row of the 16 x 16 transpose tile (conflict-free)
// Per half-warp; the first 512 bytes later hold the quantised bytes. The 8 words of padding put the two tiles of a warp
// 16 banks apart, so that the narrow stores of its two half-warps into them do not collide.
constexpr int kTileWords = 16 * kTileStride + 8;
constexpr int kStages = 2;           // row buffers: the copies run kStages - 1 rows ahead
constexpr int kNormSmemMaxK = 4096;  // rows up to this length sum their squares from the staged row, in parallel

// Persistent thread blocks, each walking rows blockIdx.x, blockIdx.x + gridDim.x, ...; the next row's bytes are copied
// into shared memory (cp.async, two row buffers, every lane reading back only what it copied) while the current row is
// worked on. A half-warp owns a PAIR of 256-groups at a time (groups 2P and 2P + 1, P = half-warp, half-warp + halves,
// ...: kPairs of them), 16 elements of each per lane, and carries element j of both in one 64-bit register, so that the
// rotation runs on packed fp32 pairs.
//   load layout  : lane h holds elements 16 h + j  -> register index j carries digits d0, d1
//   after the 16 x 16 transpose: element h + 16 j  -> register index j carries digits d2, d3
// The rotated row waits for the row-wide maximum as packed bf16 (group 2P in the low half); the quantised bytes are
// scattered into a shared tile in natural order, so each lane stores 16 (INT8) or 8 (INT4) contiguous bytes per group.
template <int kPairs, bool kNorm, bool kInt4>
__global__ void __launch_bounds__(kPairs == 1 ? 384 : 512, kPairs == 1 ? 2 : 1) rotate_quantize_kernel(const Args a, const int m) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ u32 s_warp_max[4][16];
  __shared__ float s_inv_rms;
  __shared__ float s_part[512];
  const int tid = static_cast<int>(threadIdx.x), lane = tid & 31, warp = tid >> 5, nthreads = static_cast<int>(blockDim.x);
  const int halves = nthreads >> 4, half_id = tid >> 4, h = tid & 15, nwarps = nthreads >> 5;
  const int groups = a.k / kGroup;
  const int stage_vecs = kPairs * 4 * nthreads;
  uint4* const stages = reinterpret_cast<uint4*>(smem_raw);
  u64* const tile = reinterpret_cast<u64*>(smem_raw + kStages * stage_vecs * sizeof(uint4)) + half_id * kTileWords;
  std::uint8_t* const qtile = reinterpret_cast<std::uint8_t*>(tile);

  const auto source = [&](std::int64_t row, int g) {
    const int col = g * kGroup + 16 * h;
    return a.chunk_w == 0 ? a.x + row * a.ldx + col : a.x + (col / a.chunk_w) * a.chunk_stride + row * a.ldx + col % a.chunk_w;
  };
  // Vector v (0, 1: group 2P; 2, 3: group 2P + 1) of pair slot p, for this thread: [stage][p][v][thread].
  const auto staged = [&](int st, int p, int v) { return stages + st * stage_vecs + (p * 4 + v) * nthreads + tid; };
  const auto copy_row = [&](std::int64_t row, int st) {
#pragma unroll
    for (int p = 0; p < kPairs; ++p) {
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        const int g = 2 * (half_id + p * halves) + gi;
        if (g < groups) {
          const __nv_bfloat16* src = source(row, g);
          cp_async16(staged(st, p, 2 * gi), src);
          cp_async16(staged(st, p, 2 * gi + 1), src + 8);
        }
      }
    }
  };

  std::int64_t row = blockIdx.x;
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) {
    if (row + i * static_cast<std::int64_t>(gridDim.x) < m) copy_row(row + i * static_cast<std::int64_t>(gridDim.x), i);
    cp_async_commit();
  }
  for (int it = 0; row < m; row += gridDim.x, ++it) {
    const int st = it % kStages;
    const std::int64_t ahead = row + (kStages - 1) * static_cast<std::int64_t>(gridDim.x);
    if (ahead < m) copy_row(ahead, (it + kStages - 1) % kStages);
    cp_async_commit();
    cp_async_wait<kStages - 1>();

    // The raw words of a pair slot: [0, 8) group 2P, [8, 16) group 2P + 1; zeros for a group past the row's end.
    const auto fetch = [&](int p, u32(&w)[16]) {
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        const bool on = 2 * (half_id + p * halves) + gi < groups;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const uint4 lo = on ? *staged(st, p, 2 * gi) : zero, hi = on ? *staged(st, p, 2 * gi + 1) : zero;
        w[8 * gi + 0] = lo.x, w[8 * gi + 1] = lo.y, w[8 * gi + 2] = lo.z, w[8 * gi + 3] = lo.w;
        w[8 * gi + 4] = hi.x, w[8 * gi + 5] = hi.y, w[8 * gi + 6] = hi.z, w[8 * gi + 7] = hi.w;
      }
    };

    float inv_rms = 0.f;
    if constexpr (kNorm) {
      if (kPairs == 1 && a.k <= kNormSmemMaxK) {
        // Torch's 4 * bw accumulator chains, one per thread, read from the staged row (so every thread's copies have to
        // be visible first). Chain (t, c) = torch thread t's accumulator c: elements 4 * (t + bw * i) + c, i = 0, 1, ...
        // in order. Element e sits in the copy of lane (e % 256) / 16 of the half-warp that owns pair e / 512.
        __syncthreads();
        const unsigned short* staged_row = reinterpret_cast<const unsigned short*>(stages + st * stage_vecs);
        // Element e: lane (e % 256) / 16 of half-warp e / 512, vector (e / 256 % 2) * 2 + (e / 8 % 2) (one pair slot).
        const auto square_at = [&](int e) {
          const int owner = ((e >> 9) << 4) + ((e >> 4) & 15), vec = ((e >> 8) & 1) * 2 + ((e >> 3) & 1);
          const float x = __uint_as_float(static_cast<u32>(staged_row[(vec * nthreads + owner) * 8 + (e & 7)]) << 16);
          return fmul(x, x);
        };
        const int chains = 4 * a.bw;
        for (int ct = tid; ct < chains; ct += nthreads) {
          float acc = 0.f;
          if (a.bw == 32) {
            // 128 chains: term i of chain ct is element ct + 128 i, i.e. lane (ct / 16) % 8 + 8 (i % 2) of half-warp
            // i / 4, group (i / 2) % 2 of its pair: four terms per half-warp, at fixed offsets from a moving base.
            const unsigned short* p0 = staged_row + ((((ct >> 3) & 1) * nthreads + ((ct >> 4) & 7)) * 8 + (ct & 7));
            const unsigned short* p1 = p0 + 2 * nthreads * 8;
            const auto sq = [](unsigned short bits) {
              const float x = __uint_as_float(static_cast<u32>(bits) << 16);
              return fmul(x, x);
            };
            const int terms = a.k >> 7;
            int i = 0;
#pragma unroll 2
            for (; i + 4 <= terms; i += 4, p0 += 128, p1 += 128) {
              const float t0 = sq(p0[0]), t1 = sq(p0[64]), t2 = sq(p1[0]), t3 = sq(p1[64]);
              acc = fadd(fadd(fadd(fadd(acc, t0), t1), t2), t3);
            }
            if (i < terms) acc = fadd(fadd(acc, sq(p0[0])), sq(p0[64]));
          } else {
            int e = ct;
            for (; e + 7 * chains < a.k; e += 8 * chains) {
              float t[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) t[i] = square_at(e + i * chains);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc = fadd(acc, t[i]);
            }
            for (; e < a.k; e += chains) acc = fadd(acc, square_at(e));
          }
          const float a1 = __shfl_down_sync(0xffffffffu, acc, 1), a2 = __shfl_down_sync(0xffffffffu, acc, 2);
          const float a3 = __shfl_down_sync(0xffffffffu, acc, 3);
          if ((ct & 3) == 0) s_part[ct >> 2] = fadd(fadd(fadd(acc, a1), a2), a3);
        }
        __syncthreads();
        // Torch's tree over its bw partial sums: with 32 of them (every row count from 16 up) each warp runs the shuffle
        // steps for itself; more (fewer than 16 rows) first fold in shared memory, by one warp.
        if (a.bw == 32) {
          float ss = s_part[lane];
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) ss = fadd(ss, __shfl_down_sync(0xffffffffu, ss, off));
          inv_rms = rsqrtf(fadd(fmul(__shfl_sync(0xffffffffu, ss, 0), a.factor), 1e-6f));
        } else {
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
          __syncthreads();
          inv_rms = s_inv_rms;
        }
      } else {
        if (warp == 0) {
          const float ss = torch_order_sum_squares(a.x + row * a.ldx, a.k, a.bw, s_part, lane);
          if (lane == 0) s_inv_rms = rsqrtf(fadd(fmul(ss, a.factor), 1e-6f));
        }
        __syncthreads();
        inv_rms = s_inv_rms;
      }
    }

    // The norm + modulate prologue on the raw words of one group (a no-op without it); `store_y` also writes the
    // optional bf16 copy. bf16(bf16(bf16(bf16(x*r)*w) * bf16(1+scale)) + shift): after the first rounding every operand
    // is a bf16 value, so the three remaining steps run on packed pairs (mul.rn / add.rn.bf16x2 round once, exactly as
    // the fp32 operation followed by a rounding to bf16 does for bf16 operands).
    const auto prologue = [&](u32* w, int g, bool store_y) {
      if constexpr (kNorm) {
        if (g >= groups) return;
        const float r = inv_rms;
        const int c0 = g * kGroup + 16 * h;
        u32 nw[8], sc[8], sh[8];
        load16_packed(a.weight + c0, nw);
        load16_packed(a.mod_scale + c0, sc);
        load16_packed(a.mod_shift + c0, sh);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          u32 n = pack_bf16(fmul(bf_lo(w[i]), r), fmul(bf_hi(w[i]), r));
          n = bmul2(n, nw[i]);
          n = bmul2(n, badd2(0x3F803F80u, sc[i]));  // 1.0 in both halves
          w[i] = badd2(n, sh[i]);
        }
        if (store_y && a.y != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(a.y + row * a.ldy + c0);
          dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
          dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
      }
    };

    if constexpr (kNorm) {
      // Norm + modulate alone (no quantiser output asked for): store y and go to the next row.
      if (a.q == nullptr) {
#pragma unroll
        for (int p = 0; p < kPairs; ++p) {
          if (2 * (half_id + p * halves) >= groups) continue;
          u32 w[16];
          fetch(p, w);
          prologue(w, 2 * (half_id + p * halves), true);
          prologue(w + 8, 2 * (half_id + p * halves) + 1, true);
        }
        continue;
      }
    }

    // The rotation, the rounding to bf16 and the row's absolute maximum. kExact = false is the fast form: no factor 0.5
    // in the butterflies, so the rotated values (and the maximum) are 16 times the reference's, bit for bit, provided
    // nothing overflowed on the way; its maximum propagates NaN (a NaN's bf16 pattern, sign cleared, is above every
    // number's), so that an overflow (which always ends in an inf or a NaN) or a non-finite input shows in it.
    // kExact = true follows the reference literally (fmaxf, which skips NaN). Returns the maximum as bf16 bits.
    u32 rot[kPairs][16];
    const auto rotate = [&](auto exact_tag, bool store_y, int slot) -> u32 {
      constexpr bool kExact = decltype(exact_tag)::value;
      u32 amax2 = 0;
#pragma unroll
      for (int p = 0; p < kPairs; ++p) {
        // Warp-uniform: both halves of a warp transpose together (an idle half runs on zeros).
        if (2 * ((half_id & ~1) + p * halves) >= groups) continue;
        u32 w[16];
        fetch(p, w);
        prologue(w, 2 * (half_id + p * halves), store_y);
        prologue(w + 8, 2 * (half_id + p * halves) + 1, store_y);
        u64 v[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[2 * i] = pack2(bf_lo(w[i]), bf_lo(w[8 + i]));
          v[2 * i + 1] = pack2(bf_hi(w[i]), bf_hi(w[8 + i]));
        }
        stages_on_registers<kExact>(v);
#pragma unroll
        for (int j = 0; j < 16; ++j) tile[h * kTileStride + j] = v[j];
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = tile[j * kTileStride + h];
        __syncwarp();
        stages_on_registers<kExact>(v);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float lo, hi;
          unpack2(v[j], lo, hi);
          const u32 r = pack_bf16(lo, hi);
          rot[p][j] = r;
          u32 mag = r & 0x7FFF7FFFu;
          if constexpr (kExact) {
            if ((mag & 0xFFFFu) > 0x7F80u) mag &= 0xFFFF0000u;
            if ((mag >> 16) > 0x7F80u) mag &= 0x0000FFFFu;
          }
          amax2 = __vmaxu2(amax2, mag);
        }
      }
      // A group past the row's end contributed zeros.
      u32 amax = max(amax2 & 0xFFFFu, amax2 >> 16);
      amax = __reduce_max_sync(0xffffffffu, amax);
      if (lane == 0) s_warp_max[slot][warp] = amax;
      __syncthreads();
      return __reduce_max_sync(0xffffffffu, s_warp_max[slot][lane < nwarps ? lane : 0]);
    };
    const u32 amax_bits = rotate(std::false_type{}, true, 2 * (it & 1));
    float amax, unscale = 0.0625f;           // the rotated values in registers are 16 x the reference's
    const bool clean = amax_bits < 0x7E80u;  // below 2^126: no overflow, NaN or inf anywhere (the same in every thread)
    if (clean) {
      amax = fmul(__uint_as_float(amax_bits << 16), 0.0625f);
    } else {
      amax = __uint_as_float(rotate(std::true_type{}, false, 2 * (it & 1) + 1) << 16);
      unscale = 1.0f;
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
    const u64 inv_s2 = pack2(inv_s, inv_s);
    constexpr float kLo = kInt4 ? -7.f : -128.f, kHi = kInt4 ? 7.f : 127.f;
    std::uint8_t* qr = static_cast<std::uint8_t*>(a.q) + row * a.ldq;
#pragma unroll
    for (int p = 0; p < kPairs; ++p) {
      if (2 * ((half_id & ~1) + p * halves) >= groups) continue;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x0, x1;
        unpack2(mul2(pack2(bf_lo(rot[p][j]), bf_hi(rot[p][j])), inv_s2), x0, x1);
        const u32 r = pack_bf16(x0, x1);
        x0 = bf_lo(r), x1 = bf_hi(r);
        u32 b0, b1;
        if (!kInt4 && clean) {
          // A clean row holds finite values of magnitude up to 127.5 (the scale is the row maximum / 127, rounded to
          // bf16), so only the upper clamp can act.
          unpack2(add2(pack2(fminf(kHi, x0), fminf(kHi, x1)), pack2(12582912.0f, 12582912.0f)), x0, x1);
          b0 = __float_as_uint(x0), b1 = __float_as_uint(x1);
        } else {
          // Clamp, then round to nearest even: the bounds are integers, so this equals rounding first. fmaxf sends NaN
          // to the lower bound, infinities saturate. Adding 1.5 * 2^23 rounds to an integer (ties to even) and leaves
          // its two's complement in the low mantissa bits, whose low byte is the code.
          b0 = __float_as_uint(fadd(fminf(kHi, fmaxf(kLo, x0)), 12582912.0f));
          b1 = __float_as_uint(fadd(fminf(kHi, fmaxf(kLo, x1)), 12582912.0f));
        }
        // Both groups' codes of element h + 16 j as one 16-bit store (group 2P in the low byte).
        reinterpret_cast<unsigned short*>(qtile)[h + 16 * j] = static_cast<unsigned short>(__byte_perm(b0, b1, 0x0040));
      }
      __syncwarp();
      // Elements 16 h .. 16 h + 15 of both groups, interleaved; split them into 16 bytes per group.
      const uint4 mixed[2] = {reinterpret_cast<const uint4*>(qtile)[2 * h], reinterpret_cast<const uint4*>(qtile)[2 * h + 1]};
      __syncwarp();
      const uint4 bytes[2] = {
          make_uint4(__byte_perm(mixed[0].x, mixed[0].y, 0x6420), __byte_perm(mixed[0].z, mixed[0].w, 0x6420),
                     __byte_perm(mixed[1].x, mixed[1].y, 0x6420), __byte_perm(mixed[1].z, mixed[1].w, 0x6420)),
          make_uint4(__byte_perm(mixed[0].x, mixed[0].y, 0x7531), __byte_perm(mixed[0].z, mixed[0].w, 0x7531),
                     __byte_perm(mixed[1].x, mixed[1].y, 0x7531), __byte_perm(mixed[1].z, mixed[1].w, 0x7531))};
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        const int g = 2 * (half_id + p * halves) + gi;
        if (g >= groups) continue;
        if constexpr (kInt4) {
          const u32 w[4] = {bytes[gi].x, bytes[gi].y, bytes[gi].z, bytes[gi].w};
          u32 out[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const u32 lo = w[2 * i], hi = w[2 * i + 1];
            // bytes b0..b3 -> nibbles (b0 | b1 << 4), (b2 | b3 << 4)
            const u32 p0 = (lo & 0xF) | ((lo >> 4) & 0xF0), p1 = ((lo >> 16) & 0xF) | ((lo >> 20) & 0xF0);
            const u32 p2 = (hi & 0xF) | ((hi >> 4) & 0xF0), p3 = ((hi >> 16) & 0xF) | ((hi >> 20) & 0xF0);
            out[i] = p0 | (p1 << 8) | (p2 << 16) | (p3 << 24);
          }
          *reinterpret_cast<uint2*>(qr + g * (kGroup / 2) + 8 * h) = make_uint2(out[0], out[1]);
        } else {
          *reinterpret_cast<uint4*>(qr + g * kGroup + 16 * h) = bytes[gi];
        }
      }
    }
  }
  cp_async_wait<0>();
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

// Thread blocks of one shape that fit on an SM: asked of the runtime once per shape and device.
template <int kPairs, bool kNorm, bool kInt4>
int launch_shape(const char* op, const Args& a, std::int64_t m, int threads, std::size_t smem, cudaStream_t stream) {
  static std::atomic<int> resident[64][17];  // [device][warps per block]
  int dev = 0;
  cudaGetDevice(&dev);
  const auto kernel = rotate_quantize_kernel<kPairs, kNorm, kInt4>;
  std::atomic<int>& slot = resident[dev & 63][threads >> 5];
  int per_sm = slot.load(std::memory_order_acquire);
  if (per_sm == 0) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    if (e != cudaSuccess) return fail_cuda(op, e);
    if (per_sm < 1) return fail_invalid(op, "the kernel does not fit on an SM for k = " + std::to_string(a.k));
    slot.store(per_sm, std::memory_order_release);
  }
  const std::int64_t blocks = std::min<std::int64_t>(m, static_cast<std::int64_t>(sm_count()) * per_sm);
  kernel<<<static_cast<unsigned>(blocks), static_cast<unsigned>(threads), smem, stream>>>(a, static_cast<int>(m));
  return check_launch(op);
}

template <bool kNorm, bool kInt4>
int launch(const char* op, const Args& a, std::int64_t m, cudaStream_t stream) {
  const int groups = a.k / kGroup, pairs = (groups + 1) / 2;
  // One pair of groups per half-warp up to 24 half-warps (k = 12288), two up to 32 (k = 32768).
  const int slots = pairs <= 24 ? 1 : 2;
  int halves = (pairs + slots - 1) / slots;
  halves = (halves + 1) & ~1;
  const int threads = halves * 16;
  std::size_t smem = static_cast<std::size_t>(kStages) * slots * 4 * threads * 16 + static_cast<std::size_t>(halves) * kTileWords * 8;
  if (slots == 1) return launch_shape<1, kNorm, kInt4>(op, a, m, threads, smem, stream);
  return launch_shape<2, kNorm, kInt4>(op, a, m, threads, smem, stream);
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

int b2_rms_norm_modulate(const void* x, int64_t ldx, const void* norm_weight, const void* mod_scale, const void* mod_shift,
                         void* y, int64_t ldy, int64_t m, int k, void* stream) {
  constexpr const char* op = "rms_norm_modulate";
  if (k <= 0 || k % kGroup != 0 || k > kMaxK) return fail_invalid(op, "k must be a positive multiple of 256 up to 32768, got " + std::to_string(k));
  if (m < 0 || m > 0x7fffffff) return fail_invalid(op, "row count out of range");
  if (m > 0 && (x == nullptr || y == nullptr)) return fail_invalid(op, "null operand");
  if (ldx < k || ldy < k || ldx % 8 != 0 || ldy % 8 != 0 || !aligned_to(x, 16) || !aligned_to(y, 16)) {
    return fail_invalid(op, "needs 16-byte aligned x and y with ldx, ldy >= k and multiples of 8");
  }
  int bw = 32;
  if (const int rc = check_norm(op, norm_weight, mod_scale, mod_shift, m, k, &bw)) return rc;
  if (m == 0) return B2_OK;
  Args a{};
  a.x = static_cast<const __nv_bfloat16*>(x), a.ldx = ldx, a.k = k;
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
