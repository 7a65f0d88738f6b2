// INT8 x INT8 -> INT32 GEMM for sm_100a with the dequantisation and the following element-wise op fused into the
// epilogue: out = epilogue(sum_k x_q[r,k] * w[c,k]).
//
// Structure (one persistent CTA per SM, warp-specialised; by default a CTA pair shares a 256 x 256 tile, cta_group::2):
//   warp 0  TMA producer: per 128-byte K block, this CTA's 128-row box of A and its 128 (pair) or 128 / 256 (single
//           CTA) rows of B land in a 128-byte-swizzled shared-memory stage (4 to 6 stages), completion on the stage's
//           "full" mbarrier (the leader CTA's, for a pair).
//   warp 1  MMA issuer: the warp walks the loop in uniform control flow, one elected lane issues tcgen05.mma kind::i8
//           (M 128 or 256 for a pair, N 128 or 256, K 32; four per stage) on shared-memory descriptors; tcgen05.commit
//           frees the stage ("empty" mbarrier) and, after the last K block, publishes the accumulator ("tmem_full").
//   warps 2..  epilogue (8 warps; 16 for SiTU-GLU): each warp reads its 32 TMEM lanes (one output row per thread) and
//           its share of the tile's columns, applies the epilogue and stores; its per-column vectors (w_scale, bias,
//           gate) are staged in shared memory. Two accumulators (2 x N TMEM columns) let the epilogue of tile i overlap
//           the main loop of tile i + 1.
// Tiles are visited in bands of M tiles (see tile_coords and the launch code) so that the operands stay in L2.
// The int32 accumulators are exact, so every tile shape gives the same bits. Epilogues (single-rounded fp32, no FMA
// contraction; reference: src/kernels/quant/int8_gemm_impl.cuh:73-188):
//   plain           bf16(((float)acc * xs[r]) * ws[c] + bias[c])
//   gated residual  res = bf16(res + bf16(bf16(y) * gate[c]))
//   SiTU-GLU        h = bf16(deq(acc_hidden)), g = bf16(deq(acc_gate)); out = bf16(gateF[g] * hiddenF[h]) with the two
//                   factors tabulated over every bf16 input. The B tile of output columns [128 t, 128 t + 128) is hidden
//                   rows 128 t.. followed by gate rows F + 128 t.., so one thread finds both halves in its TMEM lane.
// Every wait on an mbarrier is bounded (200 ms of %globaltimer by default); on expiry the CTA raises a status word, drains
// and frees its TMEM instead of hanging.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <string>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 128;  // bytes == int8 elements per K block: one 128-byte swizzle atom per row
constexpr std::int64_t kMaxK = 131071;

enum class Epi : int { kPlain = 0, kGatedResidual = 1, kSituGlu = 2, kAcc = 3 };
// Producer warp, MMA warp, then the epilogue warps: 8 (two per TMEM lane quarter), or 16 for the SiTU-GLU epilogue, whose
// table look-ups are latency-bound and want more warps in flight.
#ifndef B2_EPI_WARPS_GATED
#define B2_EPI_WARPS_GATED 8
#endif
#ifndef B2_EPI_WARPS_PLAIN
#define B2_EPI_WARPS_PLAIN 8
#endif
__host__ __device__ constexpr int epi_warps(Epi e, int bn, bool w4 = false) {
  // (With the W4A8 converter warps in the CTA, SiTU-GLU keeps 8 epilogue warps: the register file is shared.)
  return e == Epi::kSituGlu ? (w4 ? 8 : 16) : bn != 256 ? 8 : e == Epi::kGatedResidual ? B2_EPI_WARPS_GATED : e == Epi::kPlain ? B2_EPI_WARPS_PLAIN : 8;
}
// W4A8: eight more warps expand the packed 4-bit weight tile into the INT8 operand stage (two threads per weight row,
// 64 columns each).
constexpr int kConvWarps = 8;
constexpr std::int64_t kW4FusedMaxRows = 256;  // see fused_pays_off()
__host__ __device__ constexpr int threads_of(Epi e, int bn, bool w4 = false) {
  return 64 + 32 * epi_warps(e, bn, w4) + (w4 ? 32 * kConvWarps : 0);
}
// Shared-memory slice of the SiTU factor tables: inputs with 2^-26 <= |x| < 2^6 (bf16 exponent field 101..132), where all
// but a vanishing share of the pre-activations fall. Gate factors: [sign][exponent - 101][mantissa]; hidden factors: the
// positive half only (25 tanh(h / 25) is odd and every rounding in it is sign-symmetric, so the factor of -h is the
// factor of h with the sign bit set).
constexpr std::uint32_t kMiniExpLo = 101;
constexpr int kMiniGate = 2 * 32 * 128, kMiniHidden = 32 * 128;

struct GemmParams {
  int m, n, k;        // GEMM rows, GEMM columns (2F for SiTU-GLU), reduction length
  int m_tiles, n_tiles;
  int band_m;         // M tiles per band of the tile order (see tile_coords)
  int situ_wide;      // SiTU-GLU: out, ldo and F allow 16-byte stores (else 8-byte stores straight from the threads)
  int half;           // SiTU-GLU: F
  const float* xs;
  const float* ws;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* gate;
  __nv_bfloat16* out;  // output or residual (in place)
  std::int64_t ldo;
  std::int32_t* acc;
  std::int64_t ldacc;
  const std::uint16_t* t_gate;
  const std::uint16_t* t_hidden;
  // Plain epilogue only, column-chunked output (0 = off): columns [i * chunk_cols, (i + 1) * chunk_cols) of every row go
  // to chunk i, an [m, chunk_cols] matrix of row stride ldo that starts chunk_stride elements after chunk i - 1.
  int chunk_cols;
  std::int64_t chunk_stride;
  // W4A8 (kW4 kernels): the B tensor map covers the packed codes [n, k / 2]; group scales e4m3 [n, k / group]; the 16
  // levels (codebook or code - 8); the word that a NaN or negative scale raises.
  const std::uint8_t* w4_srel;
  int w4_group;        // a power of two >= 16
  int w4_group_shift;  // log2(group)
  const float* w4_codebook;
  unsigned* w4_invalid;
};

__device__ int g_gemm_status = 0;  // set to 1 by a CTA whose bounded wait expired
// How long a wait on an mbarrier may last. A step never comes near it (the longest wait of a healthy launch is one K
// loop, tens of microseconds); an operator does not notice it.
__device__ unsigned long long g_gemm_wait_limit_ns = 200000000ull;
// Test hook: 1 = the TMA warp of every CTA leaves out the loads of the last K block of its first tile, so that the
// stage's barrier never completes and the bounded waits run out.
__device__ int g_gemm_test_skip_stage = 0;

__device__ __forceinline__ std::uint64_t global_ns() {
  std::uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded mbarrier wait on wall time (g_gemm_wait_limit_ns). Returns false when it gave up or another role already aborted.
__device__ __forceinline__ bool wait_bar(std::uint32_t bar, std::uint32_t parity, volatile int* abort_word) {
  if (mbar_try_wait(bar, parity)) return true;
  const std::uint64_t t0 = global_ns();
  for (;;) {
    if (mbar_try_wait_hint(bar, parity)) return true;
    if (*abort_word != 0) return false;
    if (global_ns() - t0 > g_gemm_wait_limit_ns) {
      *abort_word = 1;
      return false;
    }
  }
}

__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

// Packed bf16 pairs: a * b and a + b, each half rounded once to bf16. For bf16 operands that is the fp32 operation followed
// by a rounding to bf16 (the fp32 product of two bf16 values is exact; the fp32 sum is exact unless the smaller operand is
// below the larger one's bf16 half-step, where both forms return the larger).
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
__device__ __forceinline__ std::uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const std::uint32_t*>(&h);
}

// Order of the output tiles over the persistent CTAs: bands of band_m M tiles; inside a band the M tile index runs
// fastest. The CTAs working at the same time then share a few activation row blocks and sweep the weight, so both stay
// in L2 (with M fastest over the whole problem a long-K activation matrix is re-read from DRAM once per wave).
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int* mt, int* nt) {
  const int per_band = p.band_m * p.n_tiles;
  const int band = tile / per_band, r = tile - band * per_band;
  const int rows = min(p.band_m, p.m_tiles - band * p.band_m);
  *mt = band * p.band_m + r % rows;
  *nt = r / rows;
}

// One SiTU factor of the bf16 value with these bits from the full table in global memory (the slow path for a value
// outside the shared-memory slice; same entries, so the same bits either way).
__device__ __forceinline__ float situ_factor_full(const std::uint16_t* full, std::uint32_t bits) {
  return __uint_as_float(static_cast<std::uint32_t>(__ldg(full + bits)) << 16);
}

// kCtas == 2: a CTA pair shares one 256 x 256 tile; each CTA stages its 128 rows of A and 128 of the 256 rows of B.
// kW4: the stage also holds the packed 4-bit weight tile (half the bytes of the INT8 one) that the TMA warp brings and
// the converter warps expand into the B operand.
// kOutWarps > 0: the epilogue warps pass their output rows (and, gated residual, the residual rows) through a staging
// tile of shared memory each, so that global memory sees whole 128-byte lines; the ring gives up a stage for it.
constexpr int kOutRowBytes = 144;                       // 64 bf16 of a row + 16 bytes, which spreads the rows over the banks
constexpr int kOutWarpBytes = 32 * kOutRowBytes;        // one epilogue warp's 32 rows x 64 columns
constexpr int kSituOutWarpBytes = 32 * 64;          // SiTU-GLU: one warp's 32 rows x 32 output columns, swizzled, no padding
template <int kBN, int kCtas, bool kW4 = false, int kOutWarps = 0, int kOutWarpSize = kOutWarpBytes>
struct Shape {
  static constexpr int kStages = kW4 ? 4 : (kBN == 256 && kCtas == 1) ? (kOutWarps > 0 ? 3 : 4) : kOutWarps > 0 ? 5 : 6;
  static constexpr int kABytes = kBM * kBK;
  static constexpr int kBBytes = (kBN / kCtas) * kBK;
  static constexpr int kPBytes = kW4 ? kBBytes / 2 : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + kPBytes;
  static constexpr int kOutBytes = kOutWarps * kOutWarpSize;
  static constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + 1024;  // + alignment slack
};
// Which epilogues stage their rows: all but the accumulator dump.
__host__ __device__ constexpr int out_warps(Epi e, int bn, bool w4) { return e == Epi::kAcc ? 0 : epi_warps(e, bn, w4); }
__host__ __device__ constexpr int out_warp_bytes(Epi e) { return e == Epi::kSituGlu ? kSituOutWarpBytes : kOutWarpBytes; }

// Eight 4-bit codes (nibble i = column i) -> eight INT8 values through the 16-entry table `t` of their (row, group):
// two byte permutes pick among entries 0..7 and 8..15 by the low three bits of each code, a third takes the right one by
// the code's top bit.
__device__ __forceinline__ void expand8(std::uint32_t w, const uint4& t, std::uint32_t& lo, std::uint32_t& hi) {
  const std::uint32_t s1 = w & 0x77777777u, s2 = ((w >> 1) & 0x44444444u) | 0x32103210u;
  lo = __byte_perm(__byte_perm(t.x, t.y, s1), __byte_perm(t.z, t.w, s1), s2);
  hi = __byte_perm(__byte_perm(t.x, t.y, s1 >> 16), __byte_perm(t.z, t.w, s1 >> 16), s2 >> 16);
}
__device__ __forceinline__ float e4m3_value(std::uint32_t b) {
  const std::uint32_t e = (b >> 3) & 0xF, mant = b & 7;
  float mag;
  if (e == 0xF && mant == 7) mag = __int_as_float(0x7FC00000);
  else if (e == 0) mag = static_cast<float>(mant) * 0.001953125f;  // 2^-9
  else mag = __uint_as_float(((e + 120u) << 23) | (mant << 20));
  return (b & 0x80) ? -mag : mag;
}

template <int kBN, Epi kEpi, int kCtas, bool kW4 = false>
__global__ void __launch_bounds__(threads_of(kEpi, kBN, kW4), 1)
int8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  static_assert(kCtas == 1 || kBN == 256, "CTA pairs run 256 x 256 tiles");
  static_assert(!kW4 || kBN / kCtas == 128, "W4A8: one weight row of the stage per converter thread");
  using S = Shape<kBN, kCtas, kW4, out_warps(kEpi, kBN, kW4), out_warp_bytes(kEpi)>;
  const std::uint32_t rank = kCtas == 2 ? cluster_ctarank() : 0u;   // CTA of the pair; rank 0 issues the MMAs
  const int tile0 = kCtas == 2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int tile_step = kCtas == 2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int kStages = S::kStages;
  extern __shared__ std::uint8_t smem_raw[];
  __shared__ __align__(8) std::uint64_t s_full[kStages], s_empty[kStages], s_tmem_full[2], s_tmem_empty[2];
  __shared__ __align__(8) std::uint64_t s_pfull[kW4 ? kStages : 1];  // W4A8: the packed tile of a stage has landed
  // W4A8: for every e4m3 scale byte the 16 INT8 values clamp(rint(level[c] * scale), +-127); zeros for a NaN or negative
  // scale. 4 KB, filled once per CTA.
  __shared__ __align__(16) uint4 s_lut[kW4 ? 256 : 1];
  __shared__ std::uint32_t s_tmem_base;
  __shared__ int s_abort;
  // Per epilogue warp: w_scale, bias, gate of its 128 columns (SiTU-GLU: w_scale of its 32 hidden and 32 gate columns).
  constexpr int kEpiWarps = epi_warps(kEpi, kBN, kW4), kVecFloats = kEpi == Epi::kSituGlu ? 64 * (16 / epi_warps(kEpi, kBN, kW4)) : 384;
  __shared__ __align__(16) float s_vec[kEpiWarps][kVecFloats];
  // SiTU-GLU: the slices of the two factor tables, gate factors then hidden factors.
  __shared__ std::uint16_t s_tab[kEpi == Epi::kSituGlu ? kMiniGate + kMiniHidden : 1];

  const int warp = static_cast<int>(threadIdx.x) >> 5, lane = static_cast<int>(threadIdx.x) & 31;
  const std::uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const auto a_addr = [&](int s) { return tiles_base + static_cast<std::uint32_t>(s) * S::kStageBytes; };
  const auto b_addr = [&](int s) { return a_addr(s) + S::kABytes; };
  const auto p_addr = [&](int s) { return b_addr(s) + S::kBBytes; };
  // The epilogue warps' staging tiles, after the ring (generic address of the same 1024-byte aligned base).
  [[maybe_unused]] std::uint8_t* const out_stage =
      smem_raw + (tiles_base - smem_u32(smem_raw)) + static_cast<std::uint32_t>(S::kStages) * S::kStageBytes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      // W4A8: the TMA's arrival (A) plus one per converter warp of the pair (B).
      mbar_init(smem_u32(&s_full[s]), kW4 ? 1 + kConvWarps * kCtas : 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
      if constexpr (kW4) mbar_init(smem_u32(&s_pfull[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&s_tmem_full[i]), 1);
      mbar_init(smem_u32(&s_tmem_empty[i]), kEpiWarps * kCtas);
    }
    s_abort = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    if constexpr (kCtas == 2) {
      tmem_alloc_pair(smem_u32(&s_tmem_base), 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&s_tmem_base), 512);
      tmem_relinquish();
    }
  }
  if constexpr (kW4) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      const float sc = e4m3_value(static_cast<std::uint32_t>(i));
      const bool ok = !(isnan(sc) || sc < 0.0f);
      std::uint32_t wds[4] = {0u, 0u, 0u, 0u};
      for (int c = 0; c < 16 && ok; ++c) {
        const float level = p.w4_codebook != nullptr ? p.w4_codebook[c] : static_cast<float>(c) - 8.0f;
        const float v = fminf(127.f, fmaxf(-127.f, rintf(fmul(level, sc))));
        wds[c >> 2] |= (static_cast<std::uint32_t>(static_cast<int>(v)) & 0xFFu) << (8 * (c & 3));
      }
      s_lut[i] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
    }
  }
  if constexpr (kEpi == Epi::kSituGlu) {
    for (int i = threadIdx.x; i < kMiniGate + kMiniHidden; i += blockDim.x) {
      const bool gate = i < kMiniGate;
      const std::uint32_t j = gate ? i : i - kMiniGate;  // [sign (gate only)][exponent][mantissa]
      const std::uint32_t bits = ((j >> 12) << 15) | ((((j >> 7) & 31u) + kMiniExpLo) << 7) | (j & 127u);
      s_tab[i] = __ldg((gate ? p.t_gate : p.t_hidden) + bits);
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (kCtas == 2) cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const std::uint32_t tmem_base = s_tmem_base;
  volatile int* abort_word = &s_abort;

  const int k_blocks = (p.k + kBK - 1) / kBK;
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (warp == 0) {
    if (lane == 0) {
      std::uint32_t it = 0;
      for (int tile = tile0; tile < total_tiles && *abort_word == 0; tile += tile_step) {
        int mt, nt;
        tile_coords(p, tile, &mt, &nt);
        const int row_a = mt * (kBM * kCtas) + static_cast<int>(rank) * kBM;
        int row_b0, row_b1;
        if constexpr (kEpi == Epi::kSituGlu) {
          row_b0 = nt * 128;
          row_b1 = p.half + nt * 128;
        } else {
          row_b0 = nt * kBN;
          row_b1 = nt * kBN + 128;
        }
        if (kCtas == 2 && rank == 1) row_b0 = row_b1;  // the pair's second CTA stages the second 128 rows of B
        const bool skip_last = g_gemm_test_skip_stage != 0 && tile == tile0;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = static_cast<int>(it % kStages);
          const std::uint32_t ph = (it / kStages) & 1u;
          if (!wait_bar(smem_u32(&s_empty[s]), ph ^ 1u, abort_word)) break;
          if (skip_last && kb + 1 == k_blocks) break;  // test hook: this stage never fills
          const std::uint32_t full = smem_u32(&s_full[s]);
          if constexpr (kW4) {
            // A as in the INT8 kernel; the packed weight tile (64 bytes per row and K block) lands on this CTA's own
            // barrier, where its converter warps pick it up.
            if constexpr (kCtas == 2) {
              if (rank == 0) mbar_expect_tx(full, 2 * S::kABytes);
              tma_load_2d_pair(a_addr(s), &map_a, map_to_cta(full, 0), kb * kBK, row_a);
            } else {
              mbar_expect_tx(full, S::kABytes);
              tma_load_2d(a_addr(s), &map_a, full, kb * kBK, row_a);
            }
            const std::uint32_t pfull = smem_u32(&s_pfull[s]);
            mbar_expect_tx(pfull, S::kPBytes);
            tma_load_2d(p_addr(s), &map_b, pfull, kb * (kBK / 2), row_b0);
          } else if constexpr (kCtas == 2) {
            // Both CTAs' copies complete on the leader's barrier, which expects the bytes of the whole pair.
            if (rank == 0) mbar_expect_tx(full, 2 * S::kStageBytes);
            const std::uint32_t full_leader = map_to_cta(full, 0);
            tma_load_2d_pair(a_addr(s), &map_a, full_leader, kb * kBK, row_a);
            tma_load_2d_pair(b_addr(s), &map_b, full_leader, kb * kBK, row_b0);
          } else {
            mbar_expect_tx(full, S::kStageBytes);
            tma_load_2d(a_addr(s), &map_a, full, kb * kBK, row_a);
            tma_load_2d(b_addr(s), &map_b, full, kb * kBK, row_b0);
            if constexpr (kBN == 256) tma_load_2d(b_addr(s) + 128 * kBK, &map_b, full, kb * kBK, row_b1);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // The whole warp of the issuing CTA walks the loop (uniform control flow, so descriptors and loop state stay in
    // uniform registers; every lane takes the waits); one elected lane issues the MMAs and commits.
    if (rank == 0) {
      constexpr std::uint32_t idesc = umma_idesc(/*s32*/ 2, /*s8*/ 1, /*s8*/ 1, 0, 0, kBM * kCtas, kBN);
      constexpr std::uint32_t kStageUnits = S::kStageBytes >> 4;  // descriptor address units are 16 bytes
      const std::uint64_t da0 = umma_desc_sw128(a_addr(0)), db0 = umma_desc_sw128(b_addr(0));
      std::uint32_t s = 0, ph = 0, tile_it = 0;
      bool ok = true;
      for (int tile = tile0; ok && tile < total_tiles; tile += tile_step, ++tile_it) {
        const std::uint32_t acc = tile_it & 1u, acc_ph = (tile_it >> 1) & 1u;
        ok = wait_bar(smem_u32(&s_tmem_empty[acc]), acc_ph ^ 1u, abort_word);
        ok = !__any_sync(0xffffffffu, !ok);
        if (!ok) break;
        tc_fence_after();
        const std::uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = wait_bar(smem_u32(&s_full[s]), ph, abort_word);
          ok = !__any_sync(0xffffffffu, !ok);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            const std::uint64_t da = da0 + s * kStageUnits, db = db0 + s * kStageUnits;
#pragma unroll
            for (int k4 = 0; k4 < kBK / 32; ++k4) {
              // 32 bytes further along K inside the swizzle atom: +2 in the descriptor's 16-byte address units.
              if constexpr (kCtas == 2) {
                umma_i8_pair(d_tmem, da + static_cast<std::uint64_t>(2 * k4), db + static_cast<std::uint64_t>(2 * k4), idesc,
                             (kb | k4) != 0 ? 1u : 0u);
              } else {
                umma_i8(d_tmem, da + static_cast<std::uint64_t>(2 * k4), db + static_cast<std::uint64_t>(2 * k4), idesc,
                        (kb | k4) != 0 ? 1u : 0u);
              }
            }
            if constexpr (kCtas == 2) tc_commit_pair(smem_u32(&s_empty[s]), 3);
            else tc_commit(smem_u32(&s_empty[s]));
          }
          __syncwarp();
          if (++s == kStages) s = 0, ph ^= 1u;
        }
        if (!ok) break;
        if (elect_one()) {
          if constexpr (kCtas == 2) tc_commit_pair(smem_u32(&s_tmem_full[acc]), 3);
          else tc_commit(smem_u32(&s_tmem_full[acc]));
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (kW4 && warp >= 2 + kEpiWarps) {
    // W4A8 converters: two threads per weight row of the CTA's 128-row stage, 64 columns each. Per K block a thread reads
    // its 32 packed bytes (TMA wrote the tile with the 64-byte swizzle: 16-byte chunk c of row r sits at chunk
    // c ^ ((r / 2) % 4)), takes the 16-entry table of each group from shared memory by the group's scale byte (fetched one
    // K block ahead) and writes the 64 INT8 values into the B stage in the 128-byte-swizzled layout the MMA reads (chunk
    // n of row r at n ^ (r % 8)); then the warp arrives on the stage's "full" barrier (the leader's, for a pair) in place
    // of a TMA completion.
    const int ct = (warp - 2 - kEpiWarps) * 32 + lane;
    const int r = ct & 127, half = ct >> 7;
    const int groups = p.k >> p.w4_group_shift;
    const int nsc = p.w4_group >= 64 ? 1 : 64 >> p.w4_group_shift;   // scales behind a thread's 64 columns: 1, 2 or 4
    std::uint32_t it = 0;
    bool bad = false;
    const int psw = (r >> 1) & 3, bsw = r & 7;
    for (int tile = tile0; tile < total_tiles && *abort_word == 0; tile += tile_step) {
      int mt, nt;
      tile_coords(p, tile, &mt, &nt);
      int wrow;  // the weight row behind stage row r
      if constexpr (kEpi == Epi::kSituGlu) wrow = (rank == 1 ? p.half : 0) + nt * 128 + r;  // hidden rows, gate rows
      else wrow = nt * kBN + static_cast<int>(rank) * 128 + r;
      const bool row_ok = kEpi == Epi::kSituGlu ? nt * 128 + r < p.half : wrow < p.n;
      const std::uint8_t* srow = p.w4_srel + static_cast<std::int64_t>(row_ok ? wrow : 0) * groups;
      // Scale bytes of K block kb for this thread's columns (a zero byte, i.e. zeros, past the row's or the matrix' end).
      const auto fetch = [&](int kb, std::uint32_t (&sb)[4]) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int col = kb * kBK + half * 64 + q * p.w4_group;
          sb[q] = (q < nsc && row_ok && col < p.k) ? static_cast<std::uint32_t>(__ldg(srow + (col >> p.w4_group_shift))) : 0u;
        }
      };
      std::uint32_t sb[4], sb_next[4] = {0u, 0u, 0u, 0u};
      fetch(0, sb);
      bool dead = false;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = static_cast<int>(it % kStages);
        const std::uint32_t ph = (it / kStages) & 1u;
        if (kb + 1 < k_blocks) fetch(kb + 1, sb_next);   // lands during this K block's work
        if (!wait_bar(smem_u32(&s_pfull[s]), ph, abort_word)) {
          dead = true;
          break;
        }
        const std::uint8_t* pk = smem_raw + (p_addr(s) - smem_u32(smem_raw)) + r * 64;
        std::uint8_t* brow = smem_raw + (b_addr(s) - smem_u32(smem_raw)) + r * 128;
        // The tables of this thread's four 16-column chunks: with nsc scales behind its 64 columns, chunk q uses scale
        // q * nsc / 4. (Named variables and selects: an indexed array would live in local memory.)
        const uint4 ta = s_lut[sb[0]];
        const uint4 tb = nsc >= 2 ? s_lut[sb[1]] : ta;
        const uint4 tc = nsc == 4 ? s_lut[sb[2]] : tb;
        const uint4 td = nsc == 4 ? s_lut[sb[3]] : tb;
        // NaN (0x7F, 0xFF) or negative (sign bit over a non-zero magnitude): the table row is zeros; report it.
#pragma unroll
        for (int q = 0; q < 4; ++q) bad |= (sb[q] & 0x7Fu) == 0x7Fu || sb[q] > 0x80u;
        const uint4 t0 = ta, t1 = nsc == 4 ? tb : ta, t2 = nsc == 4 ? tc : tb, t3 = nsc == 4 ? td : tb;
        {
          const uint4 w = *reinterpret_cast<const uint4*>(pk + (((2 * half) ^ psw) * 16));
          uint4 o0, o1;
          expand8(w.x, t0, o0.x, o0.y);
          expand8(w.y, t0, o0.z, o0.w);
          expand8(w.z, t1, o1.x, o1.y);
          expand8(w.w, t1, o1.z, o1.w);
          *reinterpret_cast<uint4*>(brow + (((4 * half) ^ bsw) * 16)) = o0;
          *reinterpret_cast<uint4*>(brow + (((4 * half + 1) ^ bsw) * 16)) = o1;
        }
        {
          const uint4 w = *reinterpret_cast<const uint4*>(pk + (((2 * half + 1) ^ psw) * 16));
          uint4 o0, o1;
          expand8(w.x, t2, o0.x, o0.y);
          expand8(w.y, t2, o0.z, o0.w);
          expand8(w.z, t3, o1.x, o1.y);
          expand8(w.w, t3, o1.z, o1.w);
          *reinterpret_cast<uint4*>(brow + (((4 * half + 2) ^ bsw) * 16)) = o0;
          *reinterpret_cast<uint4*>(brow + (((4 * half + 3) ^ bsw) * 16)) = o1;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kCtas == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&s_full[s]), 0));
          else mbar_arrive(smem_u32(&s_full[s]));
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) sb[q] = sb_next[q];
      }
      if (dead) break;
    }
    if (bad) atomicOr(p.w4_invalid, 1u);
  } else {
    // Epilogue: 8 warps. Warp w may touch TMEM lanes [32 (w % 4), 32 (w % 4) + 32); warps 2..5 take the first half of the
    // tile's columns, warps 6..9 the second half (SiTU-GLU: output columns, each needing its hidden and gate accumulator).
    const int quarter = warp & 3, col_half = (warp - 2) >> 2;  // SiTU-GLU: one of four 32-column parts
    std::uint32_t tile_it = 0;
    for (int tile = tile0; tile < total_tiles; tile += tile_step, ++tile_it) {
      int mt, nt;
      tile_coords(p, tile, &mt, &nt);
      const std::uint32_t acc = tile_it & 1u, acc_ph = (tile_it >> 1) & 1u;
      // This warp's per-column vectors (w_scale, bias, gate of its half of the tile's columns) -> its own slice of shared
      // memory, four columns per lane; only the warp itself reads them back, so a warp-level sync is enough.
      float* vec = s_vec[warp - 2];
      __syncwarp();
      if constexpr (kEpi != Epi::kAcc) {  // the accumulator dump reads no per-column vector (and allows any n)
        constexpr int kHalfCols = kBN / (kEpiWarps / 4);  // columns of one warp's part of the tile
        // SiTU-GLU: a warp takes 32-column parts col_half, col_half + kEpiWarps / 4, ... of the tile's 128 output columns
        // (one part with 16 epilogue warps, two with 8); 64 floats per part.
        constexpr int kSituParts = kEpi == Epi::kSituGlu ? 16 / kEpiWarps : 1;
        for (int j = lane * 4; j < (kEpi == Epi::kSituGlu ? 64 * kSituParts : 128); j += 128) {
          int col;
          bool ok;
          if constexpr (kEpi == Epi::kSituGlu) {
            const int part = col_half + (j >> 6) * (kEpiWarps / 4);
            const int oc = nt * 128 + part * 32 + (j & 31);   // output column; (j % 64) < 32 hidden, >= 32 gate
            col = ((j & 63) < 32 ? 0 : p.half) + oc;
            ok = oc < p.half;
          } else {
            col = nt * kBN + col_half * kHalfCols + j;
            ok = j < kHalfCols && col < p.n;
          }
          float4 w = make_float4(0.f, 0.f, 0.f, 0.f), b = w, g = w;
          if (ok) {
            w = ldg4(p.ws + col);
            if constexpr (kEpi == Epi::kPlain || kEpi == Epi::kGatedResidual) {
              if (p.bias != nullptr) {
                float t[4];
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.bias + col));
                t[0] = __uint_as_float(raw.x << 16), t[1] = __uint_as_float(raw.x & 0xFFFF0000u);
                t[2] = __uint_as_float(raw.y << 16), t[3] = __uint_as_float(raw.y & 0xFFFF0000u);
                b = make_float4(t[0], t[1], t[2], t[3]);
              }
            }
            if constexpr (kEpi == Epi::kGatedResidual) {
              // The gate stays packed bf16 (two words for these four columns): the epilogue multiplies packed pairs.
              const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.gate + col));
              g = make_float4(__uint_as_float(raw.x), __uint_as_float(raw.y), 0.f, 0.f);
            }
          }
          *reinterpret_cast<float4*>(vec + j) = w;
          if constexpr (kEpi != Epi::kSituGlu) {
            *reinterpret_cast<float4*>(vec + 128 + j) = b;
            *reinterpret_cast<float2*>(vec + 256 + j / 2) = make_float2(g.x, g.y);  // word c / 2 = columns c, c + 1
          }
        }
      }
      __syncwarp();
      if (!wait_bar(smem_u32(&s_tmem_full[acc]), acc_ph, abort_word)) break;
      tc_fence_after();
      const int row = mt * (kBM * kCtas) + static_cast<int>(rank) * kBM + quarter * 32 + lane;
      const bool row_ok = row < p.m;
      const float xs = row_ok ? p.xs[row] : 0.f;
      const std::uint32_t t_row = tmem_base + acc * kBN + (static_cast<std::uint32_t>(quarter * 32) << 16);

      if constexpr (kEpi == Epi::kSituGlu) {
        const int col0 = nt * 128;
        constexpr int kSituParts = 16 / kEpiWarps;
#pragma unroll 1
        for (int pi = 0; pi < kSituParts; ++pi) {
          const int c0 = (col_half + pi * (kEpiWarps / 4)) * 32;
          const float* pvec = vec + 64 * pi;
          std::uint32_t rh[32], rg[32];
          tmem_ld_32x32(t_row + c0, rh);
          tmem_ld_32x32(t_row + 128 + c0, rg);
          tmem_ld_wait();
          // The warp's 32 rows x 32 output columns pass through its staging tile (64 bytes per row, the 16-byte pieces of
          // a row permuted by the row so that neither side has bank conflicts): thread r computes row r, lane l stores
          // piece l % 4 of rows l / 4, l / 4 + 8, ..., so that global memory sees 64 contiguous bytes per row and whole
          // sectors (one thread per row storing 8 bytes at a time made every request touch 32 quarter-used sectors).
          std::uint8_t* stage_tile = out_stage + (warp - 2) * kSituOutWarpBytes;
          const bool wide = p.situ_wide != 0;  // the same in every thread
          __syncwarp();  // the stores of the part before have read the tile
          if (row_ok) {
            uint2 even = make_uint2(0u, 0u);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              const int col = col0 + c0 + 4 * v;
              uint2 packed = make_uint2(0u, 0u);
              if (col < p.half) {
                const float4 wh = *reinterpret_cast<const float4*>(pvec + 4 * v);
                const float4 wg = *reinterpret_cast<const float4*>(pvec + 32 + 4 * v);
                const float whs[4] = {wh.x, wh.y, wh.z, wh.w}, wgs[4] = {wg.x, wg.y, wg.z, wg.w};
                // Both pre-activations of an output are rounded to bf16 by one packed conversion: hidden bits in the low
                // half, gate bits in the high half. One subtraction rebases both exponents onto the shared-memory slice
                // of the tables; the look-up runs unconditionally (its index is masked into the slice) and the rare
                // output with a value outside the slice is redone from the full tables afterwards. (A borrow out of the
                // low half only happens when that half is outside the slice, which sends both halves to the redo.)
                float o[4];
                std::uint32_t both[4], outside = 0u;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float h = fmul(fmul(__int2float_rn(static_cast<int>(rh[4 * v + i])), xs), whs[i]);
                  const float g = fmul(fmul(__int2float_rn(static_cast<int>(rg[4 * v + i])), xs), wgs[i]);
                  both[i] = pack2(h, g);
                  const std::uint32_t u = both[i] - ((kMiniExpLo << 7) * 0x10001u);
                  outside |= u;
                  const std::uint32_t ih = u & 0xFFFu;
                  const std::uint32_t ig = ((u >> 16) & 0xFFFu) + ((u >> 19) & 0x1000u);
                  const std::uint32_t hb = static_cast<std::uint32_t>(s_tab[kMiniGate + ih]) | (both[i] & 0x8000u);
                  o[i] = fmul(__uint_as_float(static_cast<std::uint32_t>(s_tab[ig]) << 16), __uint_as_float(hb << 16));
                }
                if ((outside & 0x70007000u) != 0u) {
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    o[i] = fmul(situ_factor_full(p.t_gate, both[i] >> 16), situ_factor_full(p.t_hidden, both[i] & 0xFFFFu));
                  }
                }
                packed = make_uint2(pack2(o[0], o[1]), pack2(o[2], o[3]));
              }
              if (!wide) {
                // An output whose rows or width only allow 8-byte accesses: straight from the thread, as before.
                if (col < p.half) __stcs(reinterpret_cast<uint2*>(p.out + static_cast<std::int64_t>(row) * p.ldo + col), packed);
              } else if ((v & 1) == 0) {
                even = packed;
              } else {
                const int pc = (v >> 1) ^ ((lane >> 1) & 3);
                *reinterpret_cast<uint4*>(stage_tile + lane * 64 + 16 * pc) = make_uint4(even.x, even.y, packed.x, packed.y);
              }
            }
          }
          __syncwarp();
          if (wide) {
            const int pc = lane & 3, sub = lane >> 2;
            const int row_base = mt * (kBM * kCtas) + static_cast<int>(rank) * kBM + quarter * 32;
            const int pcol = col0 + c0 + 8 * pc;
            if (pcol < p.half) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = sub + 8 * i, r = row_base + rr;
                if (r < p.m) {
                  const uint4 out16 = *reinterpret_cast<const uint4*>(stage_tile + rr * 64 + 16 * (pc ^ ((rr >> 1) & 3)));
                  // Streaming store: the output (4 x the weight's size) must not push the weight out of L2.
                  __stcs(reinterpret_cast<uint4*>(p.out + static_cast<std::int64_t>(r) * p.ldo + pcol), out16);
                }
              }
            }
          }
        }
      } else {
        const int col0 = nt * kBN;
        constexpr int kHalfCols = kBN / (kEpiWarps / 4);
#pragma unroll 1
        for (int c0 = col_half * kHalfCols; c0 < (col_half + 1) * kHalfCols; c0 += 64) {
          std::uint32_t r[64];
          tmem_ld_32x32(t_row + c0, *reinterpret_cast<std::uint32_t(*)[32]>(&r[0]));
          tmem_ld_32x32(t_row + c0 + 32, *reinterpret_cast<std::uint32_t(*)[32]>(&r[32]));
          tmem_ld_wait();
          if constexpr (kEpi == Epi::kAcc) {
            if (!row_ok) continue;
            std::int32_t* arow = p.acc + static_cast<std::int64_t>(row) * p.ldacc;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              if (col0 + c0 + i < p.n) arow[col0 + c0 + i] = static_cast<std::int32_t>(r[i]);
            }
          } else {
            // The warp's 32 rows x 64 columns pass through its staging tile: lane l moves the 16-byte piece l % 8 of rows
            // l / 8, l / 8 + 4, ..., so that every global access of a quarter-warp is one whole 128-byte line, while
            // thread r computes row r. (One thread per row straight to global memory made every request touch 32
            // half-used sectors; at K = 3072 the stores and the residual loads, not the MMAs, set the pace of a tile.)
            std::uint8_t* stage_tile = out_stage + (warp - 2) * kOutWarpBytes;
            const int piece = lane & 7, sub = lane >> 3;
            const int row_base = mt * (kBM * kCtas) + static_cast<int>(rank) * kBM + quarter * 32;
            const int pcol = col0 + c0 + 8 * piece;  // first column of this lane's piece
            // Where the piece of row r lives in global memory (plain: possibly in a column chunk of its own).
            const auto global_piece = [&](int r) {
              __nv_bfloat16* dst = p.out + static_cast<std::int64_t>(r) * p.ldo + pcol;
              if constexpr (kEpi == Epi::kPlain) {
                if (p.chunk_cols != 0) {  // chunk_cols % 8 == 0: a piece of 8 columns stays inside one chunk
                  const int chunk = pcol / p.chunk_cols;
                  dst = p.out + chunk * p.chunk_stride + static_cast<std::int64_t>(r) * p.ldo + (pcol - chunk * p.chunk_cols);
                }
              }
              return dst;
            };
            if constexpr (kEpi == Epi::kGatedResidual) {
              __syncwarp();  // the tile's previous use (this warp's stores of the chunk before) is over
              if (pcol < p.n) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const int r = row_base + sub + 4 * i;
                  if (r < p.m) {
                    *reinterpret_cast<uint4*>(stage_tile + (sub + 4 * i) * kOutRowBytes + 16 * piece) =
                        *reinterpret_cast<const uint4*>(global_piece(r));
                  }
                }
              }
              __syncwarp();
            }
            if (row_ok) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                const int col = col0 + c0 + 8 * v;
                if (col >= p.n) continue;  // n % 8 == 0: a vector of 8 columns is all in or all out
                const int lc = c0 - col_half * kHalfCols + 8 * v;  // column inside this warp's half
                const float4 w0 = *reinterpret_cast<const float4*>(vec + lc);
                const float4 w1 = *reinterpret_cast<const float4*>(vec + lc + 4);
                const float4 b0 = *reinterpret_cast<const float4*>(vec + 128 + lc);
                const float4 b1 = *reinterpret_cast<const float4*>(vec + 128 + lc + 4);
                const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const float bias[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                float y[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  y[i] = fadd(fmul(fmul(__int2float_rn(static_cast<int>(r[8 * v + i])), xs), ws[i]), bias[i]);
                }
                uint4* mine = reinterpret_cast<uint4*>(stage_tile + lane * kOutRowBytes + 16 * v);
                uint4 out8 = make_uint4(pack2(y[0], y[1]), pack2(y[2], y[3]), pack2(y[4], y[5]), pack2(y[6], y[7]));
                if constexpr (kEpi == Epi::kGatedResidual) {
                  // res + bf16(bf16(y) * gate), rounded to bf16: every operand is a bf16 value after the first rounding,
                  // so both steps run on packed pairs.
                  const uint4 g = *reinterpret_cast<const uint4*>(vec + 256 + lc / 2), res = *mine;
                  out8 = make_uint4(badd2(res.x, bmul2(out8.x, g.x)), badd2(res.y, bmul2(out8.y, g.y)),
                                    badd2(res.z, bmul2(out8.z, g.z)), badd2(res.w, bmul2(out8.w, g.w)));
                }
                *mine = out8;
              }
            }
            __syncwarp();
            if (pcol < p.n) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = row_base + sub + 4 * i;
                if (r < p.m) {
                  const uint4 packed = *reinterpret_cast<const uint4*>(stage_tile + (sub + 4 * i) * kOutRowBytes + 16 * piece);
                  // Plain: streaming, the output must not push the weight out of L2. Gated residual: in place, x stays.
                  if constexpr (kEpi == Epi::kPlain) __stcs(reinterpret_cast<uint4*>(global_piece(r)), packed);
                  else *reinterpret_cast<uint4*>(global_piece(r)) = packed;
                }
              }
            }
            if constexpr (kEpi == Epi::kPlain) __syncwarp();  // before the next chunk's rows overwrite the tile
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCtas == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&s_tmem_empty[acc]), 0));
        else mbar_arrive(smem_u32(&s_tmem_empty[acc]));
      }
    }
  }

  __syncthreads();
  if (s_abort != 0) {
    // A wait expired: give in-flight copies and MMAs time to land before the TMEM goes away, then report.
    if (threadIdx.x == 0) atomicExch(&g_gemm_status, 1);
    const std::uint64_t t0 = global_ns();
    while (global_ns() - t0 < 2000000ull) {
    }
    __syncthreads();
  }
  if constexpr (kCtas == 2) cluster_sync_all();  // nothing of the pair is in flight towards this CTA any more
  if (warp == 1) {
    tc_fence_after();
    if constexpr (kCtas == 2) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// SiTU factor tables: for every bf16 input x (index = its 16 bits), the bf16 gate factor
// bf16(bf16(4 * bf16(tanh(bf16(x / 4)))) * bf16(sigmoid(x))) and hidden factor bf16(25 * bf16(tanh(bf16(x * fp32(1/25))))).
// Reference: src/kernels/fused/fused_gemm_impl.cuh:58-67, src/kernels/quant/int8_gemm_situ.cu:16-27.
// ---------------------------------------------------------------------------------------------------------------
__device__ std::uint16_t g_situ_gate[65536];
__device__ std::uint16_t g_situ_hidden[65536];

__global__ void fill_situ_tables() {
  const std::uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const float x = __uint_as_float(i << 16);
  const float sig = __fdiv_rn(1.0f, fadd(1.0f, expf(-x)));
  const float gate = rbf(fmul(rbf(fmul(4.0f, rbf(tanhf(rbf(fmul(x, 0.25f)))))), rbf(sig)));
  const float hidden = rbf(fmul(25.0f, rbf(tanhf(rbf(fmul(x, 1.0f / 25.0f))))));
  g_situ_gate[i] = static_cast<std::uint16_t>(float_to_bf_bits(gate));
  g_situ_hidden[i] = static_cast<std::uint16_t>(float_to_bf_bits(hidden));
}

struct SituTables {
  const std::uint16_t* gate = nullptr;
  const std::uint16_t* hidden = nullptr;
};

// Filled once per device. Outside stream capture the first call fills on `stream` and synchronises it (the one host
// synchronisation of this library); inside a capture the fill is enqueued into the graph and the device stays unmarked.
int situ_tables(cudaStream_t stream, SituTables* out) {
  constexpr const char* op = "int8_gemm_situ_glu";
  static std::mutex mu;
  static bool filled[64] = {};
  static SituTables ptrs[64];
  int dev = 0;
  if (const cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return fail_cuda(op, e);
  if (dev < 0 || dev >= 64) return fail_status(B2_ERR_INTERNAL, op, "device ordinal out of range");
  const std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev].gate == nullptr) {
    void *g = nullptr, *h = nullptr;
    if (const cudaError_t e = cudaGetSymbolAddress(&g, g_situ_gate); e != cudaSuccess) return fail_cuda(op, e);
    if (const cudaError_t e = cudaGetSymbolAddress(&h, g_situ_hidden); e != cudaSuccess) return fail_cuda(op, e);
    ptrs[dev].gate = static_cast<const std::uint16_t*>(g);
    ptrs[dev].hidden = static_cast<const std::uint16_t*>(h);
  }
  if (!filled[dev]) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (const cudaError_t e = cudaStreamIsCapturing(stream, &cap); e != cudaSuccess) return fail_cuda(op, e);
    fill_situ_tables<<<256, 256, 0, stream>>>();
    if (const int rc = check_launch(op)) return rc;
    if (cap == cudaStreamCaptureStatusNone) {
      if (const cudaError_t e = cudaStreamSynchronize(stream); e != cudaSuccess) return fail_cuda(op, e);
      filled[dev] = true;
    }
  }
  *out = ptrs[dev];
  return B2_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Built-in scratch of b2_w4a8_gemm_noalloc: part of the library's device image, so every GPU that loads the library
// holds these 16 MiB until the process exits. The name below is only a host-side handle; the device address is asked
// from the runtime once per device (with that device current) and that address is what the kernels receive.
// ---------------------------------------------------------------------------------------------------------------
constexpr std::size_t kStaticScratchBytes = std::size_t{16} << 20;
static __device__ __align__(256) std::int8_t g_w4_scratch[kStaticScratchBytes];

int static_scratch(std::int8_t** out) {
  constexpr const char* op = "w4a8_gemm_noalloc";
  static std::mutex mu;
  static std::int8_t* ptrs[64] = {};
  int dev = 0;
  if (const cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return fail_cuda(op, e);
  if (dev < 0 || dev >= 64) return fail_status(B2_ERR_INTERNAL, op, "device ordinal out of range");
  const std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    std::int8_t* p = nullptr;
    if (const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_w4_scratch); e != cudaSuccess) {
      return fail_cuda(op, e);
    }
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return B2_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Host: validation and launch.
// ---------------------------------------------------------------------------------------------------------------
int check_operands(const char* op, const b2_int8_operands* a) {
  if (a == nullptr) return fail_invalid(op, "null operands");
  if (a->m < 0 || a->m > 0x7fffffff || a->n <= 0 || a->n > 0x7fffffff || a->k <= 0 || a->k > kMaxK) {
    return fail_invalid(op, "needs 0 <= m < 2^31, 0 < n < 2^31, 0 < k <= 131071 (m " + std::to_string(a->m) + ", n " +
                                std::to_string(a->n) + ", k " + std::to_string(a->k) + ")");
  }
  if (a->k % 16 != 0 || a->ldx % 16 != 0 || a->ldx < a->k) {
    return fail_invalid(op, "needs k % 16 == 0 and ldx % 16 == 0, ldx >= k (k " + std::to_string(a->k) + ", ldx " +
                                std::to_string(a->ldx) + ")");
  }
  if (a->w == nullptr || a->w_scale == nullptr || !aligned_to(a->w, 16) || !aligned_to(a->w_scale, 16)) {
    return fail_invalid(op, "w and w_scale must be 16-byte aligned device pointers");
  }
  if (a->m > 0 && (a->x_q == nullptr || a->x_scale == nullptr || !aligned_to(a->x_q, 16))) {
    return fail_invalid(op, "x_q must be a 16-byte aligned device pointer and x_scale non-null");
  }
  return B2_OK;
}

int check_output(const char* op, const char* name, const void* p, std::int64_t ld, std::int64_t n_out) {
  if (p == nullptr || !aligned_to(p, 16) || ld < n_out || ld % 8 != 0 || n_out % 8 != 0) {
    return fail_invalid(op, std::string(name) + " must be 16-byte aligned with a row stride >= n and a multiple of 8, n % 8 == 0 (ld " +
                                std::to_string(ld) + ", n " + std::to_string(n_out) + ")");
  }
  return B2_OK;
}

// kW4: a->w points at the packed 4-bit codes [n, k / 2] (p.w4_* describe the rest of the weight).
template <int kBN, Epi kEpi, int kCtas, bool kW4 = false>
int launch_kernel(const char* op, const b2_int8_operands* a, GemmParams p, cudaStream_t stream) {
  using S = Shape<kBN, kCtas, kW4, out_warps(kEpi, kBN, kW4), out_warp_bytes(kEpi)>;
  CUtensorMap map_a, map_b;
  if (!make_tensor_map_2d(&map_a, a->x_q, static_cast<std::uint64_t>(a->k), static_cast<std::uint64_t>(a->m),
                          static_cast<std::uint64_t>(a->ldx), kBK, 128, op)) {
    return B2_ERR_CUDA;
  }
  if constexpr (kW4) {
    if (!make_tensor_map_2d(&map_b, a->w, static_cast<std::uint64_t>(a->k / 2), static_cast<std::uint64_t>(a->n),
                            static_cast<std::uint64_t>(a->k / 2), kBK / 2, 128, op, 64)) {
      return B2_ERR_CUDA;
    }
  } else if (!make_tensor_map_2d(&map_b, a->w, static_cast<std::uint64_t>(a->k), static_cast<std::uint64_t>(a->n),
                                 static_cast<std::uint64_t>(a->k), kBK, 128, op)) {
    return B2_ERR_CUDA;
  }
  auto kernel = int8_gemm_kernel<kBN, kEpi, kCtas, kW4>;
  // Opt in to the large dynamic shared-memory size once per device and instantiation.
  // (Setting the attribute twice from two threads is harmless; the flag only saves the call.)
  static std::atomic<bool> configured[64] = {};
  int dev = 0;
  if (const cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return fail_cuda(op, e);
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    if (const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
        e != cudaSuccess) {
      return fail_cuda(op, e);
    }
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  p.m_tiles = (p.m + kBM * kCtas - 1) / (kBM * kCtas);
  if constexpr (kEpi == Epi::kSituGlu) p.n_tiles = (p.half + 127) / 128;
  else p.n_tiles = (p.n + kBN - 1) / kBN;
  const int total = p.m_tiles * p.n_tiles;
  // M tiles per band. A weight that fits in L2 beside the activation rows in flight (up to 48 MB: every site of the block
  // but up_gate) is swept by short bands of one or two M tiles, so that it is touched again every few microseconds and
  // stays resident while the activations stream through once: at K = 12288 (down) bands of 8 M tiles read 687 MB from
  // DRAM per launch, bands of 2 read 514 MB, the time the same or slightly better. A larger weight instead streams past
  // a band of activation rows held to a fifth of L2 (band_m x tile rows x K bytes): it is then read from HBM once per
  // band rather than once per M tile.
  {
    p.band_m = std::min(2, std::max(1, (sm_count() / kCtas) / std::max(1, p.n_tiles)));
    const std::int64_t a_tile_bytes = static_cast<std::int64_t>(kBM * kCtas) * p.k;
    if (static_cast<std::int64_t>(p.n) * p.k > (48 << 20)) {
      const std::int64_t resident = std::min<std::int64_t>(p.m_tiles, (25 << 20) / std::max<std::int64_t>(1, a_tile_bytes));
      p.band_m = std::max(p.band_m, static_cast<int>(resident));
    }
  }
  if constexpr (kCtas == 2) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * std::min(total, sm_count() / 2)));
    cfg.blockDim = dim3(threads_of(kEpi, kBN, kW4));
    cfg.dynamicSmemBytes = S::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    if (const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, p); e != cudaSuccess) return fail_cuda(op, e);
    return check_launch(op);
  } else {
    const int grid = std::min(total, sm_count());
    kernel<<<grid, threads_of(kEpi, kBN, kW4), S::kSmemBytes, stream>>>(map_a, map_b, p);
    return check_launch(op);
  }
}

// Tile choice: CTA pairs on 256 x 256 tiles when there are enough of them to fill the GPU; else one CTA per 128 x 256
// tile, or 128 x 128 when even those leave SMs idle.
int pick_tile(int tile, std::int64_t m, std::int64_t n_tiles_256) {
  if (tile != B2_TILE_AUTO) return tile;
  const std::int64_t pairs = ((m + 255) / 256) * n_tiles_256;
  if (pairs >= sm_count() / 2) return B2_TILE_2CTA_256x256;
  const std::int64_t big = ((m + kBM - 1) / kBM) * n_tiles_256;
  return big >= sm_count() ? B2_TILE_128x256 : B2_TILE_128x128;
}

template <Epi kEpi>
int dispatch(const char* op, const b2_int8_operands* a, const GemmParams& p, cudaStream_t stream, int tile) {
  if constexpr (kEpi == Epi::kSituGlu) {
    const int t = pick_tile(tile, a->m, (p.half + 127) / 128);
    return t == B2_TILE_2CTA_256x256 ? launch_kernel<256, kEpi, 2>(op, a, p, stream) : launch_kernel<256, kEpi, 1>(op, a, p, stream);
  } else {
    const int t = pick_tile(tile, a->m, (a->n + 255) / 256);
    if (t == B2_TILE_2CTA_256x256) return launch_kernel<256, kEpi, 2>(op, a, p, stream);
    return t == B2_TILE_128x256 ? launch_kernel<256, kEpi, 1>(op, a, p, stream) : launch_kernel<128, kEpi, 1>(op, a, p, stream);
  }
}

// W4A8 with the decode inside the GEMM: CTA pairs (256 x 256 tiles) when there are enough of them, else 128 x 128 tiles
// (plain and gated-residual epilogues only). Returns B2_ERR_NOT_SUPPORTED when no such kernel serves the shape.
template <Epi kEpi>
int dispatch_w4(const char* op, const b2_int8_operands* a, const GemmParams& p, cudaStream_t stream) {
  const std::int64_t n256 = kEpi == Epi::kSituGlu ? (p.half + 127) / 128 : (a->n + 255) / 256;
  const int t = pick_tile(B2_TILE_AUTO, a->m, n256);
  if (t == B2_TILE_2CTA_256x256) return launch_kernel<256, kEpi, 2, true>(op, a, p, stream);
  if constexpr (kEpi == Epi::kSituGlu) return B2_ERR_NOT_SUPPORTED;
  else return launch_kernel<128, kEpi, 1, true>(op, a, p, stream);
}

// B2_W4A8_FUSED in the environment overrides the choice between the two W4A8 routes (for A/B timing): 0 = always decode
// to the scratch first, 1 = decode inside the GEMM whenever the weight's format allows.
std::atomic<int>& w4a8_route() {  // -1 automatic, 0 scratch, 1 fused; starts from the environment
  static std::atomic<int> v{[] {
    const char* e = std::getenv("B2_W4A8_FUSED");
    return e == nullptr ? -1 : e[0] == '0' ? 0 : 1;
  }()};
  return v;
}
int w4a8_fused_override() { return w4a8_route().load(std::memory_order_relaxed); }
bool w4a8_fused_enabled() { return w4a8_fused_override() != 0; }
// Decoding inside the GEMM redoes the expansion for every M tile that uses a weight tile, decoding to a scratch does it
// once but moves 2.5 bytes per weight through memory instead of 0.5: the fused kernel wins while the GEMM is bound by
// the weight's bytes (few rows), the scratch route once it is bound by the tensor core (many rows).
bool fused_pays_off(std::int64_t m) { return w4a8_fused_override() == 1 || m <= kW4FusedMaxRows; }

GemmParams base_params(const b2_int8_operands* a) {
  GemmParams p{};
  p.m = static_cast<int>(a->m), p.n = static_cast<int>(a->n), p.k = static_cast<int>(a->k);
  p.xs = a->x_scale, p.ws = a->w_scale;
  return p;
}

}  // namespace

// Used by the block driver (same translation-unit-independent entry points as the C ABI).
int gemm_status_word(int* host_value) {
  const cudaError_t e = cudaMemcpyFromSymbol(host_value, g_gemm_status, sizeof(int));
  return e == cudaSuccess ? B2_OK : fail_cuda("gemm_status", e);
}
int gemm_status_clear() {
  const int zero = 0;
  const cudaError_t e = cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
  return e == cudaSuccess ? B2_OK : fail_cuda("gemm_status", e);
}
int gemm_debug_set(unsigned long long wait_limit_ns, int skip_stage) {
  if (wait_limit_ns != 0) {
    if (const cudaError_t e = cudaMemcpyToSymbol(g_gemm_wait_limit_ns, &wait_limit_ns, sizeof(wait_limit_ns)); e != cudaSuccess) {
      return fail_cuda("debug_bounded_wait", e);
    }
  }
  const cudaError_t e = cudaMemcpyToSymbol(g_gemm_test_skip_stage, &skip_stage, sizeof(int));
  return e == cudaSuccess ? B2_OK : fail_cuda("debug_bounded_wait", e);
}

}  // namespace b2

using namespace b2;

namespace b2 {
namespace {

// Argument checks of the three epilogues, shared by the INT8 entry points and the W4A8 ones (which run them, with the
// scratch standing in for the weight, before anything is launched).
int check_plain(const char* op, const b2_int8_operands* a, const void* bias, const void* out, std::int64_t ldo) {
  if (const int rc = check_operands(op, a)) return rc;
  if (const int rc = check_output(op, "out", out, ldo, a->n)) return rc;
  if (bias != nullptr && !aligned_to(bias, 16)) return fail_invalid(op, "bias must be 16-byte aligned");
  return B2_OK;
}
int check_gated(const char* op, const b2_int8_operands* a, const void* bias, const void* gate, const void* residual,
                std::int64_t ldr) {
  if (const int rc = check_operands(op, a)) return rc;
  if (const int rc = check_output(op, "residual", residual, ldr, a->n)) return rc;
  if (bias != nullptr && !aligned_to(bias, 16)) return fail_invalid(op, "bias must be 16-byte aligned");
  if (gate == nullptr || !aligned_to(gate, 16)) return fail_invalid(op, "gate must be a 16-byte aligned device vector");
  return B2_OK;
}
int check_situ(const char* op, const b2_int8_operands* a, const void* out, std::int64_t ldo) {
  if (a != nullptr && a->n % 8 != 0) return fail_invalid(op, "n = 2F needs F % 4 == 0, got n " + std::to_string(a->n));
  if (const int rc = check_operands(op, a)) return rc;
  const std::int64_t f = a->n / 2;
  if (out == nullptr || !aligned_to(out, 8) || ldo < f || ldo % 4 != 0) {
    return fail_invalid(op, "out must be 8-byte aligned with a row stride >= F and a multiple of 4, got " + std::to_string(ldo));
  }
  return B2_OK;
}

}  // namespace
}  // namespace b2

extern "C" {

int b2_int8_gemm(const b2_int8_operands* op_, const void* bias, void* out, int64_t ldo, void* stream, int tile) {
  constexpr const char* op = "int8_gemm";
  if (const int rc = check_plain(op, op_, bias, out, ldo)) return rc;
  if (op_->m == 0) return B2_OK;
  GemmParams p = base_params(op_);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out), p.ldo = ldo;
  return dispatch<Epi::kPlain>(op, op_, p, as_stream(stream), tile);
}

int b2_int8_gemm_chunked(const b2_int8_operands* op_, const void* bias, void* out, int64_t ldo, int chunk_cols,
                         int64_t chunk_stride, void* stream, int tile) {
  constexpr const char* op = "int8_gemm_chunked";
  if (const int rc = check_operands(op, op_)) return rc;
  if (chunk_cols <= 0 || chunk_cols % 8 != 0 || op_->n % chunk_cols != 0 || chunk_stride % 8 != 0) {
    return fail_invalid(op, "needs chunk_cols % 8 == 0, n % chunk_cols == 0 and chunk_stride % 8 == 0");
  }
  if (const int rc = check_output(op, "out", out, ldo, chunk_cols)) return rc;
  if (bias != nullptr && !aligned_to(bias, 16)) return fail_invalid(op, "bias must be 16-byte aligned");
  if (op_->m == 0) return B2_OK;
  GemmParams p = base_params(op_);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out), p.ldo = ldo;
  p.chunk_cols = chunk_cols, p.chunk_stride = chunk_stride;
  return dispatch<Epi::kPlain>(op, op_, p, as_stream(stream), tile);
}

int b2_int8_gemm_gated_residual(const b2_int8_operands* op_, const void* bias, const void* gate, void* residual,
                                int64_t ldr, void* stream, int tile) {
  constexpr const char* op = "int8_gemm_gated_residual";
  if (const int rc = check_gated(op, op_, bias, gate, residual, ldr)) return rc;
  if (op_->m == 0) return B2_OK;
  GemmParams p = base_params(op_);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.out = static_cast<__nv_bfloat16*>(residual), p.ldo = ldr;
  return dispatch<Epi::kGatedResidual>(op, op_, p, as_stream(stream), tile);
}

int b2_int8_gemm_situ_glu(const b2_int8_operands* op_, void* out, int64_t ldo, void* stream, int tile) {
  constexpr const char* op = "int8_gemm_situ_glu";
  if (const int rc = check_situ(op, op_, out, ldo)) return rc;
  if (op_->m == 0) return B2_OK;
  SituTables t;
  if (const int rc = situ_tables(as_stream(stream), &t)) return rc;
  GemmParams p = base_params(op_);
  p.half = static_cast<int>(op_->n / 2);
  p.out = static_cast<__nv_bfloat16*>(out), p.ldo = ldo;
  p.situ_wide = aligned_to(out, 16) && ldo % 8 == 0 && p.half % 8 == 0;
  p.t_gate = t.gate, p.t_hidden = t.hidden;
  return dispatch<Epi::kSituGlu>(op, op_, p, as_stream(stream), tile);
}

int b2_int8_gemm_acc(const b2_int8_operands* op_, int32_t* acc, int64_t ldacc, void* stream, int tile) {
  constexpr const char* op = "int8_gemm_acc";
  if (const int rc = check_operands(op, op_)) return rc;
  if (acc == nullptr || ldacc < op_->n) return fail_invalid(op, "acc must be non-null with ldacc >= n");
  if (op_->m == 0) return B2_OK;
  GemmParams p = base_params(op_);
  p.acc = acc, p.ldacc = ldacc;
  return dispatch<Epi::kAcc>(op, op_, p, as_stream(stream), tile);
}

int b2_w4a8_gemm(const int8_t* x_q, int64_t ldx, const float* x_scale, const b2_w4_weight* w, int64_t m, int64_t n,
                 int64_t k, int epilogue, const void* aux, void* out, int64_t ldo, int8_t* scratch, void* stream) {
  constexpr const char* op = "w4a8_gemm";
  if (w == nullptr) return fail_invalid(op, "null weight");
  if (epilogue < 0 || epilogue > 2) return fail_invalid(op, "epilogue must be 0 (plain), 1 (gated residual) or 2 (SiTU-GLU)");
  // Every argument of the GEMM is checked (the scratch, or without one the packed codes, standing in for the decoded
  // weight) before anything is launched.
  const b2_int8_operands a{x_q, ldx, x_scale, scratch != nullptr ? scratch : static_cast<const std::int8_t*>(w->packed),
                           w->s_channel, m, n, k};
  if (const int rc = epilogue == 0   ? check_plain(op, &a, aux, out, ldo)
                     : epilogue == 1 ? check_gated(op, &a, nullptr, aux, out, ldo)
                                     : check_situ(op, &a, out, ldo)) {
    return rc;
  }
  if (w->packed == nullptr || w->s_rel == nullptr || !aligned_to(w->packed, 8) || w->group <= 0 || w->group % 16 != 0 ||
      k % w->group != 0 || (w->scale_kind != 0 && w->scale_kind != 1)) {
    return fail_invalid(op, "weight needs packed codes (8-byte aligned), group scales, group % 16 == 0, k % group == 0 and scale_kind 0 or 1");
  }
  if (m == 0) return B2_OK;
  // Decode inside the GEMM (no scratch traffic) for the reference's weight format: e4m3 group scales, a group size that
  // fits the 128-column K blocks, 16-byte aligned packed rows.
  const bool fusable = w->scale_kind == 0 && (w->group & (w->group - 1)) == 0 && k % 128 == 0 && fused_pays_off(m) &&
                       aligned_to(w->packed, 16) && !(epilogue == 2 && pick_tile(B2_TILE_AUTO, m, (n / 2 + 127) / 128) != B2_TILE_2CTA_256x256);
  const bool fused = fusable && w4a8_fused_enabled();
  if (!fused && scratch == nullptr) {
    return fail_invalid(op, "this weight (fp16 group scales, a group size that does not fit 128-column blocks, or a shape too "
                            "small for the fused tiles) is decoded to a scratch buffer first: scratch must not be null");
  }
  if (fused) {
    b2_int8_operands f = a;
    f.w = static_cast<const std::int8_t*>(w->packed);
    GemmParams p = base_params(&f);
    p.w4_srel = static_cast<const std::uint8_t*>(w->s_rel), p.w4_group = w->group, p.w4_codebook = w->codebook;
    for (p.w4_group_shift = 0; (1 << p.w4_group_shift) < w->group; ++p.w4_group_shift) {
    }
    void* word = nullptr;
    if (const int rc = w4_invalid_word(&word)) return rc;
    p.w4_invalid = static_cast<unsigned*>(word);
    p.out = static_cast<__nv_bfloat16*>(out), p.ldo = ldo;
    if (epilogue == 0) {
      p.bias = static_cast<const __nv_bfloat16*>(aux);
      return dispatch_w4<Epi::kPlain>(op, &f, p, as_stream(stream));
    }
    if (epilogue == 1) {
      p.gate = static_cast<const __nv_bfloat16*>(aux);
      return dispatch_w4<Epi::kGatedResidual>(op, &f, p, as_stream(stream));
    }
    SituTables t;
    if (const int rc = situ_tables(as_stream(stream), &t)) return rc;
    p.half = static_cast<int>(n / 2), p.t_gate = t.gate, p.t_hidden = t.hidden;
    p.situ_wide = aligned_to(out, 16) && ldo % 8 == 0 && p.half % 8 == 0;
    return dispatch_w4<Epi::kSituGlu>(op, &f, p, as_stream(stream));
  }
  if (const int rc = b2_decode_grouped_int8(w->packed, w->s_rel, w->scale_kind, w->codebook, n, k, w->group, scratch, nullptr, stream)) {
    return rc;
  }
  if (epilogue == 0) return b2_int8_gemm(&a, aux, out, ldo, stream, B2_TILE_AUTO);
  if (epilogue == 1) return b2_int8_gemm_gated_residual(&a, nullptr, aux, out, ldo, stream, B2_TILE_AUTO);
  return b2_int8_gemm_situ_glu(&a, out, ldo, stream, B2_TILE_AUTO);
}

int b2_debug_w4a8_route(int route) {
  if (route < -1 || route > 1) return fail_invalid("debug_w4a8_route", "route must be -1 (automatic), 0 (scratch) or 1 (fused)");
  w4a8_route().store(route, std::memory_order_relaxed);
  return B2_OK;
}

/* b2_w4a8_gemm for callers that have no device memory to lend as scratch and may not allocate any: the decoded INT8
 * weight goes to a fixed 16 MiB array that lives in this library's device image instead of a caller buffer. See the
 * header for the rules (size limit, first call, overlapping calls). */
int b2_w4a8_gemm_noalloc(const int8_t* x_q, int64_t ldx, const float* x_scale, const b2_w4_weight* w, int64_t m, int64_t n,
                         int64_t k, int epilogue, const void* aux, void* out, int64_t ldo, void* stream) {
  constexpr const char* op = "w4a8_gemm_noalloc";
  // Division, not a product: n * k cannot wrap, whatever the caller passes.
  if (n <= 0 || k <= 0 || static_cast<std::uint64_t>(n) > kStaticScratchBytes / static_cast<std::uint64_t>(k)) {
    return fail_invalid(op, "the decoded weight (n * k = " + std::to_string(n) + " * " + std::to_string(k) +
                                " bytes) does not fit the built-in scratch of " + std::to_string(kStaticScratchBytes) +
                                " bytes; use b2_w4a8_gemm with a caller-owned scratch buffer");
  }
  std::int8_t* scratch = nullptr;
  if (const int rc = static_scratch(&scratch)) return rc;
  return b2_w4a8_gemm(x_q, ldx, x_scale, w, m, n, k, epilogue, aux, out, ldo, scratch, stream);
}

}  // extern "C"
