// Shared host + device helpers of the B200 quantized-block library: status / last-error plumbing of the C ABI, exact
// single-rounded fp32 helpers, and the sm_100a PTX wrappers (mbarrier, TMA, tcgen05, TMEM) the tensor-core kernels use.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>

#include "owoinfer_b200.h"

namespace b2 {

// ---------------------------------------------------------------------------------------------------------------
// Host: status and error text (thread-local, as the reference's mi_last_error_message).
// ---------------------------------------------------------------------------------------------------------------
void set_last_error(const std::string& msg);
int fail_invalid(const char* op, const std::string& msg);   // returns B2_ERR_INVALID_ARGUMENT
int fail_cuda(const char* op, cudaError_t e);               // returns B2_ERR_CUDA
int fail_status(int status, const char* op, const std::string& msg);
inline int check_launch(const char* op) {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? B2_OK : fail_cuda(op, e);
}
inline bool aligned_to(const void* p, std::uintptr_t bytes) { return reinterpret_cast<std::uintptr_t>(p) % bytes == 0; }
inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// Device words that a tensor-core kernel raises when one of its bounded waits expired (0 = never).
int gemm_status_word(int* host_value);
int attn_status_word(int* host_value);
int gemm_status_clear();
int attn_status_clear();
// Test hooks of the GEMM kernel's bounded waits: the limit in nanoseconds (0 = leave it) and the "skip one stage" switch.
int gemm_debug_set(unsigned long long wait_limit_ns, int skip_stage);

// Number of SMs of the current device (cached per device).
int sm_count();

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
// 2-D tensor of bytes: inner extent `inner` bytes (contiguous), `rows` rows of `row_stride` bytes; box inner_box x row_box,
// swizzle of `swizzle_bytes` (128 or 64). Returns false (and sets the last error) on failure.
bool make_tensor_map_2d(CUtensorMap* map, const void* base, std::uint64_t inner, std::uint64_t rows,
                        std::uint64_t row_stride, std::uint32_t inner_box, std::uint32_t row_box, const char* op,
                        int swizzle_bytes = 128);
// The device word that a grouped 4-bit decode raises on a NaN or negative group scale (address on the current device).
int w4_invalid_word(void** out);

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------------------------
// Device: exact fp32 steps. Every reference op is one fp32 operation rounded once; the _rn intrinsics keep the
// compiler from contracting a multiply and an add into an FMA.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bf_bits_to_float(std::uint32_t bits16) { return __uint_as_float(bits16 << 16); }
// Two values rounded to bf16 with one packed conversion (half the conversion-unit work of two rbf calls).
__device__ __forceinline__ void rbf2(float& a, float& b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const std::uint32_t u = *reinterpret_cast<const std::uint32_t*>(&h);
  a = __uint_as_float(u << 16);
  b = __uint_as_float(u & 0xFFFF0000u);
}
__device__ __forceinline__ std::uint32_t float_to_bf_bits(float v) {
  return static_cast<std::uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}

// ---------------------------------------------------------------------------------------------------------------
// Device: sm_100a PTX wrappers.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ std::uint32_t smem_u32(const void* p) {
  return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(std::uint32_t bar, std::uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(std::uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(std::uint32_t bar, std::uint32_t parity) {
  std::uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same test, letting the hardware keep the thread suspended for up to `hint_ns` while the phase is incomplete (it
// resumes when the phase completes): a waiting warp then issues next to no instructions.
#ifndef B2_WAIT_HINT_NS
#define B2_WAIT_HINT_NS 20000
#endif
__device__ __forceinline__ bool mbar_try_wait_hint(std::uint32_t bar, std::uint32_t parity) {
  std::uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(static_cast<std::uint32_t>(B2_WAIT_HINT_NS))
      : "memory");
  return ok != 0;
}
// Bounded wait: spins at most kSpinLimit polls, also giving up early once another thread of the CTA has raised the
// abort word. Returns false on give-up (and raises the abort word), so the caller can unwind instead of hanging.
constexpr std::uint32_t kSpinLimit = 1u << 24;
__device__ __forceinline__ bool mbar_wait(std::uint32_t bar, std::uint32_t parity, volatile int* abort_word) {
  for (std::uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_word != 0) return false;
  }
  *abort_word = 1;
  return false;
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<std::uint64_t>(map)) : "memory");
}
// 2-D tiled TMA load global -> shared, completion on an mbarrier of this CTA. c0: inner (byte) coordinate, a multiple of
// 16; c1: row coordinate.
__device__ __forceinline__ void tma_load_2d(std::uint32_t dst, const CUtensorMap* map, std::uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<std::uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
// generic-proxy writes to shared memory made visible to the async proxy (tcgen05 / TMA reads).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// TMEM allocation (one full warp executes these).
__device__ __forceinline__ void tmem_alloc(std::uint32_t dst_smem, std::uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(std::uint32_t addr, std::uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// All prior tcgen05.mma of this thread arrive on the mbarrier when they complete.
__device__ __forceinline__ void tc_commit(std::uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor of a K-major (or MN-major, see callers) operand tile stored as 128-byte rows with the
// 128-byte swizzle (what a SWIZZLE_128B TMA box of 128 inner bytes writes): 8-row groups are 1024 bytes apart.
// Bits: [0,14) address >> 4; [16,30) leading byte offset >> 4; [32,46) stride byte offset >> 4; [46,48) version = 1 on
// sm_100; [61,64) layout type, 2 = 128-byte swizzle.
__device__ __forceinline__ std::uint64_t umma_desc_sw128(std::uint32_t smem_addr) {
  std::uint64_t d = 0;
  d |= static_cast<std::uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<std::uint64_t>(1) << 16;             // LBO = 16 bytes (unused inside one swizzle atom)
  d |= static_cast<std::uint64_t>(1024 >> 4) << 32;     // SBO = 1024 bytes
  d |= static_cast<std::uint64_t>(1) << 46;             // descriptor version
  d |= static_cast<std::uint64_t>(2) << 61;             // SWIZZLE_128B
  return d;
}

// Instruction descriptor (32 bits): [4,6) D format (1 = f32, 2 = s32); [7,10) A format; [10,13) B format (kind::i8:
// 1 = signed 8-bit; kind::f8f6f4: 0 = e4m3); bit 15 A major, bit 16 B major (0 = K-major, 1 = MN-major);
// [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr std::uint32_t umma_idesc(int d_fmt, int a_fmt, int b_fmt, int a_mn_major, int b_mn_major,
                                                       int m, int n) {
  return (static_cast<std::uint32_t>(d_fmt) << 4) | (static_cast<std::uint32_t>(a_fmt) << 7) |
         (static_cast<std::uint32_t>(b_fmt) << 10) | (static_cast<std::uint32_t>(a_mn_major) << 15) |
         (static_cast<std::uint32_t>(b_mn_major) << 16) | (static_cast<std::uint32_t>(n >> 3) << 17) |
         (static_cast<std::uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem], one thread issues. accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_i8(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                        std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f8(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                        std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster share one MMA; CTA rank 0 of the pair issues it. -------------------
__device__ __forceinline__ std::uint32_t cluster_ctarank() {
  std::uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of `smem_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ std::uint32_t map_to_cta(std::uint32_t smem_addr, std::uint32_t rank) {
  std::uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier given by its shared::cluster address (own or peer CTA).
__device__ __forceinline__ void mbar_arrive_cluster(std::uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes go to an mbarrier that may live in the peer CTA of the pair (shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(std::uint32_t dst, const CUtensorMap* map, std::uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<std::uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(std::uint32_t dst_smem, std::uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(std::uint32_t addr, std::uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
// Commit of the pair's MMAs: arrives on the mbarrier at this shared-memory offset in every CTA of `cta_mask`.
__device__ __forceinline__ void tc_commit_pair(std::uint32_t bar, std::uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask)
               : "memory");
}
// D[tmem of both CTAs] (+)= A[smem, 128 rows per CTA] * B[smem, N/2 rows per CTA]; issued by the pair's leader only.
__device__ __forceinline__ void umma_i8_pair(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                             std::uint32_t idesc, std::uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns (lane i of the warp gets TMEM lane
// lane_base + i). taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld_32x32(std::uint32_t taddr, std::uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// True in exactly one lane of a converged warp (the others skip the guarded instruction; control flow stays uniform).
__device__ __forceinline__ bool elect_one() {
  std::uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
// The same for 16 consecutive columns.
__device__ __forceinline__ void tmem_ld_32x16(std::uint32_t taddr, std::uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// registers -> TMEM, same shape.
__device__ __forceinline__ void tmem_st_32x32(std::uint32_t taddr, const std::uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
// The same 32-bit value into this warp's 32 lanes x 32 consecutive columns.
__device__ __forceinline__ void tmem_fill_32x32(std::uint32_t taddr, std::uint32_t v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, "
      "%1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1, %1};"
      ::"r"(taddr), "r"(v)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
#endif  // __CUDACC__

}  // namespace b2
