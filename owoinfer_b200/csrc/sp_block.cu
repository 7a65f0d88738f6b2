// Ulysses sequence-parallel form of the all-INT8 block: one process per GPU, P ranks share every sequence. Outside
// attention every operation of the block is local to a token row, so a rank owns a contiguous 1/P slice of each
// sequence's tokens; inside attention it owns H/P heads of the full sequences. Two exchanges per block:
//   #1  after the QKV projection: q, k, v of this rank's tokens, all heads  ->  full sequences, this rank's heads
//   #2  after attention: output of the full sequences, this rank's heads    ->  this rank's tokens, all heads
// Neither exchange needs a packing pass. The QKV weight rows are ordered [destination rank][q | k | v][head][128] (a
// load-time permutation), and the GEMM writes the column block of each destination into that destination's own
// [tokens, 3 * H/P * 128] matrix (column-chunked epilogue): every (sequence, peer) message of exchange #1 is one
// contiguous range, received straight into the rows of the full-sequence buffer that attention reads through strided
// views. Exchange #2 lands in per-source [tokens, H/P * 128] matrices that the rotate-quantise kernel of the output
// projection reads as column chunks. QK-norm + RoPE run after exchange #1 inside the attention pre-pass (they are per
// (token, head), so the bits do not depend on where they run), with the full-sequence RoPE table on every rank.
// The K mean and V maximum of the pre-pass are per (sequence, head): local after the exchange and summed in the same
// order as on one GPU, so the block output equals the single-GPU output bit for bit.
// The heads of a rank are processed in two halves so that the exchanges hide under compute: the QKV projection runs as
// two GEMMs (weight rows ordered [half][destination rank][q | k | v][head][128]); the exchange of half 0 runs on a second
// stream under the GEMM of half 1, the exchange of half 1 under the attention of half 0, the return exchange of half 0
// under the attention of half 1. What a step still waits for is the tail of the first exchange and the return exchange
// of half 1. (An odd number of heads per rank runs as one "half".)
// Transport: NCCL point-to-point calls grouped per exchange, enqueued on the communicator's own stream and fenced with
// events against the caller's stream; receive buffers are this GPU's own memory (no tensor map ever covers a peer's
// memory). The library is bound at run time (dlopen of
// libnccl.so.2, preferring a copy the process has already loaded), so the single-GPU library has no NCCL dependency.
// The reference engine is single-GPU (include/mossinfer/mossinfer.h:314); block sequencing as in
// src/models/moss_dit/dit_block_quant.cpp:196-608.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

struct b2_sp_comm {
  ncclComm_t comm = nullptr;
  int size = 0, rank = 0;
  bool local_exchange = false;  // measurement aid: every message becomes a device copy of the same size on this GPU
  cudaStream_t side = nullptr;  // the exchanges' stream
  cudaEvent_t ready[2] = {nullptr, nullptr};     // main -> side: the data of half h is ready to be sent
  cudaEvent_t arrived[2] = {nullptr, nullptr};   // side -> main: the exchange of half h has landed
};

namespace b2 {
namespace {

constexpr std::size_t kAlign = 256;
std::size_t align_up(std::size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

struct Nccl {
  decltype(&ncclGetUniqueId) get_unique_id = nullptr;
  decltype(&ncclCommInitRank) comm_init_rank = nullptr;
  decltype(&ncclCommDestroy) comm_destroy = nullptr;
  decltype(&ncclGroupStart) group_start = nullptr;
  decltype(&ncclGroupEnd) group_end = nullptr;
  decltype(&ncclSend) send = nullptr;
  decltype(&ncclRecv) recv = nullptr;
  decltype(&ncclGetErrorString) error_string = nullptr;
  bool ok = false;
  std::string why;
};

const Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy already in the process (e.g. the one torch loaded)
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) {
      n.why = "libnccl.so.2 could not be loaded";
      return;
    }
    const auto sym = [&](const char* name) {
      void* p = dlsym(h, name);
      if (p == nullptr) n.why = std::string("libnccl lacks ") + name;
      return p;
    };
    n.get_unique_id = reinterpret_cast<decltype(n.get_unique_id)>(sym("ncclGetUniqueId"));
    n.comm_init_rank = reinterpret_cast<decltype(n.comm_init_rank)>(sym("ncclCommInitRank"));
    n.comm_destroy = reinterpret_cast<decltype(n.comm_destroy)>(sym("ncclCommDestroy"));
    n.group_start = reinterpret_cast<decltype(n.group_start)>(sym("ncclGroupStart"));
    n.group_end = reinterpret_cast<decltype(n.group_end)>(sym("ncclGroupEnd"));
    n.send = reinterpret_cast<decltype(n.send)>(sym("ncclSend"));
    n.recv = reinterpret_cast<decltype(n.recv)>(sym("ncclRecv"));
    n.error_string = reinterpret_cast<decltype(n.error_string)>(sym("ncclGetErrorString"));
    n.ok = n.why.empty();
  });
  return n;
}

int fail_nccl(const char* op, ncclResult_t r) {
  const Nccl& n = nccl();
  return fail_status(B2_ERR_CUDA, op, std::string("NCCL error: ") + (n.error_string != nullptr ? n.error_string(r) : "?"));
}

struct SpLayout {
  std::size_t xq, scale, send1, full, attn_full, recv2, ffn, attn_ws, total;
  std::size_t attn_ws_bytes;
  std::int64_t tokens_local, tokens_full;
  int hp;      // heads per rank
  int halves;  // 2 when hp is even, else 1
  int hh;      // heads per half
};

int check_sp_run(const char* op, const b2_sp_run* run, int size) {
  if (run == nullptr || run->struct_size < sizeof(b2_sp_run)) return fail_invalid(op, "run is null or from an older header");
  const b2_block_run& r = run->local;
  if (r.struct_size < sizeof(b2_block_run) || r.tokens < 0 || r.D <= 0 || r.F <= 0 || r.heads <= 0 || r.D != r.heads * 128 ||
      r.D % 256 != 0 || r.F % 256 != 0) {
    return fail_invalid(op, "needs D == heads * 128, D and F multiples of 256, tokens >= 0");
  }
  if (r.tier != B2_TIER_INT8) return fail_status(B2_ERR_NOT_SUPPORTED, op, "the sequence-parallel block runs the INT8 tier only");
  if (size < 1 || r.heads % size != 0) {
    return fail_status(B2_ERR_NOT_SUPPORTED, op, "heads must split evenly over the ranks of the group");
  }
  if (r.batch < 1 || r.max_seqlen < 1 || r.cu_seqlens == nullptr || run->seq_lens_host == nullptr) {
    return fail_invalid(op, "needs cu_seqlens (device, full sequences), seq_lens_host, batch >= 1, max_seqlen >= 1");
  }
  std::int64_t local = 0;
  for (int i = 0; i < r.batch; ++i) {
    const std::int64_t s = run->seq_lens_host[i];
    if (s < 0 || s % size != 0 || s > r.max_seqlen) return fail_invalid(op, "every sequence length must be a multiple of the group size and <= max_seqlen");
    local += s / size;
  }
  if (local != r.tokens) return fail_invalid(op, "local.tokens must be the sum of seq_len / size");
  return B2_OK;
}

SpLayout carve(const b2_sp_run* run, int size) {
  SpLayout l{};
  const b2_block_run& r = run->local;
  const std::size_t L = static_cast<std::size_t>(r.tokens), D = static_cast<std::size_t>(r.D), F = static_cast<std::size_t>(r.F);
  l.tokens_local = r.tokens, l.tokens_full = r.tokens * size, l.hp = r.heads / size;
  l.halves = l.hp % 2 == 0 ? 2 : 1, l.hh = l.hp / l.halves;
  const std::size_t W = 3 * static_cast<std::size_t>(l.hp) * 128, full = L * size;  // all halves together
  std::size_t at = 0;
  const auto take = [&](std::size_t bytes) {
    const std::size_t off = at;
    at += align_up(bytes);
    return off;
  };
  l.xq = take(L * std::max(D, F));
  l.scale = take(L * 4);
  l.send1 = take(static_cast<std::size_t>(size) * L * W * 2);
  l.full = take(full * W * 2);
  l.attn_full = take(full * (W / 3) * 2);
  l.recv2 = take(static_cast<std::size_t>(size) * L * (W / 3) * 2);
  l.ffn = take(L * F * 2);
  l.attn_ws_bytes = b2_attention_q8_workspace_bytes(&r.attention, l.tokens_full, l.tokens_full, r.batch, r.max_seqlen, l.hh, l.hh);
  l.attn_ws = take(l.attn_ws_bytes);
  l.total = at;
  return l;
}

// One exchange: for every sequence i and peer s, `send_at(i, s)` (count elements) goes to s and `recv_at(i, s)` comes
// from s; the rank's own share is a device copy.
template <typename SendAt, typename RecvAt, typename Count>
int exchange(const char* op, const b2_sp_comm* c, int batch, SendAt send_at, RecvAt recv_at, Count count, cudaStream_t st) {
  const Nccl& n = nccl();
  for (int i = 0; i < batch; ++i) {
    if (count(i) == 0) continue;
    if (const cudaError_t e = cudaMemcpyAsync(recv_at(i, c->rank), send_at(i, c->rank), count(i) * 2, cudaMemcpyDeviceToDevice, st);
        e != cudaSuccess) {
      return fail_cuda(op, e);
    }
  }
  if (c->size == 1) return B2_OK;
  if (c->local_exchange) {
    for (int i = 0; i < batch; ++i) {
      for (int s = 0; s < c->size && count(i) != 0; ++s) {
        if (s == c->rank) continue;
        if (const cudaError_t e = cudaMemcpyAsync(recv_at(i, s), send_at(i, s), count(i) * 2, cudaMemcpyDeviceToDevice, st);
            e != cudaSuccess) {
          return fail_cuda(op, e);
        }
      }
    }
    return B2_OK;
  }
  if (const ncclResult_t r = n.group_start(); r != ncclSuccess) return fail_nccl(op, r);
  for (int i = 0; i < batch; ++i) {
    if (count(i) == 0) continue;
    for (int s = 0; s < c->size; ++s) {
      if (s == c->rank) continue;
      if (const ncclResult_t r = n.send(send_at(i, s), count(i), ncclBfloat16, s, c->comm, st); r != ncclSuccess) return fail_nccl(op, r);
      if (const ncclResult_t r = n.recv(recv_at(i, s), count(i), ncclBfloat16, s, c->comm, st); r != ncclSuccess) return fail_nccl(op, r);
    }
  }
  if (const ncclResult_t r = n.group_end(); r != ncclSuccess) return fail_nccl(op, r);
  return B2_OK;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" {

int b2_sp_unique_id(void* id, size_t id_bytes) {
  constexpr const char* op = "sp_unique_id";
  if (id == nullptr || id_bytes < sizeof(ncclUniqueId)) return fail_invalid(op, "needs a buffer of at least 128 bytes");
  const Nccl& n = nccl();
  if (!n.ok) return fail_status(B2_ERR_NOT_SUPPORTED, op, n.why);
  ncclUniqueId u;
  if (const ncclResult_t r = n.get_unique_id(&u); r != ncclSuccess) return fail_nccl(op, r);
  std::memcpy(id, &u, sizeof(u));
  return B2_OK;
}

int b2_sp_comm_create(const void* id, size_t id_bytes, int size, int rank, b2_sp_comm** out) {
  constexpr const char* op = "sp_comm_create";
  if (out == nullptr || size < 1 || rank < 0 || rank >= size) return fail_invalid(op, "needs 0 <= rank < size and an output pointer");
  auto* c = new b2_sp_comm();
  c->size = size, c->rank = rank;
  if (size > 1) {
    if (id == nullptr || id_bytes < sizeof(ncclUniqueId)) {
      delete c;
      return fail_invalid(op, "needs the 128-byte id that rank 0 of the group got from b2_sp_unique_id");
    }
    const Nccl& n = nccl();
    if (!n.ok) {
      delete c;
      return fail_status(B2_ERR_NOT_SUPPORTED, op, n.why);
    }
    ncclUniqueId u;
    std::memcpy(&u, id, sizeof(u));
    if (const ncclResult_t r = n.comm_init_rank(&c->comm, size, u, rank); r != ncclSuccess) {
      delete c;
      return fail_nccl(op, r);
    }
  }
  // The exchanges' stream and the four events that fence it against the caller's stream (created here, once: the block
  // itself allocates nothing).
  cudaError_t e = cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking);
  for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
    e = cudaEventCreateWithFlags(&c->ready[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->arrived[i], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) {
    b2_sp_comm_destroy(c);
    return fail_cuda(op, e);
  }
  *out = c;
  return B2_OK;
}

int b2_sp_comm_destroy(b2_sp_comm* comm) {
  if (comm == nullptr) return B2_OK;
  if (comm->side != nullptr) cudaStreamSynchronize(comm->side);
  if (comm->comm != nullptr) nccl().comm_destroy(comm->comm);
  for (int i = 0; i < 2; ++i) {
    if (comm->ready[i] != nullptr) cudaEventDestroy(comm->ready[i]);
    if (comm->arrived[i] != nullptr) cudaEventDestroy(comm->arrived[i]);
  }
  if (comm->side != nullptr) cudaStreamDestroy(comm->side);
  delete comm;
  return B2_OK;
}

int b2_sp_comm_local_exchange(b2_sp_comm* comm, int on) {
  if (comm == nullptr) return fail_invalid("sp_comm_local_exchange", "null communicator");
  comm->local_exchange = on != 0;
  return B2_OK;
}

size_t b2_block_quant_sp_workspace_bytes(const b2_sp_run* run, int size) {
  if (check_sp_run("block_quant_sp_workspace_bytes", run, size) != B2_OK) return 0;
  return carve(run, size).total;
}

int b2_run_block_quant_sp(const b2_block_weights* w, const b2_block_buffers* a, const b2_sp_run* run, b2_sp_comm* comm,
                          void* stream) {
  constexpr const char* op = "run_block_quant_sp";
  if (comm == nullptr) return fail_invalid(op, "null communicator");
  if (const int rc = check_sp_run(op, run, comm->size)) return rc;
  if (w == nullptr || a == nullptr || w->struct_size < sizeof(b2_block_weights) || a->struct_size < sizeof(b2_block_buffers)) {
    return fail_invalid(op, "weights or buffers are null or from an older header");
  }
  const SpLayout l = carve(run, comm->size);
  if (a->x == nullptr || a->mod == nullptr || a->rope == nullptr || a->workspace == nullptr || a->workspace_bytes < l.total) {
    return fail_invalid(op, "buffers do not match the run: workspace " + std::to_string(a->workspace_bytes) + " of " +
                                std::to_string(l.total) + " bytes");
  }
  for (const void* p : {static_cast<const void*>(a->x), a->mod, a->rope, static_cast<const void*>(a->workspace)}) {
    if (!aligned_to(p, kAlign)) return fail_invalid(op, "operands must be 256-byte aligned");
  }
  if (w->norm1 == nullptr || w->norm2 == nullptr || w->q_norm == nullptr || w->k_norm == nullptr || w->qkv.w == nullptr ||
      w->o.w == nullptr || w->up_gate.w == nullptr || w->down.w == nullptr) {
    return fail_invalid(op, "missing weights");
  }
  const b2_block_run& r = run->local;
  const std::int64_t L = r.tokens, D = r.D, F = r.F;
  if (L == 0) return B2_OK;
  const int P = comm->size, batch = r.batch, halves = l.halves, hh = l.hh;
  const std::int64_t Wh = 3LL * hh * 128, Wo = static_cast<std::int64_t>(hh) * 128;  // per half: q | k | v, and the output
  const std::int64_t T = l.tokens_full;
  cudaStream_t st = as_stream(stream), side = comm->side;
  auto* base = static_cast<std::uint8_t*>(a->workspace);
  auto* xq = reinterpret_cast<std::int8_t*>(base + l.xq);
  auto* scale = reinterpret_cast<float*>(base + l.scale);
  auto* send1 = reinterpret_cast<__nv_bfloat16*>(base + l.send1);      // [half][destination][L][Wh]
  auto* full = reinterpret_cast<__nv_bfloat16*>(base + l.full);        // [half][T][Wh]
  auto* attn_full = reinterpret_cast<__nv_bfloat16*>(base + l.attn_full);  // [half][T][Wo]
  auto* recv2 = reinterpret_cast<__nv_bfloat16*>(base + l.recv2);      // [source][half][L][Wo]
  auto* ffn = reinterpret_cast<__nv_bfloat16*>(base + l.ffn);
  const auto* mod = static_cast<const __nv_bfloat16*>(a->mod);
  // Row offsets of every sequence in the local shard and in the full buffers.
  std::vector<std::int64_t> off_local(batch + 1, 0), off_full(batch + 1, 0);
  for (int i = 0; i < batch; ++i) {
    off_local[i + 1] = off_local[i] + run->seq_lens_host[i] / P;
    off_full[i + 1] = off_full[i] + run->seq_lens_host[i];
  }
  const auto chunk_len = [&](int i) { return off_local[i + 1] - off_local[i]; };
  const auto cuda_ok = [&](cudaError_t e) { return e == cudaSuccess ? B2_OK : fail_cuda(op, e); };

  // QKV projection of the local rows, one GEMM per half of the heads; each destination rank's columns of a half go into
  // that destination's own [L, Wh] matrix. As soon as a half is computed its exchange starts on the side stream.
  if (const int rc = b2_rms_norm_modulate_rotate_quantize(a->x, D, w->norm1, mod + 1 * D, mod + 0 * D, xq, D, scale, L,
                                                          static_cast<int>(D), st, nullptr, 0)) {
    return rc;
  }
  const std::int64_t n_half = 3 * D / halves;
  for (int h = 0; h < halves; ++h) {
    const b2_int8_operands g{xq, D, scale, w->qkv.w + h * n_half * D, w->qkv.scale + h * n_half, L, n_half, D};
    if (const int rc = b2_int8_gemm_chunked(&g, nullptr, send1 + h * P * L * Wh, Wh, static_cast<int>(Wh), L * Wh, st, B2_TILE_AUTO)) return rc;
    if (const int rc = cuda_ok(cudaEventRecord(comm->ready[h], st))) return rc;
    // Exchange #1 of this half: tokens -> heads.
    if (const int rc = cuda_ok(cudaStreamWaitEvent(side, comm->ready[h], 0))) return rc;
    if (const int rc = exchange(
            op, comm, batch, [&](int i, int s) { return send1 + ((h * P + s) * L + off_local[i]) * Wh; },
            [&](int i, int s) { return full + (h * T + off_full[i] + s * chunk_len(i)) * Wh; },
            [&](int i) { return static_cast<std::size_t>(chunk_len(i) * Wh); }, side)) {
      return rc;
    }
    if (const int rc = cuda_ok(cudaEventRecord(comm->arrived[h], side))) return rc;
  }

  // Attention over the full sequences, this rank's heads, half by half; QK-norm + RoPE in its pre-pass from 3072 tokens
  // on. The return exchange of a half starts as soon as its attention is done.
  const bool fused = r.fused_norm_rope != 0;  // automatic (< 0) = in the pre-pass, as in the single-GPU block
  const b2_qk_norm_rope nr{w->q_norm, w->k_norm, a->rope, 128};
  b2_attention_options ao = r.attention;
  if (ao.variant == 0) ao.variant = B2_ATTENTION_Q8_FP8_F32ACC;
  const float sm_scale = static_cast<float>(1.0 / std::sqrt(128.0));
  for (int h = 0; h < halves; ++h) {
    if (const int rc = cuda_ok(cudaStreamWaitEvent(st, comm->arrived[h], 0))) return rc;
    __nv_bfloat16* fh = full + h * T * Wh;
    __nv_bfloat16* oh = attn_full + h * T * Wo;
    if (!fused) {
      if (const int rc = b2_qk_norm_rope_moss(fh, Wh, T, hh, w->q_norm, w->k_norm, a->rope, 128, st)) return rc;
    }
    const b2_view3 vq{fh, T, hh, Wh, 128}, vk{fh + Wo, T, hh, Wh, 128}, vv{fh + 2 * Wo, T, hh, Wh, 128};
    const b2_view3 vo{oh, T, hh, Wo, 128};
    if (const int rc = b2_attention_q8(&ao, &vq, &vk, &vv, &vo, r.cu_seqlens, r.cu_seqlens, batch, r.max_seqlen, sm_scale,
                                       base + l.attn_ws, l.attn_ws_bytes, st, fused ? &nr : nullptr)) {
      return rc;
    }
    if (const int rc = cuda_ok(cudaEventRecord(comm->ready[h], st))) return rc;
    // Exchange #2 of this half: heads -> tokens, into one [L, Wo] matrix per (source rank, half).
    if (const int rc = cuda_ok(cudaStreamWaitEvent(side, comm->ready[h], 0))) return rc;
    if (const int rc = exchange(
            op, comm, batch, [&](int i, int s) { return oh + (off_full[i] + s * chunk_len(i)) * Wo; },
            [&](int i, int s) { return recv2 + ((s * halves + h) * L + off_local[i]) * Wo; },
            [&](int i) { return static_cast<std::size_t>(chunk_len(i) * Wo); }, side)) {
      return rc;
    }
    if (const int rc = cuda_ok(cudaEventRecord(comm->arrived[h], side))) return rc;
  }
  for (int h = 0; h < halves; ++h) {
    if (const int rc = cuda_ok(cudaStreamWaitEvent(st, comm->arrived[h], 0))) return rc;
  }

  // x += o(attn) * gate_a, the rotation reading the per-(source, half) matrices as column chunks in head order.
  if (const int rc = b2_rotate_quantize_chunked(recv2, Wo, static_cast<int>(Wo), L * Wo, xq, D, scale, L, static_cast<int>(D), st)) return rc;
  b2_int8_operands g{};
  g = b2_int8_operands{xq, D, scale, w->o.w, w->o.scale, L, D, D};
  if (const int rc = b2_int8_gemm_gated_residual(&g, nullptr, mod + 2 * D, a->x, D, st, B2_TILE_AUTO)) return rc;

  // ffn = situ_glu(up_gate(rms_norm_modulate(x))); x += down(ffn) * gate_f.
  if (const int rc = b2_rms_norm_modulate_rotate_quantize(a->x, D, w->norm2, mod + 4 * D, mod + 3 * D, xq, D, scale, L,
                                                          static_cast<int>(D), st, nullptr, 0)) {
    return rc;
  }
  g = b2_int8_operands{xq, D, scale, w->up_gate.w, w->up_gate.scale, L, 2 * F, D};
  if (const int rc = b2_int8_gemm_situ_glu(&g, ffn, F, st, B2_TILE_AUTO)) return rc;
  if (const int rc = b2_rotate_quantize(ffn, F, xq, F, scale, L, static_cast<int>(F), st)) return rc;
  g = b2_int8_operands{xq, F, scale, w->down.w, w->down.scale, L, D, F};
  return b2_int8_gemm_gated_residual(&g, nullptr, mod + 5 * D, a->x, D, st, B2_TILE_AUTO);
}

int b2_dit_step_sp(const b2_block_weights* blocks, int num_blocks, const b2_block_buffers* a, const b2_sp_run* run,
                   b2_sp_comm* comm, void* stream) {
  if (blocks == nullptr || num_blocks < 0) return fail_invalid("dit_step_sp", "null blocks");
  for (int i = 0; i < num_blocks; ++i) {
    if (const int rc = b2_run_block_quant_sp(&blocks[i], a, run, comm, stream)) return rc;
  }
  return B2_OK;
}

}  // extern "C"
