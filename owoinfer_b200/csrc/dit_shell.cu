// The shell of MossDit::forward around the quantized block loop (src/models/moss_dit/moss_dit.cpp:1181-1477): the
// time embedding and the modulation vectors (:949-969, the fp32 form the published files use), the video embedder
// (:1100-1118), the per-row RoPE tables and joint inputs (:1330-1366), the runs of rows that execute each block with
// their zero-based cu_seqlens (:1262-1318, without reference slots), the block loop, and the head (:1468-1476).
// Everything outside the two bf16 linears (embedder 128 -> 3072, head 3072 -> 128: plain library GEMMs, cuBLASLt bound at
// run time like the reference's, src/kernels/basic/gemm.h:20-63) is specified to the bit by the reference's own kernels
// and restated here: the transposes (dit_kernels.cu:19-47), linear_fp32_row (:79-93), the head's RMSNorm + modulate
// (the norm prologue of the activation quantiser) and the host-side time vector (distill.cpp:126-150).
#include <cublasLt.h>
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <list>
#include <map>
#include <new>
#include <mutex>
#include <string>
#include <system_error>
#include <thread>
#include <vector>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int kTile = 32;
constexpr int kFreq = 256;
constexpr std::size_t kLtWorkspaceBytes = std::size_t{4} << 20;
constexpr int kParamWords = 1000;  // 32-bit words a launch carries by value (kernel parameters hold 4 KB)

// Small host arrays reach the device as kernel parameters (copied at launch: no pinned staging buffer, nothing the
// caller must keep alive, capturable), as the reference's write_params does (dit_kernels.cu:121-123).
struct ParamWords {
  std::uint32_t words[kParamWords];
};
__global__ void write_words_kernel(std::uint32_t* dst, const ParamWords p, int n) {
  for (int i = static_cast<int>(threadIdx.x); i < n; i += static_cast<int>(blockDim.x)) dst[i] = p.words[i];
}
int write_words(const char* op, void* dst, const void* src, std::size_t words, cudaStream_t stream) {
  const std::uint32_t* from = static_cast<const std::uint32_t*>(src);
  for (std::size_t at = 0; at < words; at += kParamWords) {
    const int n = static_cast<int>(std::min<std::size_t>(kParamWords, words - at));
    ParamWords p;
    std::memcpy(p.words, from + at, static_cast<std::size_t>(n) * 4);
    write_words_kernel<<<1, 256, 0, stream>>>(static_cast<std::uint32_t*>(dst) + at, p, n);
    if (const int rc = check_launch(op)) return rc;
  }
  return B2_OK;
}

// kernels::silu (src/kernels/basic/elementwise.cu:92-100, detail.h:100): bf16(x / (1 + expf(-x))), the division and the
// addition each rounded once.
__global__ void silu_bf16_kernel(const __nv_bfloat16* x, __nv_bfloat16* out, std::int64_t n) {
  for (std::int64_t i = static_cast<std::int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<std::int64_t>(gridDim.x) * blockDim.x) {
    const float v = __bfloat162float(x[i]);
    out[i] = __float2bfloat16_rn(__fdiv_rn(v, __fadd_rn(1.0f, expf(-v))));
  }
}

// out[c * ld + r] = convert(in[r * cols + c]): a [rows, cols] row-major matrix transposed through a padded shared tile,
// f32 -> bf16 (round to nearest even) or bf16 -> f32.
template <typename In, typename Out>
__global__ void __launch_bounds__(kTile * 8) transpose_kernel(const In* in, Out* out, std::int64_t rows, std::int64_t cols, std::int64_t ld) {
  __shared__ float tile[kTile][kTile + 1];
  const std::int64_t r0 = static_cast<std::int64_t>(blockIdx.y) * kTile, c0 = static_cast<std::int64_t>(blockIdx.x) * kTile;
  const int tx = static_cast<int>(threadIdx.x);
  for (int i = static_cast<int>(threadIdx.y); i < kTile; i += 8) {
    const std::int64_t r = r0 + i, c = c0 + tx;
    if (r < rows && c < cols) {
      if constexpr (std::is_same_v<In, float>) tile[i][tx] = in[r * cols + c];
      else tile[i][tx] = __bfloat162float(in[r * cols + c]);
    }
  }
  __syncthreads();
  for (int i = static_cast<int>(threadIdx.y); i < kTile; i += 8) {
    const std::int64_t c = c0 + i, r = r0 + tx;
    if (r < rows && c < cols) {
      if constexpr (std::is_same_v<Out, float>) out[c * ld + r] = tile[tx][i];
      else out[c * ld + r] = __float2bfloat16_rn(tile[tx][i]);
    }
  }
}

template <typename In, typename Out>
int launch_transpose(const char* op, const In* in, Out* out, std::int64_t rows, std::int64_t cols, std::int64_t ld, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B2_OK;
  const dim3 grid(static_cast<unsigned>((cols + kTile - 1) / kTile), static_cast<unsigned>((rows + kTile - 1) / kTile));
  transpose_kernel<In, Out><<<grid, dim3(kTile, 8), 0, stream>>>(in, out, rows, cols, ld);
  return check_launch(op);
}

// One warp per output row, 8 weights per 16-byte load: lane l takes chunks l, l + 32, ... and accumulates with one fma
// per weight in column order; the 32 partial sums meet in a butterfly of adds (offsets 16, 8, 4, 2, 1);
// out = bf16(sum + bias). The order of every operation is the reference kernel's, so the bits are.
__global__ void __launch_bounds__(256) linear_fp32_row_kernel(const __nv_bfloat16* w, const float* x, const float* bias,
                                                              __nv_bfloat16* out, int n, int k) {
  const int row = static_cast<int>(blockIdx.x) * (static_cast<int>(blockDim.x) / 32) + static_cast<int>(threadIdx.x) / 32;
  const int lane = static_cast<int>(threadIdx.x) % 32;
  if (row >= n) return;
  const uint4* wr = reinterpret_cast<const uint4*>(w + static_cast<std::int64_t>(row) * k);
  float acc = 0.0f;
  for (int i = lane; i < k / 8; i += 32) {
    const uint4 v = wr[i];
    const std::uint32_t words[4] = {v.x, v.y, v.z, v.w};
    const float4 x0 = reinterpret_cast<const float4*>(x)[2 * i], x1 = reinterpret_cast<const float4*>(x)[2 * i + 1];
    const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc = fmaf(__uint_as_float(words[j] << 16), xs[2 * j], acc);
      acc = fmaf(__uint_as_float(words[j] & 0xFFFF0000u), xs[2 * j + 1], acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o /= 2) acc = fadd(acc, __shfl_xor_sync(0xffffffffu, acc, o));
  if (lane == 0) out[row] = __float2bfloat16_rn(fadd(acc, bias[row]));
}

// ------------------------------------------------------------------------------------------------ cuBLASLt, bound late

struct LtApi {
  cublasStatus_t (*create)(cublasLtHandle_t*);
  cublasStatus_t (*desc_create)(cublasLtMatmulDesc_t*, cublasComputeType_t, cudaDataType_t);
  cublasStatus_t (*desc_destroy)(cublasLtMatmulDesc_t);
  cublasStatus_t (*desc_set)(cublasLtMatmulDesc_t, cublasLtMatmulDescAttributes_t, const void*, size_t);
  cublasStatus_t (*layout_create)(cublasLtMatrixLayout_t*, cudaDataType, uint64_t, uint64_t, int64_t);
  cublasStatus_t (*layout_destroy)(cublasLtMatrixLayout_t);
  cublasStatus_t (*pref_create)(cublasLtMatmulPreference_t*);
  cublasStatus_t (*pref_destroy)(cublasLtMatmulPreference_t);
  cublasStatus_t (*pref_set)(cublasLtMatmulPreference_t, cublasLtMatmulPreferenceAttributes_t, const void*, size_t);
  cublasStatus_t (*heuristic)(cublasLtHandle_t, cublasLtMatmulDesc_t, cublasLtMatrixLayout_t, cublasLtMatrixLayout_t,
                              cublasLtMatrixLayout_t, cublasLtMatrixLayout_t, cublasLtMatmulPreference_t, int,
                              cublasLtMatmulHeuristicResult_t*, int*);
  cublasStatus_t (*matmul)(cublasLtHandle_t, cublasLtMatmulDesc_t, const void*, const void*, cublasLtMatrixLayout_t, const void*,
                           cublasLtMatrixLayout_t, const void*, const void*, cublasLtMatrixLayout_t, void*,
                           cublasLtMatrixLayout_t, const cublasLtMatmulAlgo_t*, void*, size_t, cudaStream_t);
  bool ok = false;
};

// The library a process already holds (a Python process with torch does) comes first, then the loader's search path,
// then the toolkit's usual place.
const LtApi& lt() {
  static LtApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libcublasLt.so.12", RTLD_NOW | RTLD_NOLOAD);
    if (h == nullptr) h = dlopen("libcublasLt.so.12", RTLD_NOW);
    if (h == nullptr) h = dlopen("/usr/local/cuda/lib64/libcublasLt.so.12", RTLD_NOW);
    if (h == nullptr) return;
    bool all = true;
    const auto bind = [&](auto& fn, const char* name) {
      fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(h, name));
      all = all && fn != nullptr;
    };
    bind(api.create, "cublasLtCreate");
    bind(api.desc_create, "cublasLtMatmulDescCreate");
    bind(api.desc_destroy, "cublasLtMatmulDescDestroy");
    bind(api.desc_set, "cublasLtMatmulDescSetAttribute");
    bind(api.layout_create, "cublasLtMatrixLayoutCreate");
    bind(api.layout_destroy, "cublasLtMatrixLayoutDestroy");
    bind(api.pref_create, "cublasLtMatmulPreferenceCreate");
    bind(api.pref_destroy, "cublasLtMatmulPreferenceDestroy");
    bind(api.pref_set, "cublasLtMatmulPreferenceSetAttribute");
    bind(api.heuristic, "cublasLtMatmulAlgoGetHeuristic");
    bind(api.matmul, "cublasLtMatmul");
    api.ok = all;
  });
  return api;
}

// fn(r0, r1) over [0, rows) in up to eight contiguous pieces, one host thread each (the caller's thread takes the first);
// a host that cannot start a thread runs that piece itself.
template <typename Fn>
void rows_in_parallel(std::int64_t rows, Fn fn) {
  const unsigned hw = std::thread::hardware_concurrency();
  const std::int64_t pieces = rows < 1024 ? 1 : std::max<std::int64_t>(1, std::min<std::int64_t>(8, hw == 0 ? 1 : hw));
  const std::int64_t per = (rows + pieces - 1) / pieces;
  std::vector<std::thread> workers;
  for (std::int64_t i = 1; i < pieces; ++i) {
    const std::int64_t r0 = std::min(rows, i * per), r1 = std::min(rows, (i + 1) * per);
    if (r0 >= r1) break;
    try {
      workers.emplace_back([=] { fn(r0, r1); });
    } catch (const std::system_error&) {
      fn(r0, r1);
    }
  }
  fn(0, std::min(rows, per));
  for (std::thread& w : workers) w.join();
}

int lt_handle(cublasLtHandle_t* out) {
  static std::mutex mu;
  static std::map<int, cublasLtHandle_t> handles;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  auto it = handles.find(dev);
  if (it == handles.end()) {
    cublasLtHandle_t h = nullptr;
    if (lt().create(&h) != CUBLAS_STATUS_SUCCESS) return fail_status(B2_ERR_NOT_SUPPORTED, "linear_bf16", "cublasLtCreate failed");
    it = handles.emplace(dev, h).first;
  }
  *out = it->second;
  return B2_OK;
}

// ------------------------------------------------------------------------------------------------ forward: host plan

struct Run {
  int r0, r1;        // rows [r0, r1)
  std::int64_t t0, t1;
  int cu_at;         // index of its first entry in the cu_seqlens array (and in the cu_seqlens_k array)
  int max_len;
  bool slot_a = false, slot_b = false;  // with reference images: which slots its key rows reach
};

std::size_t align_up(std::size_t v) { return (v + 255) & ~static_cast<std::size_t>(255); }

struct Carve {
  std::size_t x, rope, mod, head, time, tokens, y, cu, lt, block, total;
};

int check_extension(const char* op, const b2_dit_model* m) {
  if (m->ext_w == nullptr) return B2_OK;
  if (m->ext_bias == nullptr || m->ext_channels <= 0 || m->ext_channels % 8 != 0 || m->ext_channels > 4096) {
    return fail_invalid(op, "an input extension needs a bias and 8, 16, ... extra channels");
  }
  return B2_OK;
}

// embed_video (moss_dit.cpp:1100-1118): latent plane [128, hw] (+ the extension's plane [c, hw], or zeros for it when
// `extra` is null) -> tokens -> linear -> rows of x.
int embed_video(const b2_dit_model& m, const float* plane, const float* extra, std::int64_t hw, __nv_bfloat16* tokens,
                __nv_bfloat16* dst, void* lt_ws, cudaStream_t stream) {
  const char* op = "dit_forward";
  const std::int64_t D = m.D;
  if (m.ext_w == nullptr) {
    if (const int rc = b2_latent_to_tokens(plane, 128, hw, tokens, 128, stream)) return rc;
    return b2_linear_bf16(tokens, 128, m.video_w, m.video_bias, dst, D, hw, static_cast<int>(D), 128, lt_ws, kLtWorkspaceBytes, stream);
  }
  const int cin = 128 + m.ext_channels;
  if (const int rc = b2_latent_to_tokens(plane, 128, hw, tokens, cin, stream)) return rc;
  if (extra != nullptr) {
    if (const int rc = b2_latent_to_tokens(extra, m.ext_channels, hw, tokens + 128, cin, stream)) return rc;
  } else if (const cudaError_t e = cudaMemset2DAsync(tokens + 128, static_cast<std::size_t>(cin) * 2, 0, static_cast<std::size_t>(m.ext_channels) * 2,
                                                     static_cast<std::size_t>(hw), stream); e != cudaSuccess) {
    return fail_cuda(op, e);
  }
  return b2_linear_bf16(tokens, cin, m.ext_w, m.ext_bias, dst, D, hw, static_cast<int>(D), cin, lt_ws, kLtWorkspaceBytes, stream);
}

int plan_forward(const char* op, const b2_dit_model* m, const b2_forward* f, std::vector<std::int64_t>* off, Carve* c,
                 b2_block_run* widest) {
  if (m == nullptr || f == nullptr || m->struct_size < sizeof(b2_dit_model) || f->struct_size < offsetof(b2_forward, mod)) {
    return fail_invalid(op, "null model or forward, or one from an older header");
  }
  if (m->blocks == nullptr || m->num_blocks < 0 || m->num_blocks > 64) return fail_invalid(op, "0..64 blocks (skip masks are 64 bits)");
  if (m->D != 3072 || m->heads != 24 || m->latent_channels != 128) {
    return fail_invalid(op, "the MOSS-Image DiT has D = 3072, 24 heads and 128 latent channels");
  }
  if (f->height < 1 || f->width < 1 || f->num_latents < 1 || f->num_rows < 1 || f->num_rows > 8 || f->rows == nullptr) {
    return fail_invalid(op, "needs a latent grid, 1..8 rows and at least one latent");
  }
  if (const int rc = check_extension(op, m)) return rc;
  if (m->ext_w != nullptr && f->extra == nullptr) return fail_invalid(op, "the model's input extension needs the forward's extra latents");
  const std::int64_t R = f->ref_tokens;
  if (R < 0 || (R > 0) != (f->ref_kv != nullptr)) return fail_invalid(op, "ref_kv and ref_tokens go together");
  if (R > 0 && (f->num_latents != 1 || f->num_rows > 2)) {
    return fail_invalid(op, "a forward with reference images takes one latent and at most 2 rows");
  }
  const std::int64_t hw = static_cast<std::int64_t>(f->height) * f->width;
  off->assign(1, 0);
  int max_len = 0;
  for (int r = 0; r < f->num_rows; ++r) {
    const b2_forward_row& row = f->rows[r];
    if (row.text == nullptr || row.text_len < 1 || row.out == nullptr) return fail_invalid(op, "a row needs text [S >= 1, 3072] and an output");
    if (row.latent < 0 || row.latent >= f->num_latents) return fail_invalid(op, "a row reads a latent that is not there");
    off->push_back(off->back() + hw + row.text_len);
    max_len = std::max<std::int64_t>(max_len, hw + row.text_len);
  }
  const std::int64_t total = off->back();
  if (total > 0x7fffffff) return fail_invalid(op, "too many joint tokens");
  *widest = b2_block_run{};
  widest->struct_size = sizeof(b2_block_run);
  widest->tokens = total, widest->D = m->D, widest->F = m->F, widest->heads = m->heads, widest->batch = f->num_rows;
  widest->max_seqlen = max_len, widest->tier = f->tier, widest->attention = f->attention, widest->fused_norm_rope = -1;
  static const std::int32_t placeholder = 0;  // sizing reads no offsets; every run of the forward brings its own
  widest->cu_seqlens = &placeholder;
  if (R > 0) {
    widest->slot_rows = R, widest->slot_kv[0] = widest->slot_kv[1] = &placeholder, widest->cu_seqlens_k = &placeholder;
    widest->k0 = 0, widest->k1 = total + 2 * R, widest->max_seqlen = static_cast<int>(max_len + R);
  }
  const std::size_t block_bytes = b2_block_quant_workspace_bytes(widest);
  if (block_bytes == 0) return B2_ERR_INVALID_ARGUMENT;  // the block's own message stands
  const std::size_t D = static_cast<std::size_t>(m->D);
  std::size_t at = 0;
  const auto take = [&](std::size_t bytes) {
    const std::size_t here = at;
    at += align_up(bytes);
    return here;
  };
  c->x = take(static_cast<std::size_t>(total) * D * 2);
  c->rope = take(static_cast<std::size_t>(total) * 128 * 2);
  c->mod = take(6 * D * 2);
  c->head = take(2 * D * 2);
  c->time = take(D * 4);
  c->tokens = take(static_cast<std::size_t>(hw) * static_cast<std::size_t>(128 + (m->ext_w != nullptr ? m->ext_channels : 0)) * 2);
  c->y = take(static_cast<std::size_t>(hw) * D * 2);
  c->cu = take(static_cast<std::size_t>(f->num_rows + 1) * (f->num_rows * (f->num_rows + 1) / 2) * 4 * 2);  // cu_seqlens and cu_seqlens_k
  c->lt = take(kLtWorkspaceBytes);
  c->block = take(block_bytes);
  c->total = at;
  return B2_OK;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" {

int b2_latent_to_tokens(const float* latents, int channels, int64_t hw, void* tokens, int64_t ld, void* stream) {
  constexpr const char* op = "latent_to_tokens";
  if (channels < 0 || hw < 0 || ld < channels) return fail_invalid(op, "needs channels, hw >= 0 and ld >= channels");
  if (channels > 0 && hw > 0 && (latents == nullptr || tokens == nullptr)) return fail_invalid(op, "null operand");
  return launch_transpose(op, latents, static_cast<__nv_bfloat16*>(tokens), channels, hw, ld, as_stream(stream));
}

int b2_tokens_to_latent(const void* tokens, float* latents, int channels, int64_t hw, void* stream) {
  constexpr const char* op = "tokens_to_latent";
  if (channels < 0 || hw < 0) return fail_invalid(op, "needs channels, hw >= 0");
  if (channels > 0 && hw > 0 && (latents == nullptr || tokens == nullptr)) return fail_invalid(op, "null operand");
  return launch_transpose(op, static_cast<const __nv_bfloat16*>(tokens), latents, hw, channels, hw, as_stream(stream));
}

int b2_linear_fp32_row(const void* w, const float* x, const float* bias, void* out, int n, int k, void* stream) {
  constexpr const char* op = "linear_fp32_row";
  if (n < 0 || k <= 0 || k % 8 != 0) return fail_invalid(op, "needs n >= 0 and k a positive multiple of 8");
  if (n == 0) return B2_OK;
  if (w == nullptr || x == nullptr || bias == nullptr || out == nullptr || !aligned_to(w, 16) || !aligned_to(x, 16)) {
    return fail_invalid(op, "needs a 16-byte aligned bf16 w [n, k], a 16-byte aligned f32 x [k], an f32 bias [n] and a bf16 out [n]");
  }
  linear_fp32_row_kernel<<<static_cast<unsigned>((n + 7) / 8), 256, 0, as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(w), x, bias, static_cast<__nv_bfloat16*>(out), n, k);
  return check_launch(op);
}

int b2_time_sinusoid(float timestep, float* emb) {
  if (emb == nullptr) return fail_invalid("time_sinusoid", "null output");
  constexpr int kHalf = kFreq / 2;
  for (int i = 0; i < kHalf; ++i) {
    const double freq = std::pow(10000.0, -static_cast<double>(i) / kHalf);
    const double phase = static_cast<double>(timestep) * freq;
    emb[i] = static_cast<float>(std::cos(phase));
    emb[kHalf + i] = static_cast<float>(std::sin(phase));
  }
  return B2_OK;
}

int b2_time_vector_fp32(const b2_time_embedding* te, float timestep, float* time) {
  constexpr const char* op = "time_vector_fp32";
  if (te == nullptr || te->struct_size < sizeof(b2_time_embedding) || time == nullptr) return fail_invalid(op, "null argument");
  if (te->w0 == nullptr || te->b0 == nullptr || te->w2 == nullptr || te->b2 == nullptr || te->dim < 1) {
    return fail_invalid(op, "needs w0 [dim, 256], b0 [dim], w2 [dim, dim], b2 [dim] on the host");
  }
  float emb[kFreq];
  b2_time_sinusoid(timestep, emb);
  const std::int64_t dim = te->dim;
  try {
    std::vector<float> h(static_cast<std::size_t>(dim));
    // Rows are independent and each one is summed in the reference's order, so splitting them over a few host threads
    // changes no bit (about 10 ms on one core for dim 3072, most of it the second linear).
    rows_in_parallel(dim, [&](std::int64_t r0, std::int64_t r1) {
      for (std::int64_t r = r0; r < r1; ++r) {
        double acc = te->b0[r];
        const float* w = te->w0 + r * kFreq;
        for (int c = 0; c < kFreq; ++c) acc += static_cast<double>(w[c]) * emb[c];
        const float v = static_cast<float>(acc);
        h[static_cast<std::size_t>(r)] = v / (1.0f + std::exp(-v));  // silu
      }
    });
    rows_in_parallel(dim, [&](std::int64_t r0, std::int64_t r1) {
      for (std::int64_t r = r0; r < r1; ++r) {
        double acc = te->b2[r];
        const float* w = te->w2 + r * dim;
        for (std::int64_t c = 0; c < dim; ++c) acc += static_cast<double>(w[c]) * h[static_cast<std::size_t>(c)];
        time[r] = static_cast<float>(acc);
      }
    });
  } catch (const std::exception& e) {  // nothing may cross the C boundary
    return fail_status(B2_ERR_INTERNAL, op, e.what());
  }
  return B2_OK;
}

size_t b2_linear_bf16_workspace_bytes(void) { return kLtWorkspaceBytes; }

int b2_silu_bf16(const void* x, void* out, int64_t n, void* stream) {
  constexpr const char* op = "silu_bf16";
  if (n < 0 || (n > 0 && (x == nullptr || out == nullptr))) return fail_invalid(op, "needs bf16 x and out of n values");
  if (n == 0) return B2_OK;
  const unsigned blocks = static_cast<unsigned>(std::min<std::int64_t>((n + 255) / 256, 4096));
  silu_bf16_kernel<<<blocks, 256, 0, as_stream(stream)>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n);
  return check_launch(op);
}

size_t b2_time_modulation_bf16_workspace_bytes(const b2_time_mlp_bf16* m) {
  if (m == nullptr || m->dim < 8) return 0;
  return 1024 + 2 * align_up(static_cast<std::size_t>(m->dim) * 2) + kLtWorkspaceBytes;
}

int b2_time_modulation_bf16(const b2_time_mlp_bf16* m, float timestep, void* mod, void* head, void* workspace,
                            size_t workspace_bytes, void* stream) {
  constexpr const char* op = "time_modulation_bf16";
  if (m == nullptr || m->struct_size < sizeof(b2_time_mlp_bf16) || mod == nullptr || head == nullptr) return fail_invalid(op, "null argument");
  if (m->dim < 8 || m->dim % 8 != 0 || m->dim > (1 << 16) || m->in_w == nullptr || m->out_w == nullptr || m->block_mod_w == nullptr ||
      m->head_mod_w == nullptr) {
    return fail_invalid(op, "needs the four bf16 weights of the timestep MLP and the modulation linears, dim a multiple of 8");
  }
  if (workspace == nullptr || !aligned_to(workspace, 256) || workspace_bytes < b2_time_modulation_bf16_workspace_bytes(m)) {
    return fail_invalid(op, "workspace must be 256-byte aligned and hold b2_time_modulation_bf16_workspace_bytes()");
  }
  // The sinusoid in double, rounded to fp32 and then to bf16 (moss_dit.cpp:979-985).
  float emb[kFreq];
  b2_time_sinusoid(timestep, emb);
  std::uint32_t packed[kFreq / 2];
  for (int i = 0; i < kFreq; i += 2) {
    const auto bits = [](float v) {
      std::uint32_t u;
      std::memcpy(&u, &v, 4);
      return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
    };
    packed[i / 2] = bits(emb[i]) | (bits(emb[i + 1]) << 16);
  }
  unsigned char* base = static_cast<unsigned char*>(workspace);
  const std::size_t row = align_up(static_cast<std::size_t>(m->dim) * 2);
  void *t_in = base, *hidden = base + 1024, *time = base + 1024 + row, *lt_ws = base + 1024 + 2 * row;
  const int D = static_cast<int>(m->dim);
  if (const int rc = write_words(op, t_in, packed, kFreq / 2, as_stream(stream))) return rc;
  if (const int rc = b2_linear_bf16(t_in, kFreq, m->in_w, m->in_bias, hidden, D, 1, D, kFreq, lt_ws, kLtWorkspaceBytes, stream)) return rc;
  if (const int rc = b2_silu_bf16(hidden, hidden, D, stream)) return rc;
  if (const int rc = b2_linear_bf16(hidden, D, m->out_w, m->out_bias, time, D, 1, D, D, lt_ws, kLtWorkspaceBytes, stream)) return rc;
  if (const int rc = b2_linear_bf16(time, D, m->block_mod_w, m->block_mod_bias, mod, 6 * D, 1, 6 * D, D, lt_ws, kLtWorkspaceBytes, stream)) return rc;
  return b2_linear_bf16(time, D, m->head_mod_w, m->head_mod_bias, head, 2 * D, 1, 2 * D, D, lt_ws, kLtWorkspaceBytes, stream);
}

int b2_linear_bf16(const void* x, int64_t ldx, const void* w, const void* bias, void* out, int64_t ldo, int64_t m, int n,
                   int k, void* workspace, size_t workspace_bytes, void* stream) {
  constexpr const char* op = "linear_bf16";
  if (m < 0 || n <= 0 || k <= 0 || ldx < k || ldo < n || k % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) {
    return fail_invalid(op, "needs m >= 0, n, k > 0, k, ldx, ldo multiples of 8, ldx >= k and ldo >= n");
  }
  if (m == 0) return B2_OK;
  if (x == nullptr || w == nullptr || out == nullptr || !aligned_to(x, 16) || !aligned_to(w, 16) || !aligned_to(out, 16) ||
      (bias != nullptr && !aligned_to(bias, 16))) {
    return fail_invalid(op, "needs 16-byte aligned bf16 x [m, k], w [n, k], out [m, n] (bias bf16 [n] or NULL)");
  }
  if (workspace_bytes > 0 && (workspace == nullptr || !aligned_to(workspace, 256))) return fail_invalid(op, "workspace must be 256-byte aligned");
  const LtApi& api = lt();
  if (!api.ok) return fail_status(B2_ERR_NOT_SUPPORTED, op, "libcublasLt.so.12 was not found");
  cublasLtHandle_t handle = nullptr;
  if (const int rc = lt_handle(&handle)) return rc;
  // Row-major out [m, n] = x [m, k] * w [n, k]^T is column-major out^T [n, m] = w^T-as-stored (op T) * x-as-stored.
  cublasLtMatmulDesc_t desc = nullptr;
  cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
  cublasLtMatmulPreference_t pref = nullptr;
  cublasStatus_t st = api.desc_create(&desc, CUBLAS_COMPUTE_32F, CUDA_R_32F);
  const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
  if (st == CUBLAS_STATUS_SUCCESS) st = api.desc_set(desc, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof ta);
  if (st == CUBLAS_STATUS_SUCCESS) st = api.desc_set(desc, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof tb);
  if (st == CUBLAS_STATUS_SUCCESS && bias != nullptr) {
    const cublasLtEpilogue_t ep = CUBLASLT_EPILOGUE_BIAS;
    st = api.desc_set(desc, CUBLASLT_MATMUL_DESC_EPILOGUE, &ep, sizeof ep);
    if (st == CUBLAS_STATUS_SUCCESS) st = api.desc_set(desc, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof bias);
  }
  if (st == CUBLAS_STATUS_SUCCESS) st = api.layout_create(&la, CUDA_R_16BF, static_cast<uint64_t>(k), static_cast<uint64_t>(n), k);
  if (st == CUBLAS_STATUS_SUCCESS) st = api.layout_create(&lb, CUDA_R_16BF, static_cast<uint64_t>(k), static_cast<uint64_t>(m), ldx);
  if (st == CUBLAS_STATUS_SUCCESS) st = api.layout_create(&lc, CUDA_R_16BF, static_cast<uint64_t>(n), static_cast<uint64_t>(m), ldo);
  if (st == CUBLAS_STATUS_SUCCESS) st = api.pref_create(&pref);
  if (st == CUBLAS_STATUS_SUCCESS) st = api.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes, sizeof workspace_bytes);
  cublasLtMatmulHeuristicResult_t found{};
  int count = 0;
  if (st == CUBLAS_STATUS_SUCCESS) st = api.heuristic(handle, desc, la, lb, lc, lc, pref, 1, &found, &count);
  if (st == CUBLAS_STATUS_SUCCESS && count == 0) st = CUBLAS_STATUS_NOT_SUPPORTED;
  const float one = 1.0f, zero = 0.0f;
  if (st == CUBLAS_STATUS_SUCCESS) {
    st = api.matmul(handle, desc, &one, w, la, x, lb, &zero, out, lc, out, lc, &found.algo, workspace, workspace_bytes,
                    as_stream(stream));
  }
  if (pref != nullptr) api.pref_destroy(pref);
  if (lc != nullptr) api.layout_destroy(lc);
  if (lb != nullptr) api.layout_destroy(lb);
  if (la != nullptr) api.layout_destroy(la);
  if (desc != nullptr) api.desc_destroy(desc);
  if (st != CUBLAS_STATUS_SUCCESS) return fail_status(B2_ERR_CUDA, op, "cuBLASLt status " + std::to_string(static_cast<int>(st)));
  return B2_OK;
}

size_t b2_dit_forward_workspace_bytes(const b2_dit_model* model, const b2_forward* forward) {
  std::vector<std::int64_t> off;
  Carve c{};
  b2_block_run widest{};
  if (plan_forward("dit_forward_workspace_bytes", model, forward, &off, &c, &widest) != B2_OK) return 0;
  return c.total;
}

namespace {
int dit_forward_impl(const b2_dit_model* model, const b2_forward* forward, const float* time_device, void* stream_);
}

int b2_dit_forward(const b2_dit_model* model, const b2_forward* forward, void* stream) {
  try {
    return dit_forward_impl(model, forward, nullptr, stream);
  } catch (const std::exception& e) {  // host containers may throw; nothing may cross the C boundary
    return fail_status(B2_ERR_INTERNAL, "dit_forward", e.what());
  }
}

namespace {
// time_device: the time vector already on the device (fp32 [D]), read in place of forward->time_vector; a captured
// forward takes it so that its graph does not freeze one step's time vector.
int dit_forward_impl(const b2_dit_model* model, const b2_forward* forward, const float* time_device, void* stream_) {
  constexpr const char* op = "dit_forward";
  std::vector<std::int64_t> off;
  Carve c{};
  b2_block_run widest{};
  if (const int rc = plan_forward(op, model, forward, &off, &c, &widest)) return rc;
  const b2_dit_model& m = *model;
  const b2_forward& f = *forward;
  // The modulation vectors computed by the caller (b2_time_modulation_bf16, or anything else), when the struct has them.
  const bool given = f.struct_size >= sizeof(b2_forward) && f.mod != nullptr && f.head != nullptr;
  if (f.struct_size >= sizeof(b2_forward) && (f.mod != nullptr) != (f.head != nullptr)) return fail_invalid(op, "mod and head go together");
  if (f.latents == nullptr || (!given && f.time_vector == nullptr && time_device == nullptr)) {
    return fail_invalid(op, "needs latents and the host time vector (or mod and head)");
  }
  if ((!given && (m.block_mod_w == nullptr || m.block_mod_bias == nullptr || m.head_mod_w == nullptr || m.head_mod_bias == nullptr)) ||
      (m.video_w == nullptr && m.ext_w == nullptr) || m.final_norm == nullptr || m.final_w == nullptr) {
    return fail_invalid(op, "the model lacks a modulation, embedder or head tensor");
  }
  if (f.workspace == nullptr || !aligned_to(f.workspace, 256) || f.workspace_bytes < c.total) {
    return fail_invalid(op, "workspace must be 256-byte aligned and hold b2_dit_forward_workspace_bytes() = " + std::to_string(c.total));
  }
  cudaStream_t stream = as_stream(stream_);
  const std::int64_t hw = static_cast<std::int64_t>(f.height) * f.width, D = m.D;
  unsigned char* base = static_cast<unsigned char*>(f.workspace);
  __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(base + c.x);
  __nv_bfloat16* rope = reinterpret_cast<__nv_bfloat16*>(base + c.rope);
  __nv_bfloat16* mod = given ? static_cast<__nv_bfloat16*>(const_cast<void*>(f.mod)) : reinterpret_cast<__nv_bfloat16*>(base + c.mod);
  __nv_bfloat16* head = given ? static_cast<__nv_bfloat16*>(const_cast<void*>(f.head)) : reinterpret_cast<__nv_bfloat16*>(base + c.head);
  const float* time = time_device != nullptr ? time_device : reinterpret_cast<const float*>(base + c.time);
  __nv_bfloat16* tokens = reinterpret_cast<__nv_bfloat16*>(base + c.tokens);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(base + c.y);
  std::int32_t* cu_dev = reinterpret_cast<std::int32_t*>(base + c.cu);

  // The runs of contiguous rows that execute each block, one varlen batch each with zero-based cu_seqlens; a run that
  // recurs (the usual case: no skips, one run over all rows) is described once.
  std::vector<std::int32_t> cu, cu_k;
  const std::int64_t R = f.ref_tokens;
  std::map<std::pair<int, int>, Run> unique;
  std::vector<std::vector<Run>> block_runs(static_cast<std::size_t>(m.num_blocks));
  for (int bi = 0; bi < m.num_blocks; ++bi) {
    const auto skips = [&](int r) { return ((f.rows[r].skip >> bi) & 1u) != 0; };
    for (int r0 = 0; r0 < f.num_rows;) {
      if (skips(r0)) {
        ++r0;
        continue;
      }
      int r1 = r0;
      while (r1 < f.num_rows && !skips(r1)) ++r1;
      auto it = unique.find({r0, r1});
      if (it == unique.end()) {
        Run run{r0, r1, off[static_cast<std::size_t>(r0)], off[static_cast<std::size_t>(r1)], static_cast<int>(cu.size()), 0};
        for (int r = r0; r <= r1; ++r) {
          cu.push_back(static_cast<std::int32_t>(off[static_cast<std::size_t>(r)] - off[static_cast<std::size_t>(r0)]));
          // With reference images sequence j of the run also has j slots of R rows before its keys begin: the first
          // sequence takes slot A when the run starts at row 0, every other one slot B (moss_dit.cpp:1283-1300).
          cu_k.push_back(static_cast<std::int32_t>(cu.back() + static_cast<std::int64_t>(r - r0) * R));
          if (r < r1) run.max_len = std::max<int>(run.max_len, static_cast<int>(off[static_cast<std::size_t>(r) + 1] - off[static_cast<std::size_t>(r)]));
        }
        if (R > 0) {
          run.slot_a = r0 == 0;
          run.slot_b = r1 - r0 == 2 || !run.slot_a;
          run.max_len += static_cast<int>(R);
        }
        it = unique.emplace(std::make_pair(r0, r1), run).first;
      }
      block_runs[static_cast<std::size_t>(bi)].push_back(it->second);
      r0 = r1;
    }
  }
  if (const int rc = write_words(op, cu_dev, cu.data(), cu.size(), stream)) return rc;
  std::int32_t* cu_k_dev = cu_dev + cu.size();
  if (R > 0) {
    if (const int rc = write_words(op, cu_k_dev, cu_k.data(), cu_k.size(), stream)) return rc;
  }
  // time_modulation: the time vector (host, fp32) through the two modulation linears.
  if (!given) {
    if (time_device == nullptr) {
      if (const int rc = write_words(op, base + c.time, f.time_vector, static_cast<std::size_t>(D), stream)) return rc;
    }
    if (const int rc = b2_linear_fp32_row(m.block_mod_w, time, m.block_mod_bias, mod, static_cast<int>(6 * D), static_cast<int>(D), stream)) return rc;
    if (const int rc = b2_linear_fp32_row(m.head_mod_w, time, m.head_mod_bias, head, static_cast<int>(2 * D), static_cast<int>(D), stream)) return rc;
  }

  // Joint inputs [video_r | text_r] and per-row RoPE tables. The video embedding is the same for every row of a latent:
  // computed once, into the first row that reads the latent, and copied to its other rows.
  const std::size_t row_bytes = static_cast<std::size_t>(D) * 2;
  for (int r = 0; r < f.num_rows; ++r) {
    int src = r;
    for (int q = 0; q < r; ++q) {
      if (f.rows[q].latent == f.rows[r].latent) {
        src = q;
        break;
      }
    }
    __nv_bfloat16* xr = x + off[static_cast<std::size_t>(r)] * D;
    if (src == r) {
      const std::size_t l = static_cast<std::size_t>(f.rows[r].latent), plane_size = static_cast<std::size_t>(hw);
      const float* plane = f.latents + l * 128 * plane_size;
      const float* extra = m.ext_w != nullptr ? f.extra + l * static_cast<std::size_t>(m.ext_channels) * plane_size : nullptr;
      if (const int rc = embed_video(m, plane, extra, hw, tokens, xr, base + c.lt, stream)) return rc;
    } else if (const cudaError_t e = cudaMemcpyAsync(xr, x + off[static_cast<std::size_t>(src)] * D, static_cast<std::size_t>(hw) * row_bytes, cudaMemcpyDeviceToDevice, stream); e != cudaSuccess) {
      return fail_cuda(op, e);
    }
    if (const int rc = b2_moss_rope_table(rope + off[static_cast<std::size_t>(r)] * 128, 128, f.height, f.width, static_cast<int>(f.rows[r].text_len), stream)) return rc;
    if (const cudaError_t e = cudaMemcpyAsync(xr + hw * D, f.rows[r].text, static_cast<std::size_t>(f.rows[r].text_len) * row_bytes, cudaMemcpyDeviceToDevice, stream); e != cudaSuccess) {
      return fail_cuda(op, e);
    }
  }

  // The blocks.
  for (int bi = 0; bi < m.num_blocks; ++bi) {
    for (const Run& run : block_runs[static_cast<std::size_t>(bi)]) {
      b2_block_run br = widest;
      br.tokens = run.t1 - run.t0, br.batch = run.r1 - run.r0, br.max_seqlen = run.max_len, br.cu_seqlens = cu_dev + run.cu_at;
      br.slot_rows = 0, br.slot_kv[0] = br.slot_kv[1] = nullptr, br.cu_seqlens_k = nullptr, br.k0 = br.k1 = 0;
      if (R > 0) {
        // Block bi's cached reference keys and values, the same rows for both slots.
        const __nv_bfloat16* cached = static_cast<const __nv_bfloat16*>(f.ref_kv) + static_cast<std::size_t>(bi) * static_cast<std::size_t>(R) * 2 * static_cast<std::size_t>(D);
        br.slot_rows = R, br.cu_seqlens_k = cu_k_dev + run.cu_at;
        br.slot_kv[0] = run.slot_a ? cached : nullptr, br.slot_kv[1] = run.slot_b ? cached : nullptr;
        br.k0 = run.slot_a ? 0 : R, br.k1 = R + br.tokens + (run.slot_b ? R : 0);
      }
      b2_block_buffers bb{};
      bb.struct_size = sizeof bb;
      bb.x = x + run.t0 * D, bb.mod = mod, bb.rope = rope + run.t0 * 128, bb.workspace = base + c.block;
      bb.workspace_bytes = c.total - c.block;
      if (const int rc = b2_run_block_quant(&m.blocks[bi], &bb, &br, stream)) return rc;
    }
  }

  // Head: final norm with the head modulation (shift = head[0], scale = head[1]), linear, transpose.
  for (int r = 0; r < f.num_rows; ++r) {
    const __nv_bfloat16* xr = x + off[static_cast<std::size_t>(r)] * D;
    if (const int rc = b2_rms_norm_modulate(xr, D, m.final_norm, head + D, head, y, D, hw, static_cast<int>(D), stream)) return rc;
    if (const int rc = b2_linear_bf16(y, D, m.final_w, m.final_bias, tokens, 128, hw, 128, static_cast<int>(D), base + c.lt, kLtWorkspaceBytes, stream)) return rc;
    if (const int rc = b2_tokens_to_latent(tokens, f.rows[r].out, 128, hw, stream)) return rc;
  }
  return B2_OK;
}
}  // namespace

}  // extern "C"

namespace b2 {
// ------------------------------------------------------------------------------------------------ step graphs
// CUDA graphs of whole forwards (moss_dit::StepGraphs, src/models/moss_dit/dit_graph.h:14-66, over runtime::GraphCache,
// src/runtime/graph_cache.h:20-58). A graph freezes kernel arguments and addresses, so an entry's key is everything the
// enqueued work depends on except device memory contents: the model structure and its block table (weight addresses
// and shapes), the latent grid, every row (text address and length, skip set, latent index, output address), the
// tier and attention options, the workspace, the reference cache and the device. The step's time vector is the one
// host array that changes between steps of the same shape: it is written to a buffer of the cache ahead of the graph
// and the captured forward reads it from there. Entries are found by a 64-bit hash and the whole key is compared on a
// hit, so two keys with one hash run the second one eagerly rather than replaying the wrong graph.
namespace {

struct GraphEntry {
  std::uint64_t hash = 0;
  std::vector<unsigned char> key;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
};

void destroy_entry(GraphEntry& e) {
  if (e.exec != nullptr) cudaGraphExecDestroy(e.exec);
  if (e.graph != nullptr) cudaGraphDestroy(e.graph);
  e.exec = nullptr, e.graph = nullptr;
}

template <typename T>
void put(std::vector<unsigned char>* key, const T& v) {
  static_assert(std::is_trivially_copyable_v<T>, "keys are raw bytes");
  const auto* p = reinterpret_cast<const unsigned char*>(&v);
  key->insert(key->end(), p, p + sizeof(T));
}

std::uint64_t fnv1a(const std::vector<unsigned char>& key) {
  std::uint64_t h = 1469598103934665603ull;
  for (const unsigned char c : key) h = (h ^ c) * 1099511628211ull;
  return h;
}

}  // namespace
}  // namespace b2

struct b2_dit_graphs {
  std::size_t capacity = 0;
  std::list<b2::GraphEntry> lru;  // front = most recently used
  std::map<std::uint64_t, std::list<b2::GraphEntry>::iterator> by_hash;
  b2_dit_graph_stats stats{};
  float* time = nullptr;  // device fp32 [D]: the time vector of the step being enqueued
  int device = -1;
};

namespace b2 {
namespace {

// Field by field (struct padding is not part of a key).
void forward_key(const b2_dit_model& m, const b2_forward& f, int device, std::vector<unsigned char>* key) {
  key->clear();
  put(key, device);
  put(key, m.blocks), put(key, m.num_blocks), put(key, m.D), put(key, m.F), put(key, m.heads), put(key, m.latent_channels);
  put(key, m.block_mod_w), put(key, m.block_mod_bias), put(key, m.head_mod_w), put(key, m.head_mod_bias);
  put(key, m.video_w), put(key, m.video_bias), put(key, m.final_norm), put(key, m.final_w), put(key, m.final_bias);
  put(key, m.ext_w), put(key, m.ext_bias), put(key, m.ext_channels);
  for (int b = 0; b < m.num_blocks; ++b) {
    const b2_block_weights& w = m.blocks[b];
    put(key, w.norm1), put(key, w.norm2), put(key, w.q_norm), put(key, w.k_norm);
    for (const b2_linear* l : {&w.qkv, &w.o, &w.up_gate, &w.down}) {
      put(key, l->w), put(key, l->scale), put(key, l->w4);
      if (l->w4 != nullptr) {
        const b2_w4_weight& q = *l->w4;
        put(key, q.packed), put(key, q.s_rel), put(key, q.scale_kind), put(key, q.group), put(key, q.codebook), put(key, q.s_channel);
      }
    }
  }
  put(key, f.latents), put(key, f.num_latents), put(key, f.height), put(key, f.width), put(key, f.num_rows), put(key, f.tier);
  put(key, f.attention.variant), put(key, f.attention.p_range), put(key, f.attention.v_range);
  put(key, f.workspace), put(key, f.workspace_bytes), put(key, f.extra), put(key, f.ref_kv), put(key, f.ref_tokens);
  if (f.struct_size >= sizeof(b2_forward)) put(key, f.mod), put(key, f.head);
  for (int r = 0; r < f.num_rows; ++r) {
    const b2_forward_row& row = f.rows[r];
    put(key, row.text), put(key, row.text_len), put(key, row.skip), put(key, row.latent), put(key, row.out);
  }
}

int graphed_impl(b2_dit_graphs* g, const b2_dit_model* model, const b2_forward* forward, void* stream_, int* replayed) {
  constexpr const char* op = "dit_forward_graphed";
  if (replayed != nullptr) *replayed = 0;
  if (g == nullptr) return fail_invalid(op, "null cache");
  if (stream_ == nullptr) return fail_invalid(op, "capture needs a stream of its own, not the default stream");
  // Everything a caller can get wrong is refused before anything is enqueued.
  std::vector<std::int64_t> off;
  Carve c{};
  b2_block_run widest{};
  if (const int rc = plan_forward(op, model, forward, &off, &c, &widest)) return rc;
  const bool given = forward->struct_size >= sizeof(b2_forward) && forward->mod != nullptr && forward->head != nullptr;
  if (!given && forward->time_vector == nullptr) return fail_invalid(op, "needs the host time vector (or mod and head)");
  cudaStream_t stream = as_stream(stream_);
  int device = 0;
  if (const cudaError_t e = cudaGetDevice(&device); e != cudaSuccess) return fail_cuda(op, e);
  if (g->time == nullptr) {
    if (const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&g->time), static_cast<std::size_t>(model->D) * sizeof(float)); e != cudaSuccess) {
      return fail_cuda(op, e);
    }
    g->device = device;
  }
  if (g->device != device) return fail_invalid(op, "a cache belongs to the device of its first forward");
  if (!given) {
    if (const int rc = write_words(op, g->time, forward->time_vector, static_cast<std::size_t>(model->D), stream)) return rc;
  }

  std::vector<unsigned char> key;
  forward_key(*model, *forward, device, &key);
  const std::uint64_t hash = fnv1a(key);
  const auto hit = g->by_hash.find(hash);
  if (hit != g->by_hash.end()) {
    if (hit->second->key != key) {
      ++g->stats.collisions;
      return dit_forward_impl(model, forward, g->time, stream_);
    }
    g->lru.splice(g->lru.begin(), g->lru, hit->second);
    if (const cudaError_t e = cudaGraphLaunch(hit->second->exec, stream); e != cudaSuccess) return fail_cuda(op, e);
    ++g->stats.replays;
    if (replayed != nullptr) *replayed = 1;
    return B2_OK;
  }
  if (g->capacity == 0) {
    ++g->stats.eager;
    return dit_forward_impl(model, forward, g->time, stream_);
  }
  // What the library sets up once per device and cannot do inside a capture.
  cublasLtHandle_t handle = nullptr;
  if (const int rc = lt_handle(&handle)) return rc;

  GraphEntry entry;
  entry.hash = hash, entry.key = std::move(key);
  if (const cudaError_t e = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal); e != cudaSuccess) return fail_cuda(op, e);
  const int rc = dit_forward_impl(model, forward, g->time, stream_);
  const cudaError_t ended = cudaStreamEndCapture(stream, &entry.graph);
  cudaError_t made = cudaSuccess;
  if (rc == B2_OK && ended == cudaSuccess && entry.graph != nullptr) made = cudaGraphInstantiate(&entry.exec, entry.graph, 0);
  if (rc != B2_OK || ended != cudaSuccess || entry.graph == nullptr || made != cudaSuccess) {
    // Nothing of a failed capture ran. Run the forward as it is; the next call with this key tries again.
    destroy_entry(entry);
    cudaGetLastError();
    ++g->stats.eager;
    return dit_forward_impl(model, forward, g->time, stream_);
  }
  if (const cudaError_t e = cudaGraphLaunch(entry.exec, stream); e != cudaSuccess) {
    destroy_entry(entry);
    return fail_cuda(op, e);
  }
  g->lru.push_front(std::move(entry));
  g->by_hash[hash] = g->lru.begin();
  ++g->stats.captures;
  while (g->lru.size() > g->capacity) {
    g->by_hash.erase(g->lru.back().hash);
    destroy_entry(g->lru.back());
    g->lru.pop_back();
    ++g->stats.evictions;
  }
  return B2_OK;
}

void clear_graphs(b2_dit_graphs* g) {
  for (GraphEntry& e : g->lru) destroy_entry(e);
  g->lru.clear();
  g->by_hash.clear();
}

}  // namespace
}  // namespace b2

extern "C" {

int b2_dit_graphs_create(size_t capacity, b2_dit_graphs** out) {
  if (out == nullptr) return fail_invalid("dit_graphs_create", "null output");
  *out = nullptr;
  b2_dit_graphs* g = new (std::nothrow) b2_dit_graphs;
  if (g == nullptr) return fail_status(B2_ERR_INTERNAL, "dit_graphs_create", "out of host memory");
  g->capacity = capacity;
  *out = g;
  return B2_OK;
}

int b2_dit_graphs_clear(b2_dit_graphs* graphs) {
  if (graphs == nullptr) return fail_invalid("dit_graphs_clear", "null cache");
  clear_graphs(graphs);
  return B2_OK;
}

int b2_dit_graphs_destroy(b2_dit_graphs* graphs) {
  if (graphs == nullptr) return B2_OK;
  clear_graphs(graphs);
  if (graphs->time != nullptr) cudaFree(graphs->time);
  delete graphs;
  return B2_OK;
}

int b2_dit_graphs_stats(const b2_dit_graphs* graphs, b2_dit_graph_stats* stats) {
  if (graphs == nullptr || stats == nullptr) return fail_invalid("dit_graphs_stats", "null argument");
  *stats = graphs->stats;
  stats->size = graphs->lru.size();
  return B2_OK;
}

int b2_dit_forward_graphed(b2_dit_graphs* graphs, const b2_dit_model* model, const b2_forward* forward, void* stream, int* replayed) {
  try {
    return graphed_impl(graphs, model, forward, stream, replayed);
  } catch (const std::exception& e) {  // nothing may cross the C boundary
    return fail_status(B2_ERR_INTERNAL, "dit_forward_graphed", e.what());
  }
}

}  // extern "C"

extern "C" {

namespace {
struct PrefillCarve {
  std::size_t x, rope, mod, time, tokens, cu, lt, block, total;
};
int plan_prefill(const char* op, const b2_dit_model* m, const b2_prefill* f, std::int64_t* total, PrefillCarve* c, b2_block_run* run) {
  if (m == nullptr || f == nullptr || m->struct_size < sizeof(b2_dit_model) || f->struct_size < sizeof(b2_prefill)) {
    return fail_invalid(op, "null model or prefill, or one from an older header");
  }
  if (m->blocks == nullptr || m->num_blocks < 1 || m->D != 3072 || m->heads != 24 || m->latent_channels != 128) {
    return fail_invalid(op, "needs the blocks of the MOSS-Image DiT");
  }
  if (const int rc = check_extension(op, m)) return rc;
  if (f->num_refs < 1 || f->latents == nullptr || f->heights == nullptr || f->widths == nullptr) {
    return fail_invalid(op, "prefill needs at least one reference latent with its grid");
  }
  std::int64_t n = 0, widest = 0;
  for (int i = 0; i < f->num_refs; ++i) {
    if (f->latents[i] == nullptr || f->heights[i] < 1 || f->widths[i] < 1) return fail_invalid(op, "a reference latent must be [128, h, w]");
    const std::int64_t hw = static_cast<std::int64_t>(f->heights[i]) * f->widths[i];
    n += hw, widest = std::max(widest, hw);
    if (n > (1 << 20)) return fail_invalid(op, "the reference images hold too many tokens");
  }
  *total = n;
  *run = b2_block_run{};
  run->struct_size = sizeof(b2_block_run);
  run->tokens = n, run->D = m->D, run->F = m->F, run->heads = m->heads, run->batch = 1, run->max_seqlen = static_cast<int>(n);
  run->tier = f->tier, run->attention = f->attention, run->fused_norm_rope = -1;
  static const std::int32_t placeholder = 0;
  run->cu_seqlens = &placeholder;
  const std::size_t block_bytes = b2_block_quant_workspace_bytes(run);
  if (block_bytes == 0) return B2_ERR_INVALID_ARGUMENT;
  const std::size_t D = static_cast<std::size_t>(m->D);
  std::size_t at = 0;
  const auto take = [&](std::size_t bytes) {
    const std::size_t here = at;
    at += align_up(bytes);
    return here;
  };
  c->x = take(static_cast<std::size_t>(n) * D * 2);
  c->rope = take(static_cast<std::size_t>(n) * 128 * 2);
  c->mod = take(6 * D * 2);
  c->time = take(D * 4);
  c->tokens = take(static_cast<std::size_t>(widest) * static_cast<std::size_t>(128 + (m->ext_w != nullptr ? m->ext_channels : 0)) * 2);
  c->cu = take(256);
  c->lt = take(kLtWorkspaceBytes);
  c->block = take(block_bytes);
  c->total = at;
  return B2_OK;
}

int prefill_impl(const b2_dit_model* model, const b2_prefill* prefill, void* stream_) {
  constexpr const char* op = "dit_prefill_references";
  std::int64_t total = 0;
  PrefillCarve c{};
  b2_block_run run{};
  if (const int rc = plan_prefill(op, model, prefill, &total, &c, &run)) return rc;
  const b2_dit_model& m = *model;
  const b2_prefill& f = *prefill;
  if (f.time_vector == nullptr || f.kv_out == nullptr) return fail_invalid(op, "needs the host time vector and the cache to fill");
  if (m.block_mod_w == nullptr || m.block_mod_bias == nullptr || (m.video_w == nullptr && m.ext_w == nullptr)) {
    return fail_invalid(op, "the model lacks the modulation linear or the embedder");
  }
  if (f.workspace == nullptr || !aligned_to(f.workspace, 256) || f.workspace_bytes < c.total) {
    return fail_invalid(op, "workspace must be 256-byte aligned and hold b2_dit_prefill_workspace_bytes() = " + std::to_string(c.total));
  }
  cudaStream_t stream = as_stream(stream_);
  const std::int64_t D = m.D;
  unsigned char* base = static_cast<unsigned char*>(f.workspace);
  __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(base + c.x);
  __nv_bfloat16* rope = reinterpret_cast<__nv_bfloat16*>(base + c.rope);
  __nv_bfloat16* mod = reinterpret_cast<__nv_bfloat16*>(base + c.mod);
  float* time = reinterpret_cast<float*>(base + c.time);
  __nv_bfloat16* tokens = reinterpret_cast<__nv_bfloat16*>(base + c.tokens);
  std::int32_t* cu_dev = reinterpret_cast<std::int32_t*>(base + c.cu);
  const std::int32_t cu[2] = {0, static_cast<std::int32_t>(total)};
  if (const int rc = write_words(op, cu_dev, cu, 2, stream)) return rc;
  if (const int rc = write_words(op, time, f.time_vector, static_cast<std::size_t>(D), stream)) return rc;
  if (const int rc = b2_linear_fp32_row(m.block_mod_w, time, m.block_mod_bias, mod, static_cast<int>(6 * D), static_cast<int>(D), stream)) return rc;
  std::int64_t at = 0;
  for (int i = 0; i < f.num_refs; ++i) {
    const std::int64_t hw = static_cast<std::int64_t>(f.heights[i]) * f.widths[i];
    if (const int rc = b2_moss_rope_table_reference(rope + at * 128, 128, f.heights[i], f.widths[i], i, stream)) return rc;
    if (const int rc = embed_video(m, f.latents[i], nullptr, hw, tokens, x + at * D, base + c.lt, stream)) return rc;
    at += hw;
  }
  run.cu_seqlens = cu_dev;
  for (int bi = 0; bi < m.num_blocks; ++bi) {
    b2_block_run tap = run;
    tap.kv_tap = static_cast<__nv_bfloat16*>(f.kv_out) + static_cast<std::size_t>(bi) * static_cast<std::size_t>(total) * 2 * static_cast<std::size_t>(D);
    b2_block_buffers bb{};
    bb.struct_size = sizeof bb;
    bb.x = x, bb.mod = mod, bb.rope = rope, bb.workspace = base + c.block, bb.workspace_bytes = c.total - c.block;
    if (const int rc = b2_run_block_quant(&m.blocks[bi], &bb, &tap, stream)) return rc;
  }
  return B2_OK;
}
}  // namespace

size_t b2_dit_prefill_workspace_bytes(const b2_dit_model* model, const b2_prefill* prefill) {
  std::int64_t total = 0;
  PrefillCarve c{};
  b2_block_run run{};
  if (plan_prefill("dit_prefill_workspace_bytes", model, prefill, &total, &c, &run) != B2_OK) return 0;
  return c.total;
}

int b2_dit_prefill_references(const b2_dit_model* model, const b2_prefill* prefill, void* stream) {
  try {
    return prefill_impl(model, prefill, stream);
  } catch (const std::exception& e) {  // nothing may cross the C boundary
    return fail_status(B2_ERR_INTERNAL, "dit_prefill_references", e.what());
  }
}

}  // extern "C"
