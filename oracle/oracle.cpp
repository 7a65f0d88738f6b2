// CPU oracle for the quantized MOSS-Image DiT block path. TEST INFRASTRUCTURE ONLY: this file restates, in plain
// scalar C++, the arithmetic that the reference engine's CUDA kernels perform, so that the GPU library can be checked
// against it. Nothing on the product path may call into it. Build with -O2 -ffp-contract=off -fno-fast-math: the
// reference's numerics are single-rounded fp32 operations in a fixed order, and a contracted multiply-add would change
// bits.
//
// Parity status: pinned. The functions below reproduce the reference's own golden vectors bit for bit where the
// arithmetic is ordered fp32 / integer work (rotation + quantisation, GEMM accumulators and epilogues, grouped 4-bit
// decode, weight quantiser), and within the reference's stated tolerances where transcendental approximations of the
// GPU differ from libm (attention). tests/test_oracle_golden.py holds those checks.
//
// Every function cites the reference file it follows (paths inside the reference project).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

using i64 = std::int64_t;
using u16 = std::uint16_t;
using u8 = std::uint8_t;
using i8 = std::int8_t;

inline float bits_f(std::uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline std::uint32_t f_bits(float f) {
  std::uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float bf2f(u16 v) { return bits_f(static_cast<std::uint32_t>(v) << 16); }
// fp32 -> bf16 bits, round to nearest even; NaN stays NaN (quiet), matching cvt.rn.bf16.f32.
inline u16 f2bf(float v) {
  const std::uint32_t u = f_bits(v);
  if (std::isnan(v)) return 0x7FFF;
  return static_cast<u16>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
inline float rbf(float v) { return bf2f(f2bf(v)); }

// Run fn(begin, end) over [0, n) on `threads` host threads (1 = inline).
void parallel_for(i64 n, int threads, const std::function<void(i64, i64)>& fn) {
  if (n <= 0) return;
  if (threads <= 1 || n == 1) {
    fn(0, n);
    return;
  }
  const i64 t = std::min<i64>(threads, n), chunk = (n + t - 1) / t;
  std::vector<std::thread> pool;
  for (i64 i = 0; i < t; ++i) {
    const i64 b = i * chunk, e = std::min(n, b + chunk);
    if (b < e) pool.emplace_back([=, &fn] { fn(b, e); });
  }
  for (auto& th : pool) th.join();
}

int g_threads = 1;

// ---------------------------------------------------------------------------------------------------------------
// Rotation: x · H256 per 256-column group, four radix-4 stages over the base-4 digits of the in-group index (strides
// 1, 4, 16, 64). Stage output for digit d is 0.5 * (((m0' + m1') + m2') + m3') with operand 3 - d negated.
// Follows src/kernels/quant/rotate_quantize.cu:45-77 (h4 / hadamard256) and the numerics note in
// src/kernels/quant/quant.h:4-23.
void hadamard256(float* v) {
  float y[256];
  for (int st = 1; st <= 64; st *= 4) {
    for (int e = 0; e < 256; ++e) {
      const int d = (e / st) & 3, base = e - d * st;
      float m[4] = {v[base], v[base + st], v[base + 2 * st], v[base + 3 * st]};
      m[3 - d] = -m[3 - d];
      y[e] = 0.5f * (((m[0] + m[1]) + m[2]) + m[3]);
    }
    std::memcpy(v, y, sizeof(y));
  }
}

constexpr float kBf16Max = 3.38953139e38f;

// fmaxf / fminf semantics of the GPU: a NaN operand is dropped.
inline float fmax_nan(float a, float b) { return std::fmax(a, b); }
inline float fmin_nan(float a, float b) { return std::fmin(a, b); }

// Per-row INT8 quantisation of a rotated bf16 row. src/kernels/quant/rotate_quantize.cu:186-214.
void quantize_row_int8(const float* rot, int k, i8* q, float* scale) {
  float amax = 0.0f;
  for (int c = 0; c < k; ++c) amax = fmax_nan(amax, std::fabs(rot[c]));
  const float s = fmax_nan(fmin_nan(amax, kBf16Max) * (1.0f / 127.0f), 1e-30f);
  *scale = s;
  const float s_bf = rbf(s);
  for (int c = 0; c < k; ++c) {
    const float qv = std::nearbyint(rbf(rot[c] / s_bf));
    q[c] = static_cast<i8>(fmin_nan(127.0f, fmax_nan(-128.0f, qv)));
  }
}

// Per-row INT4 quantisation (W4A4 activations). src/kernels/quant4/convrot_quantize.cu:217-246.
void quantize_row_int4(const float* rot, int k, u8* q, float* scale) {
  float amax = 0.0f;
  for (int c = 0; c < k; ++c) amax = fmax_nan(amax, std::fabs(rot[c]));
  const float amax_bf = rbf(fmax_nan(fmin_nan(amax, kBf16Max), 1e-10f));
  const float s_bf = rbf(amax_bf * (1.0f / 7.0f));
  *scale = s_bf;
  for (int c = 0; c < k; c += 2) {
    int nib[2];
    for (int j = 0; j < 2; ++j) {
      const float qv = std::nearbyint(rbf(rot[c + j] / s_bf));
      nib[j] = static_cast<int>(fmin_nan(7.0f, fmax_nan(-7.0f, qv)));
    }
    q[c / 2] = static_cast<u8>((nib[0] & 0xF) | ((nib[1] & 0xF) << 4));
  }
}

// torch's launch shape for a last-dim fp32 mean over `rows` rows of length d: threads per row.
// src/kernels/basic/norm.cu:30-45, src/kernels/quant/norm_prologue.cuh:66-81. Returns 0 when torch would split a row
// across warps (the reference refuses that shape).
int torch_reduce_threads(i64 rows, i64 d) {
  const auto last_pow2 = [](i64 n) {
    i64 p = 1;
    while (p * 2 <= n) p *= 2;
    return p;
  };
  const i64 kMax = 512;
  const i64 dim0 = d / 4 < kMax ? last_pow2(d / 4) : kMax;
  const i64 dim1 = rows < kMax ? last_pow2(rows) : kMax;
  i64 bw = std::min<i64>(dim0, 32);
  const i64 bh = std::min(dim1, kMax / bw);
  bw = std::min(dim0, kMax / bh);
  if ((d + bw - 1) / bw >= std::min<i64>(bh * 16, 256)) return 0;
  return static_cast<int>(bw);
}

// Sum of squares of one row in torch's reduce order with bw cooperating threads: per-thread four accumulators over
// 4-element vectors strided by bw, combined ((a0+a1)+a2)+a3, a halving tree down to 32 values, then a shuffle-down
// tree. src/kernels/basic/norm.cu:83-113, src/kernels/quant/norm_prologue.cuh:23-54.
float torch_sum_squares(const u16* x, int k, int bw) {
  std::vector<float> v(static_cast<std::size_t>(std::max(bw, 32)), 0.0f);
  for (int t = 0; t < bw; ++t) {
    float acc[4] = {0, 0, 0, 0};
    for (int idx = t; idx * 4 + 3 < k; idx += bw) {
      for (int i = 0; i < 4; ++i) {
        const float e = bf2f(x[idx * 4 + i]);
        acc[i] = acc[i] + e * e;
      }
    }
    v[static_cast<std::size_t>(t)] = ((acc[0] + acc[1]) + acc[2]) + acc[3];
  }
  for (int off = bw / 2; off >= 32; off >>= 1) {
    for (int t = 0; t < off; ++t) v[static_cast<std::size_t>(t)] = v[static_cast<std::size_t>(t)] + v[static_cast<std::size_t>(t + off)];
  }
  for (int off = 16; off > 0; off >>= 1) {
    for (int t = 0; t < off; ++t) v[static_cast<std::size_t>(t)] = v[static_cast<std::size_t>(t)] + v[static_cast<std::size_t>(t + off)];
  }
  return v[0];
}

// 1 / sqrt on the CPU. The GPU's rsqrtf is an approximation with <= 2 ulp error; results that depend on it are gated
// with a tolerance in the tests, not bit for bit.
inline float inv_sqrt(float v) { return 1.0f / std::sqrt(v); }

// One element of the MOSS RMSNorm + adaLN modulate: bf16(bf16(bf16(bf16(x*r)*w) * bf16(1+scale)) + shift).
// src/kernels/basic/norm.cu:117-124, src/kernels/quant/norm_prologue.cuh:57-61.
inline float moss_modulate(float x, float r, float w, float sc, float sh) {
  const float y = rbf(x * r) * w;
  const float one_plus = rbf(1.0f + sc);
  return rbf(rbf(rbf(y) * one_plus) + sh);
}

// MOSS SiTU factors on bf16 inputs. src/kernels/fused/fused_gemm_impl.cuh:58-67 (op order),
// src/kernels/basic/detail.h:99-100 (sigmoid = 1 / (1 + exp(-x)) with IEEE division).
inline float sigmoid_f32(float x) { return 1.0f / (1.0f + std::exp(-x)); }
inline float situ_gate_factor(float g) { return rbf(rbf(4.0f * rbf(std::tanh(rbf(g * 0.25f)))) * rbf(sigmoid_f32(g))); }
inline float situ_hidden_factor(float h) { return rbf(25.0f * rbf(std::tanh(rbf(h * (1.0f / 25.0f))))); }

// Dequantisation of one accumulator: ((float)acc * xs) * ws + bias, one rounding per op.
// src/kernels/quant/int8_gemm_impl.cuh:73-76.
inline float dequant(std::int32_t acc, float xs, float ws, float bias) {
  return (static_cast<float>(acc) * xs) * ws + bias;
}

// Weight row that GEMM column n of the SiTU-GLU epilogue reads. src/kernels/quant/int8_gemm_impl.cuh:108-112.
inline i64 up_gate_row(i64 n, i64 half) { return ((n / 4) % 2) * half + (n / 8) * 4 + n % 4; }

inline std::int32_t dot_i8(const i8* a, const i8* b, i64 k) {
  std::int32_t acc = 0;
  for (i64 i = 0; i < k; ++i) acc += static_cast<std::int32_t>(a[i]) * static_cast<std::int32_t>(b[i]);
  return acc;
}

// e4m3 (fn) helpers. Decode: src/weights/quant/quant_codec.cpp:133-141. Encode: cvt.rn.satfinite.e4m3x2.f32
// (round to nearest even, saturate to +-448, NaN -> 0x7F).
float e4m3_to_float(u8 v) {
  const int e = (v >> 3) & 0xF, m = v & 7;
  float mag;
  if (e == 0xF && m == 7) mag = std::nanf("");
  else if (e == 0) mag = std::ldexp(static_cast<float>(m), -9);
  else mag = std::ldexp(1.0f + static_cast<float>(m) / 8.0f, e - 7);
  return (v & 0x80) ? -mag : mag;
}
u8 float_to_e4m3(float x) {
  const u8 sign = std::signbit(x) ? 0x80 : 0;
  if (std::isnan(x)) return static_cast<u8>(sign | 0x7F);
  const float a = std::fabs(x);
  if (a >= 448.0f) return static_cast<u8>(sign | 0x7E);
  if (a < std::ldexp(1.0f, -6)) {
    const int m = static_cast<int>(std::nearbyint(a * 512.0f));  // subnormal step 2^-9; m == 8 is the first normal
    return static_cast<u8>(sign | m);
  }
  int e;
  std::frexp(a, &e);  // a = f * 2^e, f in [0.5, 1)
  e -= 1;             // a = (1 + frac) * 2^e
  int m = static_cast<int>(std::nearbyint((std::ldexp(a, -e) - 1.0f) * 8.0f));
  if (m == 8) {
    m = 0;
    e += 1;
  }
  const int code = ((e + 7) << 3) | m;
  return static_cast<u8>(sign | std::min(code, 0x7E));
}

// fp16 bits -> float (for the group scales of the fp16-scale W4A8 layout).
float half_to_float(u16 h) {
  const int s = h >> 15, e = (h >> 10) & 0x1F, m = h & 0x3FF;
  float v;
  if (e == 0) v = std::ldexp(static_cast<float>(m), -24);
  else if (e == 31) v = m ? std::nanf("") : INFINITY;
  else v = std::ldexp(1.0f + static_cast<float>(m) / 1024.0f, e - 15);
  return s ? -v : v;
}

// cvt.rni.sat.s8.f32: round to nearest even, saturate; NaN -> 0.
inline i8 float_to_int8_rn(float v) {
  if (std::isnan(v)) return 0;
  const float r = std::nearbyint(v);
  return static_cast<i8>(std::min(127.0f, std::max(-128.0f, r)));
}

// int32 -> fp32 with round toward zero (__int2float_rz).
inline float int2float_rz(std::int32_t v) {
  const float f = static_cast<float>(v);  // nearest
  if (static_cast<double>(f) == static_cast<double>(v)) return f;
  const bool away = std::fabs(static_cast<double>(f)) > std::fabs(static_cast<double>(v));
  return away ? std::nextafter(f, 0.0f) : f;
}

}  // namespace

extern "C" {

void orc_set_threads(int threads) { g_threads = threads < 1 ? 1 : threads; }

// quant::rotate_quantize, src/kernels/quant/quant.h:48 / rotate_quantize.cu:126.
void orc_rotate_quantize(const u16* x, i64 ldx, i8* q, i64 ldq, float* scale, i64 m, int k) {
  parallel_for(m, g_threads, [&](i64 b, i64 e) {
    std::vector<float> row(static_cast<std::size_t>(k));
    for (i64 r = b; r < e; ++r) {
      for (int c = 0; c < k; ++c) row[static_cast<std::size_t>(c)] = bf2f(x[r * ldx + c]);
      for (int g = 0; g < k; g += 256) hadamard256(row.data() + g);
      for (int c = 0; c < k; ++c) row[static_cast<std::size_t>(c)] = rbf(row[static_cast<std::size_t>(c)]);
      quantize_row_int8(row.data(), k, q + r * ldq, scale + r);
    }
  });
}

// kernels::rms_norm_modulate_moss, src/kernels/basic/norm.cu:67-128: the bf16 tensor before rotation.
// Returns 0, or -1 when torch's reduce would split a row across warps.
int orc_rms_norm_modulate(const u16* x, i64 ldx, const u16* w, const u16* mod_scale, const u16* mod_shift, u16* y,
                          i64 ldy, i64 m, int k) {
  const int bw = torch_reduce_threads(m, k);
  if (bw == 0) return -1;
  const float factor = static_cast<float>(m) / static_cast<float>(m * k);
  parallel_for(m, g_threads, [&](i64 b, i64 e) {
    for (i64 r = b; r < e; ++r) {
      const float ss = torch_sum_squares(x + r * ldx, k, bw);
      const float inv = inv_sqrt(ss * factor + 1e-6f);
      for (int c = 0; c < k; ++c) {
        y[r * ldy + c] = f2bf(moss_modulate(bf2f(x[r * ldx + c]), inv, bf2f(w[c]), bf2f(mod_scale[c]), bf2f(mod_shift[c])));
      }
    }
  });
  return 0;
}

// quant::rms_norm_modulate_rotate_quantize, src/kernels/quant/quant.h:62. y (optional) receives the bf16 norm output.
int orc_rms_norm_modulate_rotate_quantize(const u16* x, i64 ldx, const u16* w, const u16* mod_scale,
                                          const u16* mod_shift, i8* q, i64 ldq, float* scale, i64 m, int k, u16* y,
                                          i64 ldy) {
  std::vector<u16> tmp;
  if (y == nullptr) {
    tmp.resize(static_cast<std::size_t>(m) * k);
    y = tmp.data();
    ldy = k;
  }
  if (orc_rms_norm_modulate(x, ldx, w, mod_scale, mod_shift, y, ldy, m, k) != 0) return -1;
  orc_rotate_quantize(y, ldy, q, ldq, scale, m, k);
  return 0;
}

// quant4::convrot_quantize_int4, src/kernels/quant4/quant4.h:45 / convrot_quantize.cu:152.
void orc_convrot_quantize_int4(const u16* x, i64 ldx, u8* q, i64 ldq, float* scale, i64 m, int k) {
  parallel_for(m, g_threads, [&](i64 b, i64 e) {
    std::vector<float> row(static_cast<std::size_t>(k));
    for (i64 r = b; r < e; ++r) {
      for (int c = 0; c < k; ++c) row[static_cast<std::size_t>(c)] = bf2f(x[r * ldx + c]);
      for (int g = 0; g < k; g += 256) hadamard256(row.data() + g);
      for (int c = 0; c < k; ++c) row[static_cast<std::size_t>(c)] = rbf(row[static_cast<std::size_t>(c)]);
      quantize_row_int4(row.data(), k, q + r * ldq, scale + r);
    }
  });
}

// quant4::rms_norm_modulate_convrot_quantize_int4, src/kernels/quant4/quant4.h:51.
int orc_rms_norm_modulate_convrot_quantize_int4(const u16* x, i64 ldx, const u16* w, const u16* mod_scale,
                                                const u16* mod_shift, u8* q, i64 ldq, float* scale, i64 m, int k) {
  std::vector<u16> y(static_cast<std::size_t>(m) * k);
  if (orc_rms_norm_modulate(x, ldx, w, mod_scale, mod_shift, y.data(), k, m, k) != 0) return -1;
  orc_convrot_quantize_int4(y.data(), k, q, ldq, scale, m, k);
  return 0;
}

// moss_dit::unpack_int4 (src/models/moss_dit/dit_kernels.cu:109) and quant::decode_int4_rows
// (src/weights/quant/quant_codec.cpp:210-217): signed nibbles, even column = low nibble.
void orc_unpack_int4(const u8* packed, i64 ldp, i8* out, i64 ldo, i64 rows, i64 k) {
  for (i64 r = 0; r < rows; ++r) {
    for (i64 c = 0; c < k; ++c) {
      const int nib = (packed[r * ldp + c / 2] >> ((c & 1) * 4)) & 0xF;
      out[r * ldo + c] = static_cast<i8>(nib >= 8 ? nib - 16 : nib);
    }
  }
}

// Grouped 4-bit codes -> INT8 grid: level = codebook[code] or code - 8; w8 = clamp(rint(level * s_rel), -127, 127).
// src/weights/quant/quant_codec.cpp:184-208, src/kernels/quant/w4a8_decode.cu:28-64. scale_kind 0: e4m3 bytes
// (the reference's file format); 1: fp16 bits (every e4m3 value is exact in fp16, so kind 0 is a subset).
// Returns 0, or -1 when a scale is NaN or negative (the reference rejects the file).
int orc_decode_grouped_int8(const u8* packed, const void* s_rel, int scale_kind, const float* codebook, i64 rows, i64 k,
                            int group, i8* out) {
  const i64 groups = k / group;
  for (i64 r = 0; r < rows; ++r) {
    const u8* p = packed + r * (k / 2);
    for (i64 gi = 0; gi < groups; ++gi) {
      const float s = scale_kind == 0 ? e4m3_to_float(static_cast<const u8*>(s_rel)[r * groups + gi])
                                      : half_to_float(static_cast<const u16*>(s_rel)[r * groups + gi]);
      if (std::isnan(s) || s < 0.0f) return -1;
      for (i64 c = gi * group; c < (gi + 1) * group; ++c) {
        const unsigned code = (p[c / 2] >> ((c & 1) * 4)) & 0xFu;
        const float level = codebook != nullptr ? codebook[code] : static_cast<float>(code) - 8.0f;
        const float v = std::nearbyint(level * s);
        out[r * k + c] = static_cast<i8>(std::min(127.0f, std::max(-127.0f, v)));
      }
    }
  }
  return 0;
}

// The same decode under the GPU kernel's rule for untrusted scales (src/kernels/quant/w4a8_decode.cu:57-62): a group
// whose scale is NaN or negative decodes to zeros and ORs 1 into *invalid; every other group decodes as above.
void orc_decode_grouped_int8_device_rule(const u8* packed, const void* s_rel, int scale_kind, const float* codebook,
                                         i64 rows, i64 k, int group, i8* out, unsigned* invalid) {
  const i64 groups = k / group;
  for (i64 r = 0; r < rows; ++r) {
    const u8* p = packed + r * (k / 2);
    for (i64 gi = 0; gi < groups; ++gi) {
      const float s = scale_kind == 0 ? e4m3_to_float(static_cast<const u8*>(s_rel)[r * groups + gi])
                                      : half_to_float(static_cast<const u16*>(s_rel)[r * groups + gi]);
      const bool ok = !(std::isnan(s) || s < 0.0f);
      if (!ok) *invalid |= 1u;
      for (i64 c = gi * group; c < (gi + 1) * group; ++c) {
        const unsigned code = (p[c / 2] >> ((c & 1) * 4)) & 0xFu;
        const float level = codebook != nullptr ? codebook[code] : static_cast<float>(code) - 8.0f;
        const float v = std::nearbyint(level * s);
        out[r * k + c] = ok ? static_cast<i8>(std::min(127.0f, std::max(-127.0f, v))) : i8{0};
      }
    }
  }
}

// Offline ConvRot weight quantiser (what turns bf16 weights into the GEMM's INT8 operand):
// W_rot = W · H_g per group with the products summed in column order, s = max(absmax / 127, 1e-30), q = rne(W_rot / s).
// src/weights/quant/quant_codec.cpp:50-96,148-159.
void orc_quantize_convrot_rows_bf16(const u16* w, i64 rows, i64 k, int g, i8* q, float* scale) {
  int logg = 0;
  while ((1 << (2 * logg)) < g) ++logg;
  const float inv = 1.0f / static_cast<float>(1 << logg);
  std::vector<float> h(static_cast<std::size_t>(g) * g);
  for (int i = 0; i < g; ++i) {
    for (int j = 0; j < g; ++j) {
      int neg = 0;
      for (int n = 0, a = i, b = j; n < logg; ++n, a >>= 2, b >>= 2) neg ^= ((a & 3) + (b & 3) == 3) ? 1 : 0;
      h[static_cast<std::size_t>(i) * g + j] = neg ? -inv : inv;
    }
  }
  parallel_for(rows, g_threads, [&](i64 b, i64 e) {
    std::vector<float> row(static_cast<std::size_t>(k)), rot(static_cast<std::size_t>(k));
    for (i64 r = b; r < e; ++r) {
      for (i64 c = 0; c < k; ++c) row[static_cast<std::size_t>(c)] = bf2f(w[r * k + c]);
      for (i64 c0 = 0; c0 < k; c0 += g) {
        for (int j = 0; j < g; ++j) {
          float acc = 0.0f;
          for (int i = 0; i < g; ++i) acc += row[static_cast<std::size_t>(c0 + i)] * h[static_cast<std::size_t>(i) * g + j];
          rot[static_cast<std::size_t>(c0 + j)] = acc;
        }
      }
      float amax = 0.0f;
      for (i64 c = 0; c < k; ++c) amax = std::max(amax, std::fabs(rot[static_cast<std::size_t>(c)]));
      const float s = std::max(amax * (1.0f / 127.0f), 1e-30f);
      for (i64 c = 0; c < k; ++c) {
        const float v = std::nearbyint(rot[static_cast<std::size_t>(c)] / s);
        q[r * k + c] = static_cast<i8>(std::min(127.0f, std::max(-128.0f, v)));
      }
      scale[r] = s;
    }
  });
}

// Exact int32 accumulators of the INT8 GEMM: acc[r, c] = sum_k xq[r, k] * wq[c, k].
// tests/unit/test_quant_kernels.cu:208-231 (scalar oracle kernel).
void orc_int8_gemm_acc(const i8* xq, i64 ldx, const i8* wq, i64 m, i64 n, i64 k, std::int32_t* acc, i64 ldacc) {
  parallel_for(m, g_threads, [&](i64 b, i64 e) {
    for (i64 r = b; r < e; ++r) {
      for (i64 c = 0; c < n; ++c) acc[r * ldacc + c] = dot_i8(xq + r * ldx, wq + c * k, k);
    }
  });
}

// quant::int8_gemm: out = bf16(((float)acc * xs[r]) * ws[c] + bias[c]). src/kernels/quant/quant.h:92,
// int8_gemm_impl.cuh:73-93.
void orc_int8_gemm(const i8* xq, i64 ldx, const float* xs, const i8* wq, const float* ws, i64 m, i64 n, i64 k,
                   const u16* bias, u16* out, i64 ldo) {
  parallel_for(m, g_threads, [&](i64 b, i64 e) {
    for (i64 r = b; r < e; ++r) {
      for (i64 c = 0; c < n; ++c) {
        const std::int32_t acc = dot_i8(xq + r * ldx, wq + c * k, k);
        out[r * ldo + c] = f2bf(dequant(acc, xs[r], ws[c], bias ? bf2f(bias[c]) : 0.0f));
      }
    }
  });
}

// quant::int8_gemm_gated_residual: res = bf16(res + bf16(bf16(y) * gate[c])) in place.
// src/kernels/quant/quant.h:98, int8_gemm_impl.cuh:96-106.
void orc_int8_gemm_gated_residual(const i8* xq, i64 ldx, const float* xs, const i8* wq, const float* ws, i64 m, i64 n,
                                  i64 k, const u16* bias, const u16* gate, u16* res, i64 ldr) {
  parallel_for(m, g_threads, [&](i64 b, i64 e) {
    for (i64 r = b; r < e; ++r) {
      for (i64 c = 0; c < n; ++c) {
        const std::int32_t acc = dot_i8(xq + r * ldx, wq + c * k, k);
        const float y = rbf(dequant(acc, xs[r], ws[c], bias ? bf2f(bias[c]) : 0.0f));
        res[r * ldr + c] = f2bf(bf2f(res[r * ldr + c]) + rbf(y * bf2f(gate[c])));
      }
    }
  });
}

// quant::int8_gemm_situ_glu: weight [2F, k] stored [hidden | gate]; out[r, j] = bf16(gateF(g) * hiddenF(h)) with h, g the
// bf16-rounded dequantised halves. src/kernels/quant/quant.h:110, int8_gemm_impl.cuh:134-188. (The column permutation
// the reference's GEMM applies is an implementation detail: output column j pairs weight rows j and F + j.)
void orc_int8_gemm_situ_glu(const i8* xq, i64 ldx, const float* xs, const i8* wq, const float* ws, i64 m, i64 n2, i64 k,
                            u16* out, i64 ldo) {
  const i64 f = n2 / 2;
  parallel_for(m, g_threads, [&](i64 b, i64 e) {
    for (i64 r = b; r < e; ++r) {
      for (i64 j = 0; j < f; ++j) {
        const float h = rbf(dequant(dot_i8(xq + r * ldx, wq + j * k, k), xs[r], ws[j], 0.0f));
        const float g = rbf(dequant(dot_i8(xq + r * ldx, wq + (f + j) * k, k), xs[r], ws[f + j], 0.0f));
        out[r * ldo + j] = f2bf(situ_gate_factor(g) * situ_hidden_factor(h));
      }
    }
  });
}

// The permuted weight row of GEMM column n (exposed so tests can check the kernel's B-row mapping).
i64 orc_up_gate_row(i64 n, i64 half) { return up_gate_row(n, half); }

// kernels::situ_glu on a stored [m, 2F] bf16 tensor (src/kernels/basic/elementwise.cu:38-43): the definition the
// epilogue follows. Used to pin the oracle on tests/data/basic/situ_*.npy.
void orc_situ_glu(const u16* up_gate, i64 ld, u16* out, i64 ldo, i64 m, i64 f) {
  for (i64 r = 0; r < m; ++r) {
    for (i64 j = 0; j < f; ++j) {
      out[r * ldo + j] = f2bf(situ_gate_factor(bf2f(up_gate[r * ld + f + j])) * situ_hidden_factor(bf2f(up_gate[r * ld + j])));
    }
  }
}

// The two 65536-entry bf16 factor tables. src/kernels/quant/int8_gemm_situ.cu:22-27.
void orc_situ_tables(u16* gate, u16* hidden) {
  for (std::uint32_t i = 0; i < 65536; ++i) {
    const float x = bits_f(i << 16);
    gate[i] = f2bf(situ_gate_factor(x));
    hidden[i] = f2bf(situ_hidden_factor(x));
  }
}

// kernels::fused::qk_norm_rope_moss: per (token, q or k head) RMS norm over 128 dims in torch's reduce order, weight,
// RoPE on pairs (d, d + 64) with table rows [sin(64) | cos(64)]. src/kernels/fused/qk_norm_rope.cu:43-89.
void orc_qk_norm_rope(u16* qkv, i64 ld, i64 tokens, int heads, const u16* q_norm, const u16* k_norm, const u16* table,
                      i64 table_ld) {
  const i64 rows = tokens * heads;
  const float factor = static_cast<float>(rows) / static_cast<float>(rows * 128);
  parallel_for(tokens, g_threads, [&](i64 b, i64 e) {
    for (i64 t = b; t < e; ++t) {
      for (int head = 0; head < 2 * heads; ++head) {
        u16* row = qkv + t * ld + static_cast<i64>(head) * 128;
        const u16* w = head < heads ? q_norm : k_norm;
        const float ss = torch_sum_squares(row, 128, 32);
        const float r = inv_sqrt(ss * factor + 1e-6f);
        float y[128];
        for (int d = 0; d < 128; ++d) y[d] = rbf(rbf(bf2f(row[d]) * r) * bf2f(w[d]));
        const u16* tab = table + t * table_ld;
        for (int d = 0; d < 64; ++d) {
          const float si = bf2f(tab[d]), co = bf2f(tab[64 + d]);
          const float lo = y[d], hi = y[d + 64];
          row[d] = f2bf(rbf(lo * co) + rbf(-hi * si));
          row[d + 64] = f2bf(rbf(hi * co) + rbf(lo * si));
        }
      }
    }
  });
}

// kernels::moss_rope_table: image tokens first (coords r = 0, f = text_length, centred h, w), then text tokens
// (f = index); per axis 16 bands; row = [sin(64) | cos(64)]. src/kernels/basic/rope.h:18-37, rope.cu:30-51.
// bands: the 16 fp32 frequencies 1 / 1e4^(i/16).
void orc_moss_rope_table(u16* out, i64 ld, int height, int width, int text_length, const float* bands) {
  const i64 hw = static_cast<i64>(height) * width, n = hw + text_length;
  const float h_mid = static_cast<float>((height - 1) / 2.0), w_mid = static_cast<float>((width - 1) / 2.0);
  for (i64 r = 0; r < n; ++r) {
    for (int c = 0; c < 128; ++c) {
      const int p = c & 63, axis = p >> 4, band = p & 15;
      float coord = 0.0f;
      if (r < hw) {
        if (axis == 1) coord = static_cast<float>(text_length);
        if (axis == 2) coord = static_cast<float>(r / width) - h_mid;
        if (axis == 3) coord = static_cast<float>(r % width) - w_mid;
      } else if (axis == 1) {
        coord = static_cast<float>(r - hw);
      }
      const float phase = coord * bands[band];
      out[r * ld + c] = f2bf(c < 64 ? std::sin(phase) : std::cos(phase));
    }
  }
}

// kernels::moss_rope_table_reference (src/kernels/basic/rope.cu:53-71): reference image `index` of the edit layout at
// coordinates (index + 1, 0, centred row, centred column); no text rows.
void orc_moss_rope_table_reference(u16* out, i64 ld, int height, int width, int index, const float* bands) {
  const i64 hw = static_cast<i64>(height) * width;
  const float h_mid = static_cast<float>((height - 1) / 2.0), w_mid = static_cast<float>((width - 1) / 2.0);
  for (i64 r = 0; r < hw; ++r) {
    for (int c = 0; c < 128; ++c) {
      const int p = c & 63, axis = p >> 4, band = p & 15;
      float coord = 0.0f;
      if (axis == 0) coord = static_cast<float>(index + 1);
      if (axis == 2) coord = static_cast<float>(r / width) - h_mid;
      if (axis == 3) coord = static_cast<float>(r % width) - w_mid;
      const float phase = coord * bands[band];
      out[r * ld + c] = f2bf(c < 64 ? std::sin(phase) : std::cos(phase));
    }
  }
}

// Attention pre-pass (unfused form; with QK-norm + RoPE the reference's fused pass gives the same bits as
// orc_qk_norm_rope followed by this). src/kernels/attention_q8/q8_preprocess.cu:67-385.
//   k_mean[b,h,c]   = bf16(sum / len), the sum taken as: 16 row-threads each adding tokens row, row+16, ... of a 512-key
//                     chunk, then the 16 partials in order, then the chunks in order.
//   q_i8 / q_scale  per (32 tokens, head): amax floored at 1e-7, scale = amax / 127, q = rni(x * (127 / amax)).
//   k_i8 / k_scale  per (64 keys, head) after subtracting k_mean.
//   v8 / v_scale    per channel over the sequence: amax; v_scale = amax / v_range, v_recp = v_range / amax (amax 0 -> 1, 1);
//                   v8 = e4m3(v * v_recp).
// Layouts here are the natural ones: q_i8, k_i8, v8 [tokens, heads, 128]; q_scale [batch, heads, q_blocks];
// k_scale [batch, heads, k_blocks]; k_mean, v_scale [batch, heads, 128]. q_blocks = ceil(max_seqlen/128)*4,
// k_blocks = ceil(max_seqlen/64). q/k/v are bf16 views with a row stride (elements) and head stride 128.
void orc_attention_prepass(const u16* q, const u16* k, const u16* v, i64 row_stride, const std::int32_t* cu, int batch,
                           int heads, int max_seqlen, float v_range, i8* q_i8, i8* k_i8, u8* v8, float* q_scale,
                           float* k_scale, float* k_mean, float* v_scale) {
  const int q_blocks = (max_seqlen + 127) / 128 * 4, k_blocks = (max_seqlen + 63) / 64;
  const i64 items = static_cast<i64>(batch) * heads;
  parallel_for(items, g_threads, [&](i64 ib, i64 ie) {
    for (i64 item = ib; item < ie; ++item) {
      const int b = static_cast<int>(item / heads), h = static_cast<int>(item % heads);
      const i64 start = cu[b];
      const int len = cu[b + 1] - cu[b];
      const auto at = [&](const u16* p, i64 t, int c) { return bf2f(p[(start + t) * row_stride + static_cast<i64>(h) * 128 + c]); };
      float mean[128], vrecp[128];
      for (int c = 0; c < 128; ++c) {
        float total = 0.0f, amax = 0.0f;
        for (int ch = 0; ch * 512 < std::max(len, 1); ++ch) {
          const int t_end = std::min(len, (ch + 1) * 512);
          float part[16];
          for (int row = 0; row < 16; ++row) {
            float s = 0.0f;
            for (int t = ch * 512 + row; t < t_end; t += 16) s += at(k, t, c);
            part[row] = s;
          }
          float s = 0.0f;
          for (int row = 0; row < 16; ++row) s += part[row];
          total += s;
        }
        for (int t = 0; t < len; ++t) amax = fmax_nan(amax, std::fabs(at(v, t, c)));
        mean[c] = len > 0 ? rbf(total / static_cast<float>(len)) : 0.0f;
        k_mean[item * 128 + c] = mean[c];
        v_scale[item * 128 + c] = amax > 0.0f ? amax / v_range : 1.0f;
        vrecp[c] = amax > 0.0f ? v_range / amax : 1.0f;
      }
      for (int bx = 0; bx < q_blocks; ++bx) {
        float amax = 0.0000001f;
        for (int t = bx * 32; t < std::min(len, bx * 32 + 32); ++t) {
          for (int c = 0; c < 128; ++c) amax = fmax_nan(amax, std::fabs(at(q, t, c)));
        }
        q_scale[item * q_blocks + bx] = amax / 127.0f;
        const float mulq = 127.0f / amax;
        for (int t = bx * 32; t < std::min(len, bx * 32 + 32); ++t) {
          for (int c = 0; c < 128; ++c) q_i8[((start + t) * heads + h) * 128 + c] = float_to_int8_rn(at(q, t, c) * mulq);
        }
      }
      for (int bx = 0; bx < k_blocks; ++bx) {
        float amax = 0.0000001f;
        for (int t = bx * 64; t < std::min(len, bx * 64 + 64); ++t) {
          for (int c = 0; c < 128; ++c) amax = fmax_nan(amax, std::fabs(at(k, t, c) - mean[c]));
        }
        k_scale[item * k_blocks + bx] = amax / 127.0f;
        const float mulk = 127.0f / amax;
        for (int t = bx * 64; t < std::min(len, bx * 64 + 64); ++t) {
          for (int c = 0; c < 128; ++c) {
            k_i8[((start + t) * heads + h) * 128 + c] = float_to_int8_rn((at(k, t, c) - mean[c]) * mulk);
          }
        }
      }
      for (int t = 0; t < len; ++t) {
        for (int c = 0; c < 128; ++c) v8[((start + t) * heads + h) * 128 + c] = float_to_e4m3(at(v, t, c) * vrecp[c]);
      }
    }
  });
}

// Exact int32 scores of one (sequence, head): S[i, j] = q_i8[i] · k_i8[j] (for the "QK^T accumulators bit-exact" check).
void orc_qk_scores(const i8* q_i8, const i8* k_i8, int heads, int head, i64 q0, int qn, i64 k0, int kn, std::int32_t* s) {
  for (int i = 0; i < qn; ++i) {
    for (int j = 0; j < kn; ++j) {
      s[static_cast<i64>(i) * kn + j] = dot_i8(q_i8 + ((q0 + i) * heads + head) * 128, k_i8 + ((k0 + j) * heads + head) * 128, 128);
    }
  }
}

// The attention kernel on pre-pass outputs, kInt8Fp8F32Acc semantics (e4m3 P and V, fp32 accumulation):
// per (query row, head, sequence), 64-key tiles: S int32 -> fp32 (round toward zero); c = (sm_scale * log2e) * (q_scale *
// k_scale[tile]); m_new = max(m, max(S) * c - off); O *= 2^(m_old - m_new); d likewise; P = 2^(S * c - m_new);
// d += sum P (fp32, unrounded P); P8 = e4m3(P); O += P8 · V8; out = O / d * v_scale[c] -> bf16.
// off = floor(log2(p_range) * 1000) / 1000. m starts at -5e6, d at 1.
// third_party/sageattention/csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:54-743, attn_utils.cuh:357-440,534-559,728-778;
// src/kernels/attention_q8/attention_q8.cu:277-279 (offset). exp2 / reciprocal are exact here, hardware approximations
// on the GPU: compare with a tolerance.
void orc_attention_q8_core(const i8* q_i8, const i8* k_i8, const u8* v8, const float* q_scale, const float* k_scale,
                           const float* v_scale, const std::int32_t* cu, int batch, int heads, int max_seqlen,
                           float sm_scale, float p_range, u16* out, i64 out_row_stride) {
  const int q_blocks = (max_seqlen + 127) / 128 * 4, k_blocks = (max_seqlen + 63) / 64;
  const float off = static_cast<float>(std::floor(std::log2(static_cast<double>(p_range)) * 1000.0) / 1000.0);
  const float scale2 = sm_scale * 1.44269504088896340736f;
  std::vector<float> v_lut(256);
  for (int i = 0; i < 256; ++i) v_lut[static_cast<std::size_t>(i)] = e4m3_to_float(static_cast<u8>(i));
  i64 total_rows = 0;
  std::vector<i64> row_b;
  for (int b = 0; b < batch; ++b) total_rows += cu[b + 1] - cu[b];
  const i64 items = total_rows * heads;
  parallel_for(items, g_threads, [&](i64 ib, i64 ie) {
    for (i64 item = ib; item < ie; ++item) {
      const i64 row = item / heads;
      const int h = static_cast<int>(item % heads);
      int b = 0;
      while (cu[b + 1] <= row) ++b;
      const i64 start = cu[b];
      const int len = cu[b + 1] - cu[b], ti = static_cast<int>(row - start);
      const float qs = q_scale[(static_cast<i64>(b) * heads + h) * q_blocks + ti / 32];
      const i8* qv = q_i8 + (row * heads + h) * 128;
      float m = -5000000.0f, d = 1.0f, o[128] = {};
      for (int t0 = 0; t0 < len; t0 += 64) {
        const int tn = std::min(64, len - t0);
        const float c = scale2 * (qs * k_scale[(static_cast<i64>(b) * heads + h) * k_blocks + t0 / 64]);
        float sf[64], mx = -5000000.0f;
        for (int j = 0; j < tn; ++j) {
          sf[j] = int2float_rz(dot_i8(qv, k_i8 + ((start + t0 + j) * heads + h) * 128, 128));
          mx = std::max(mx, sf[j]);
        }
        const float m_new = std::max(m, mx * c - off);
        const float resc = std::exp2(m - m_new);
        d *= resc;
        for (int e = 0; e < 128; ++e) o[e] *= resc;
        m = m_new;
        for (int j = 0; j < tn; ++j) {
          const float p = std::exp2(sf[j] * c - m);
          d += p;
          const float p8 = v_lut[float_to_e4m3(p)];
          const u8* vr = v8 + ((start + t0 + j) * heads + h) * 128;
          for (int e = 0; e < 128; ++e) o[e] += p8 * v_lut[vr[e]];
        }
      }
      const float rd = 1.0f / d;
      for (int e = 0; e < 128; ++e) {
        const float val = len > 0 ? o[e] * rd * v_scale[(static_cast<i64>(b) * heads + h) * 128 + e] : 0.0f;
        out[row * out_row_stride + static_cast<i64>(h) * 128 + e] = f2bf(val);
      }
    }
  });
}

// attention_q8 (self-attention, heads == kv_heads, cu_seqlens_q == cu_seqlens_k), optional fused QK-norm + RoPE:
// src/kernels/attention_q8/attention_q8.cu:201-371. qkv: bf16 [total, >= 3 * heads * 128] with q at column 0, k at
// heads*128, v at 2*heads*128 (k is rewritten normed + roped when norm_rope != 0, as the reference does; q is also
// rewritten here, which the reference leaves undefined). out: bf16 rows of out_row_stride.
void orc_attention_q8(u16* qkv, i64 ld, const std::int32_t* cu, int batch, int heads, int max_seqlen, float sm_scale,
                      float p_range, float v_range, int norm_rope, const u16* q_norm, const u16* k_norm,
                      const u16* table, i64 table_ld, u16* out, i64 out_row_stride) {
  const i64 total = cu[batch];
  if (norm_rope) orc_qk_norm_rope(qkv, ld, total, heads, q_norm, k_norm, table, table_ld);
  const int q_blocks = (max_seqlen + 127) / 128 * 4, k_blocks = (max_seqlen + 63) / 64;
  std::vector<i8> q_i8(static_cast<std::size_t>(total) * heads * 128), k_i8(q_i8.size());
  std::vector<u8> v8(q_i8.size());
  std::vector<float> q_scale(static_cast<std::size_t>(batch) * heads * q_blocks), k_scale(static_cast<std::size_t>(batch) * heads * k_blocks);
  std::vector<float> k_mean(static_cast<std::size_t>(batch) * heads * 128), v_scale(k_mean.size());
  orc_attention_prepass(qkv, qkv + static_cast<i64>(heads) * 128, qkv + static_cast<i64>(2 * heads) * 128, ld, cu, batch, heads,
                        max_seqlen, v_range, q_i8.data(), k_i8.data(), v8.data(), q_scale.data(), k_scale.data(),
                        k_mean.data(), v_scale.data());
  orc_attention_q8_core(q_i8.data(), k_i8.data(), v8.data(), q_scale.data(), k_scale.data(), v_scale.data(), cu, batch,
                        heads, max_seqlen, sm_scale, p_range, out, out_row_stride);
}

// Exact softmax attention in double precision on the same bf16 q, k, v (accuracy yardstick).
// tests/unit/test_attention_q8.cu:100-146.
void orc_attention_exact(const u16* q, const u16* k, const u16* v, i64 row_stride, const std::int32_t* cu, int batch,
                         int heads, float sm_scale, float* out) {
  const i64 total = cu[batch];
  parallel_for(total * heads, g_threads, [&](i64 ib, i64 ie) {
    std::vector<double> s;
    for (i64 item = ib; item < ie; ++item) {
      const i64 row = item / heads;
      const int h = static_cast<int>(item % heads);
      int b = 0;
      while (cu[b + 1] <= row) ++b;
      const i64 start = cu[b];
      const int len = cu[b + 1] - cu[b];
      s.assign(static_cast<std::size_t>(len), 0.0);
      double mx = -1e300;
      for (int j = 0; j < len; ++j) {
        double acc = 0;
        for (int e = 0; e < 128; ++e) {
          acc += static_cast<double>(bf2f(q[row * row_stride + static_cast<i64>(h) * 128 + e])) *
                 static_cast<double>(bf2f(k[(start + j) * row_stride + static_cast<i64>(h) * 128 + e]));
        }
        s[static_cast<std::size_t>(j)] = acc * sm_scale;
        mx = std::max(mx, s[static_cast<std::size_t>(j)]);
      }
      double den = 0;
      for (int j = 0; j < len; ++j) {
        s[static_cast<std::size_t>(j)] = std::exp(s[static_cast<std::size_t>(j)] - mx);
        den += s[static_cast<std::size_t>(j)];
      }
      for (int e = 0; e < 128; ++e) {
        double acc = 0;
        for (int j = 0; j < len; ++j) {
          acc += s[static_cast<std::size_t>(j)] * static_cast<double>(bf2f(v[(start + j) * row_stride + static_cast<i64>(h) * 128 + e]));
        }
        out[(row * heads + h) * 128 + e] = len > 0 ? static_cast<float>(acc / den) : 0.0f;
      }
    }
  });
}

// One all-INT8 DiT block on L tokens: the sequencing of moss_dit::run_block_quant's INT8 branch with 8-bit attention
// (src/models/moss_dit/dit_block_quant.cpp:365-368, 432-444, 471-480, 538-542, 590-599).
//   x [L, D] bf16 in place; mod = [shift_a, scale_a, gate_a, shift_f, scale_f, gate_f] each [D]; rope table [L, 128];
//   weights int8 with per-row f32 scales: qkv [3D, D], o [D, D], up_gate [2F, D] stored [hidden | gate], down [D, F].
//   tier 0: INT8 activations; tier 1: INT4 activations in INT8 lanes (the W4A4-via-INT8 route; weights must then hold
//   int4 values).
int orc_block_quant(u16* x, i64 L, int D, int F, int heads, const u16* mod, const u16* rope, const u16* norm1,
                    const u16* norm2, const u16* q_norm, const u16* k_norm, const i8* w_qkv, const float* s_qkv,
                    const i8* w_o, const float* s_o, const i8* w_up, const float* s_up, const i8* w_down,
                    const float* s_down, const std::int32_t* cu, int batch, int max_seqlen, float p_range, float v_range,
                    int tier) {
  const i64 dmax = std::max(D, F);
  std::vector<i8> xq(static_cast<std::size_t>(L) * dmax);
  std::vector<u8> x4(static_cast<std::size_t>(L) * dmax / 2);
  std::vector<float> xs(static_cast<std::size_t>(L));
  std::vector<u16> qkv(static_cast<std::size_t>(L) * 3 * D), attn(static_cast<std::size_t>(L) * D), ffn(static_cast<std::size_t>(L) * F);
  const auto quant_norm = [&](const u16* nw, const u16* sc, const u16* sh) {
    if (tier == 0) return orc_rms_norm_modulate_rotate_quantize(x, D, nw, sc, sh, xq.data(), D, xs.data(), L, D, nullptr, 0);
    const int rc = orc_rms_norm_modulate_convrot_quantize_int4(x, D, nw, sc, sh, x4.data(), D / 2, xs.data(), L, D);
    orc_unpack_int4(x4.data(), D / 2, xq.data(), D, L, D);
    return rc;
  };
  const auto quant_plain = [&](const u16* in, int k) {
    if (tier == 0) {
      orc_rotate_quantize(in, k, xq.data(), k, xs.data(), L, k);
    } else {
      orc_convrot_quantize_int4(in, k, x4.data(), k / 2, xs.data(), L, k);
      orc_unpack_int4(x4.data(), k / 2, xq.data(), k, L, k);
    }
  };
  if (quant_norm(norm1, mod + 1 * D, mod + 0 * D) != 0) return -1;
  orc_int8_gemm(xq.data(), D, xs.data(), w_qkv, s_qkv, L, 3 * D, D, nullptr, qkv.data(), 3 * D);
  const float sm_scale = static_cast<float>(1.0 / std::sqrt(128.0));
  orc_attention_q8(qkv.data(), 3 * D, cu, batch, heads, max_seqlen, sm_scale, p_range, v_range, 1, q_norm, k_norm, rope,
                   128, attn.data(), D);
  quant_plain(attn.data(), D);
  orc_int8_gemm_gated_residual(xq.data(), D, xs.data(), w_o, s_o, L, D, D, nullptr, mod + 2 * D, x, D);
  if (quant_norm(norm2, mod + 4 * D, mod + 3 * D) != 0) return -1;
  orc_int8_gemm_situ_glu(xq.data(), D, xs.data(), w_up, s_up, L, 2 * F, D, ffn.data(), F);
  quant_plain(ffn.data(), F);
  orc_int8_gemm_gated_residual(xq.data(), F, xs.data(), w_down, s_down, L, D, F, nullptr, mod + 5 * D, x, D);
  return 0;
}

// ------------------------------------------------------------------------------------------------ forward shell

// moss_dit::linear_fp32_row (src/models/moss_dit/dit_kernels.cu:79-93): one "warp" per output row; lane l takes the
// 8-weight chunks l, l + 32, ... with one fmaf per weight in column order; the 32 partial sums meet in a butterfly
// (lane ^ 16, 8, 4, 2, 1: every lane adds its partner's value to its own); out = bf16(lane 0's sum + bias).
void orc_linear_fp32_row(const u16* w, const float* x, const float* bias, u16* out, int n, int k) {
  parallel_for(n, g_threads, [&](i64 begin, i64 end) {
   for (i64 row = begin; row < end; ++row) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
      float acc = 0.0f;
      for (int i = l; i < k / 8; i += 32) {
        for (int j = 0; j < 8; ++j) acc = std::fmaf(bf2f(w[row * k + 8 * i + j]), x[8 * i + j], acc);
      }
      lane[l] = acc;
    }
    for (int o = 16; o > 0; o /= 2) {
      float next[32];
      for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ o];
      std::memcpy(lane, next, sizeof lane);
    }
    out[row] = f2bf(lane[0] + bias[row]);
   }
  });
}

// moss_dit::time_vector_fp32 (src/models/moss_dit/distill.cpp:126-150): the official sinusoid in double rounded to fp32,
// linear (double accumulation from the bias on, rounded to fp32), SiLU in fp32, linear.
void orc_time_vector_fp32(const float* w0, const float* b0, const float* w2, const float* b2, i64 dim, float timestep,
                          float* emb_out, float* time) {
  float emb[256];
  for (int i = 0; i < 128; ++i) {
    const double freq = std::pow(10000.0, -static_cast<double>(i) / 128);
    const double phase = static_cast<double>(timestep) * freq;
    emb[i] = static_cast<float>(std::cos(phase));
    emb[128 + i] = static_cast<float>(std::sin(phase));
  }
  if (emb_out != nullptr) std::memcpy(emb_out, emb, sizeof emb);
  std::vector<float> h(static_cast<std::size_t>(dim));
  for (i64 r = 0; r < dim; ++r) {
    double acc = b0[r];
    for (int c = 0; c < 256; ++c) acc += static_cast<double>(w0[r * 256 + c]) * emb[c];
    const float v = static_cast<float>(acc);
    h[static_cast<std::size_t>(r)] = v / (1.0f + std::exp(-v));
  }
  for (i64 r = 0; r < dim; ++r) {
    double acc = b2[r];
    for (i64 c = 0; c < dim; ++c) acc += static_cast<double>(w2[r * dim + c]) * h[static_cast<std::size_t>(c)];
    time[r] = static_cast<float>(acc);
  }
}

}  // extern "C"
