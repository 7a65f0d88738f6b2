// C-ABI shim over the reference's own CPU weight codec (src/weights/quant/quant_codec.{h,cpp}), compiled from the
// reference tree where it lies; used only to validate the oracle's restatement. TEST INFRASTRUCTURE ONLY.
#include <cstdint>

#include "weights/quant/quant_codec.h"

extern "C" {

int ref_quantize_convrot_rows_bf16(const std::uint16_t* w, std::int64_t rows, std::int64_t k, int g, std::int8_t* q,
                                   float* scale) {
  return mi::quant::quantize_convrot_rows_bf16(w, rows, k, g, q, scale) ? 0 : -1;
}

int ref_decode_grouped_rows(const std::uint8_t* packed, const std::uint8_t* s_rel, const float* codebook,
                            std::int64_t rows, std::int64_t k, int bits, int group, std::int8_t* out) {
  return mi::quant::decode_grouped_rows(packed, s_rel, codebook, rows, k, bits, group, out) ? 0 : -1;
}

void ref_decode_int4_rows(const std::uint8_t* packed, std::int64_t rows, std::int64_t k, std::int8_t* out) {
  mi::quant::decode_int4_rows(packed, rows, k, out);
}

float ref_e4m3_to_float(std::uint8_t v) { return mi::quant::e4m3_to_float(v); }

int ref_hadamard_sign(int g, int i, int j) { return mi::quant::hadamard_sign(g, i, j); }

}  // extern "C"
