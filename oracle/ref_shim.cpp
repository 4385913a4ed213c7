// C entry points over the reference project's own block codecs, so the tests can call them through ctypes. This file
// holds no codec code: QuantizeQ8_0 and Dequantize come from the reference's engine/core/gguf_quant.cpp, compiled from
// where it lies by oracle/Makefile into oracle/_ref/. TEST INFRASTRUCTURE ONLY; nothing shipped links against it.
#include <cstdint>

#include "core/gguf_quant.hpp"

extern "C" {

// engine/core/gguf_quant.cpp:310-320
void yah_ref_quantize_q8_0(const float* x, std::uint64_t n, std::uint8_t* dst) { yah::core::QuantizeQ8_0(x, n, dst); }

// engine/core/gguf_quant.cpp:291-308; type ids are ggml's (Q4_0 = 2, Q8_0 = 8). Returns -1 where the reference throws.
int yah_ref_dequantize(std::uint32_t type, const std::uint8_t* src, float* dst, std::uint64_t n) {
  try {
    yah::core::Dequantize(static_cast<yah::core::GgmlType>(type), src, dst, n);
    return 0;
  } catch (...) {
    return -1;
  }
}

}  // extern "C"
