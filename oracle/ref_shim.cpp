// Thin C wrapper that compiles the reference's OWN host code for the Q4_K format
// (engine/src/quant.h of the reference checkout, included from where it lies; nothing is copied).
// Built only when the reference checkout is present; used to pin the restatement in hp_oracle.cpp.
#include <algorithm>   // quant.h:162-168 uses std::min/max without including it
#include <cstdint>
#include "engine/src/quant.h"

extern "C" {
float ref_f16_to_f32(uint16_t h) { return hip::f16_to_f32(h); }
uint16_t ref_f32_to_f16(float f) { return hip::f32_to_f16(f); }
void ref_get_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) { hip::get_scale_min_k4(j, q, d, m); }
// dequant_row(type 12 = Q4_K, ...) : quant.h:185-201
void ref_dequant_row_q4k(const uint8_t* src, float* dst, uint64_t ne0) { hip::dequant_row(12, src, dst, ne0); }
}
