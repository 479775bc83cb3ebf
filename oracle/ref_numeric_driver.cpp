// Exports the reference's own scalar numeric helpers (src/kernels/dev.hip.hpp, compiled where it lies under the
// reference checkout through oracle/hip_shim) behind a C interface, so the pin tests can sweep the CPU oracle
// against them. Built only where the reference checkout is present; output goes to oracle/_ref/. TEST
// INFRASTRUCTURE ONLY.
#include "kernels/dev.hip.hpp"

namespace d = unholy::dev;

extern "C" {
float ref_bf16_to_f32(uint16_t v) { return d::bf16_to_f32(v); }
uint16_t ref_f32_to_bf16(float f) { return d::f32_to_bf16(f); }
float ref_e4m3_to_f32(uint8_t v) { return d::e4m3_to_f32(v); }
uint8_t ref_f32_to_e4m3(float x) { return d::f32_to_e4m3(x); }
float ref_e8m0_to_f32(uint8_t v) { return d::e8m0_to_f32(v); }
float ref_e2m1_to_f32(uint32_t n) { return d::e2m1_to_f32(n); }
float ref_round_e2m1(float x) { return d::round_e2m1(x); }
uint8_t ref_pow2_ceil_e8m0(float v) { return d::pow2_ceil_e8m0(v); }

// Array sweeps (one call per test instead of one per value).
void ref_f32_to_bf16_n(const float* x, uint16_t* y, long n) {
  for (long i = 0; i < n; ++i) y[i] = d::f32_to_bf16(x[i]);
}
void ref_f32_to_e4m3_n(const float* x, uint8_t* y, long n) {
  for (long i = 0; i < n; ++i) y[i] = d::f32_to_e4m3(x[i]);
}
void ref_round_e2m1_n(const float* x, float* y, long n) {
  for (long i = 0; i < n; ++i) y[i] = d::round_e2m1(x[i]);
}
void ref_pow2_ceil_e8m0_n(const float* x, uint8_t* y, long n) {
  for (long i = 0; i < n; ++i) y[i] = d::pow2_ceil_e8m0(x[i]);
}
}
