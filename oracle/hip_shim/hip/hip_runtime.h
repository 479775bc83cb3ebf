// Host stand-in for <hip/hip_runtime.h>, used only to compile the reference's scalar numeric helpers
// (src/kernels/dev.hip.hpp) with g++ for the pin tests. It defines just enough for that header to parse: the
// function-space qualifiers vanish, the bit casts become memcpy, and the AMD lane builtins (used only by wave
// reductions the pin tests never call) become identities. TEST INFRASTRUCTURE ONLY.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>

#define __device__
#define __host__
#define __global__
#define __forceinline__ inline
#define __shared__ static

struct pkv_shim_dim3 {
  unsigned x = 1, y = 1, z = 1;
};
static pkv_shim_dim3 threadIdx, blockIdx, blockDim, gridDim;
using dim3 = pkv_shim_dim3;
inline void __syncthreads() {}

inline uint32_t __float_as_uint(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float __uint_as_float(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline int __float_as_int(float f) { return int(__float_as_uint(f)); }
inline float __int_as_float(int i) { return __uint_as_float(uint32_t(i)); }

inline int __builtin_amdgcn_permlanex16(int a, int, unsigned, unsigned, bool, bool) { return a; }
inline int __builtin_amdgcn_update_dpp(int, int b, int, int, int, bool) { return b; }
inline unsigned __builtin_amdgcn_permlane16(unsigned a, unsigned, unsigned, unsigned, bool, bool) { return a; }

using std::max;
using std::min;
