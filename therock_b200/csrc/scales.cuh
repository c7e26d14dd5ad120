// Scale rules shared by the quantising row kernels and the block-scaled GEMM epilogue.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fmoe {

// Scale of one 1x128 group from its absolute maximum.  f32 flavour: absmax/448.  UE8M0 flavour:
// the smallest power of two that is >= absmax/448, clamped to the exponent range 1..254 of the
// format; `byte` receives the biased exponent.
template <bool kHw>
__device__ __forceinline__ float group_scale(float amax, uint32_t& byte) {
  if (amax <= 0.0f) { byte = 127u; return 1.0f; }
  const float t = amax / 448.0f;
  if (!kHw) { byte = 0u; return t; }
  const uint32_t bits = __float_as_uint(t);
  uint32_t e = (bits >> 23) + ((bits & 0x7fffffu) ? 1u : 0u);
  e = e < 1u ? 1u : (e > 254u ? 254u : e);
  byte = e;
  return __uint_as_float(e << 23);
}

// UE8M0 scale arrays are row-major bytes [rows, pitch], pitch = K groups rounded up to four.
__host__ __device__ __forceinline__ int scale_pitch(int k_groups) { return (k_groups + 3) & ~3; }

}  // namespace fmoe
