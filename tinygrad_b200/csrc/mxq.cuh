// MXFP8 quantiser arithmetic shared by the byte kernels (mxfp8.cu) and the fused GEMM epilogue (mxfp8_gemm.cu).
#pragma once
#include <cuda_fp8.h>
#include <math.h>

namespace {

// ---------------------------------------------------------------------------
// quantize_mxfp8: one warp per block of 32 values, lane = element.
//   e8 = clamp(floor(log2(max(amax, 1e-38))) + 127, 0, 254);  q = e4m3(clamp(x * 2^(127 - e8), +-448))
// floor(log2()) is taken the way the reference's fp32 tensor op yields it: log2 rounded to fp32, then floor
// (so an amax within half an fp32 ulp below a power of two lands on that power).
__device__ __forceinline__ uint8_t mx_scale_exponent(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  // at most 10 mantissa bits (any bf16 / fp16 value): log2 stays more than half an fp32 ulp below the next integer, so the
  // floor is the exponent field itself (0 for everything below 2^-126, like the 1e-38 clamp; 255 = inf/nan clamps to 254)
  if ((bits & 0x1FFFu) == 0) return (uint8_t)min((bits >> 23) & 0xFFu, 254u);
  const float lg = (float)log2((double)fmaxf(amax, 1e-38f));
  const float e = fminf(fmaxf(floorf(lg) + 127.f, 0.f), 254.f);
  return (uint8_t)e;
}
__device__ __forceinline__ float mx_inv_scale(uint8_t e8) {     // 2^(127 - e8), exact (2^-127 is a denormal)
  return e8 < 254 ? __uint_as_float((uint32_t)(254 - e8) << 23) : __uint_as_float(0x00400000u);
}
// eight values -> eight E4M3 codes (round to nearest even, saturating), element i in byte i
__device__ __forceinline__ uint2 mx_quant8(const float (&v)[8], uint8_t e8) {
  const float sc = mx_inv_scale(e8);
  uint32_t w[2];
#pragma unroll
  for (int h = 0; h < 2; h++) {
    uint32_t acc = 0;
#pragma unroll
    for (int p = 0; p < 2; p++) {
      const float a = fminf(fmaxf(v[h * 4 + p * 2] * sc, -448.f), 448.f), b = fminf(fmaxf(v[h * 4 + p * 2 + 1] * sc, -448.f), 448.f);
      acc |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3) << (16 * p);
    }
    w[h] = acc;
  }
  return make_uint2(w[0], w[1]);
}

}  // namespace
