// Per-tensor FP8 (E4M3) linear: `quantize_to_fp8` and the scaling behind the product of `FP8Linear.__call__`
// (extra/fp8/fp8_linear.py:4-16,43-63): scale = 448 / (max|x| + 1e-8) over the WHOLE tensor, q = e4m3(clamp(x * scale, +-448)), the
// returned factor is 1 / scale; y = (x_q . w_q^T, fp32) * w_factor * x_factor + bias, cast to the activation dtype.
// The contraction itself is the grouped tcgen05 GEMM with unit block scales and fp32 output (b200q_grouped_mxfp8_gemm_f32).
#include "common.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, int64_t i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

// |x| is non-negative, so its bit pattern orders like the value: the maximum is an integer atomicMax (NaN inputs are not expected)
template <typename T>
__global__ void fp8_absmax_kernel(const T* __restrict__ x, int64_t n, unsigned* __restrict__ amax_bits) {
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) m = fmaxf(m, fabsf(ldf<T>(x, i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));
}

template <typename T>
__global__ void fp8_quantize_kernel(const T* __restrict__ x, int64_t n, const float* __restrict__ amax, uint8_t* __restrict__ q, float* __restrict__ factor) {
  const float d = __fadd_rn(*amax, 1e-8f), scale = __fdiv_rn(448.f, d);
  if (blockIdx.x == 0 && threadIdx.x == 0) *factor = __fmul_rn(d, 1.f / 448.f);      // the reference's simplified (448 / d).reciprocal()
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = fminf(fmaxf(__fmul_rn(ldf<T>(x, i), scale), -448.f), 448.f);
    q[i] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  }
}

template <typename T> __device__ __forceinline__ void stf(T* p, int64_t i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, int64_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__half>(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

template <typename T>
__global__ void fp8_scale_bias_kernel(const float* __restrict__ acc, int64_t rows, int n, const float* __restrict__ fw, const float* __restrict__ fx,
                                      const float* __restrict__ bias, T* __restrict__ y) {
  const float w = *fw, xx = *fx;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rows * n; i += (int64_t)gridDim.x * blockDim.x) {
    float v = __fmul_rn(__fmul_rn(acc[i], w), xx);                 // y * w_scale * x_scale, in that order
    if (bias) v = __fadd_rn(v, bias[i % n]);
    stf<T>(y, i, v);
  }
}

int grid_for(int64_t n) { const int64_t b = (n + 255) / 256; return (int)(b < 1 ? 1 : (b > 4096 ? 4096 : b)); }

}  // namespace

extern "C" int b200q_fp8_absmax(const void* x, int x_dtype, int64_t n, float* amax, void* stream) {
  if (!x || !amax || n <= 0) return B200Q_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  B200Q_CHECK_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), st));
  if (x_dtype == B200Q_F32) fp8_absmax_kernel<float><<<grid_for(n), 256, 0, st>>>((const float*)x, n, (unsigned*)amax);
  else if (x_dtype == B200Q_F16) fp8_absmax_kernel<__half><<<grid_for(n), 256, 0, st>>>((const __half*)x, n, (unsigned*)amax);
  else if (x_dtype == B200Q_BF16) fp8_absmax_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((const __nv_bfloat16*)x, n, (unsigned*)amax);
  else return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_fp8_quantize(const void* x, int x_dtype, int64_t n, const float* amax, void* q, float* factor, void* stream) {
  if (!x || !amax || !q || !factor || n <= 0) return B200Q_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (x_dtype == B200Q_F32) fp8_quantize_kernel<float><<<grid_for(n), 256, 0, st>>>((const float*)x, n, amax, (uint8_t*)q, factor);
  else if (x_dtype == B200Q_F16) fp8_quantize_kernel<__half><<<grid_for(n), 256, 0, st>>>((const __half*)x, n, amax, (uint8_t*)q, factor);
  else if (x_dtype == B200Q_BF16) fp8_quantize_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, st>>>((const __nv_bfloat16*)x, n, amax, (uint8_t*)q, factor);
  else return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_fp8_scale_bias(const float* acc, int64_t rows, int n, const float* factor_w, const float* factor_x, const float* bias, void* y, int y_dtype,
                                    void* stream) {
  if (!acc || !factor_w || !factor_x || !y || rows <= 0 || n <= 0) return B200Q_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = grid_for(rows * n);
  if (y_dtype == B200Q_F32) fp8_scale_bias_kernel<float><<<g, 256, 0, st>>>(acc, rows, n, factor_w, factor_x, bias, (float*)y);
  else if (y_dtype == B200Q_F16) fp8_scale_bias_kernel<__half><<<g, 256, 0, st>>>(acc, rows, n, factor_w, factor_x, bias, (__half*)y);
  else if (y_dtype == B200Q_BF16) fp8_scale_bias_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(acc, rows, n, factor_w, factor_x, bias, (__nv_bfloat16*)y);
  else return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
