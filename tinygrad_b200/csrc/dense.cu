// Dense (unquantised) weight GEMV: y[m, n_out] = f(x)[m, n_in] . W[n_out, n_in]^T with W stored fp16, bf16 or fp32.
// It serves the Linears a GGUF file keeps unquantised or in a block format without a fused kernel (F16 / F32 / BF16 tensors,
// Q6_K after b200q_dequant_raw to fp16): the router `ffn_gate_inp`, tied or Q6_K output heads.  Same call shape as the
// quantised GEMV: optional fused RMSNorm on the activations (tinygrad/nn/__init__.py:300-304), bias, residual.
// Numerics: weight as stored, widened to fp32; fp32 products and fp32 accumulation (tinygrad/mixin/op.py:367-392 with
// fp32 activations; with fp16 activations the products are formed from the fp16-rounded activation, which is what
// least_upper_dtype gives for an fp16 weight).  HBM-bound: 16-byte weight loads, four in flight per lane, activations staged
// once per CTA in shared memory, a persistent grid of a few CTAs per SM.
#include "common.cuh"
#include <cuda_bf16.h>

namespace {

constexpr int THREADS = 256, WARPS = THREADS / 32, MAX_M = 4;

template <typename W> struct WLoad;
template <> struct WLoad<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 u = ldg_stream(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
};
template <> struct WLoad<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = ldg_stream(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
  }
};
template <> struct WLoad<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const uint4 a = ldg_stream(reinterpret_cast<const uint4*>(p)), b = ldg_stream(reinterpret_cast<const uint4*>(p + 4));
    v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
  }
};

struct DenseParams {
  const void* w; const void* x; const __half* norm_w; const __half* bias; const void* residual; void* y;
  int n_out, n_in, m; float eps; bool x_f16, y_f16;
};

template <typename W, int M>
__global__ void __launch_bounds__(THREADS) dense_gemv_kernel(const DenseParams p) {
  extern __shared__ float xs[];                    // [M][n_in]
  __shared__ float red[WARPS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t row0 = (size_t)blockIdx.y * MAX_M;        // this CTA's group of activation rows
  pdl_launch_dependents();
  pdl_wait();
  // stage the activations (normalised like RMSNorm: fp32 x * rsqrt(mean(x^2) + eps), cast to the input dtype, times the weight)
#pragma unroll 1
  for (int r = 0; r < M; r++) {
    float ss = 0.f;
    for (int i = tid; i < p.n_in; i += THREADS) {
      const float v = p.x_f16 ? __half2float(reinterpret_cast<const __half*>(p.x)[(row0 + r) * p.n_in + i]) : reinterpret_cast<const float*>(p.x)[(row0 + r) * p.n_in + i];
      xs[r * p.n_in + i] = v;
      ss += v * v;
    }
    if (p.norm_w) {
      ss = warp_sum(ss);
      __syncthreads();
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < WARPS; i++) tot += red[i];
      const float sc = 1.0f / sqrtf(tot / (float)p.n_in + p.eps);
      for (int i = tid; i < p.n_in; i += THREADS) {
        float n = xs[r * p.n_in + i] * sc;
        if (p.x_f16) n = __half2float(__float2half_rn(n));
        xs[r * p.n_in + i] = n * __half2float(p.norm_w[i]);
      }
    }
  }
  __syncthreads();
  const W* w = reinterpret_cast<const W*>(p.w);
  for (int row = blockIdx.x * WARPS + warp; row < p.n_out; row += gridDim.x * WARPS) {
    const W* wr = w + (size_t)row * p.n_in;
    float acc[M];
#pragma unroll
    for (int r = 0; r < M; r++) acc[r] = 0.f;
    int c = lane * 8;
    for (int c0 = 0; c0 + 4 * 256 <= p.n_in; c0 += 4 * 256, c += 4 * 256) {          // four 16-byte loads in flight
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; u++) WLoad<W>::load(wr + c + u * 256, v[u]);
#pragma unroll
      for (int u = 0; u < 4; u++)
#pragma unroll
        for (int r = 0; r < M; r++) {
          const float4 x0 = *reinterpret_cast<const float4*>(xs + r * p.n_in + c + u * 256), x1 = *reinterpret_cast<const float4*>(xs + r * p.n_in + c + u * 256 + 4);
          acc[r] += v[u][0] * x0.x + v[u][1] * x0.y + v[u][2] * x0.z + v[u][3] * x0.w + v[u][4] * x1.x + v[u][5] * x1.y + v[u][6] * x1.z + v[u][7] * x1.w;
        }
    }
    for (; c < p.n_in; c += 256) {
      float v[8];
      WLoad<W>::load(wr + c, v);
#pragma unroll
      for (int r = 0; r < M; r++) {
        const float4 x0 = *reinterpret_cast<const float4*>(xs + r * p.n_in + c), x1 = *reinterpret_cast<const float4*>(xs + r * p.n_in + c + 4);
        acc[r] += v[0] * x0.x + v[1] * x0.y + v[2] * x0.z + v[3] * x0.w + v[4] * x1.x + v[5] * x1.y + v[6] * x1.z + v[7] * x1.w;
      }
    }
#pragma unroll
    for (int r = 0; r < M; r++) {
      float s = warp_sum(acc[r]);
      if (lane == 0) {
        if (p.bias) s += __half2float(p.bias[row]);
        const size_t o = (row0 + r) * p.n_out + row;
        if (p.residual) s += p.y_f16 ? __half2float(reinterpret_cast<const __half*>(p.residual)[o]) : reinterpret_cast<const float*>(p.residual)[o];
        if (p.y_f16) reinterpret_cast<__half*>(p.y)[o] = __float2half_rn(s); else reinterpret_cast<float*>(p.y)[o] = s;
      }
    }
  }
}

// m rows = full groups of MAX_M rows (grid.y of them, M = MAX_M) and one launch for the remainder
template <typename W>
cudaError_t launch_dense_m(const DenseParams& p, int mrows, int groups, int grid, size_t smem, cudaStream_t st, bool pdl) {
  switch (mrows) {
    case 1: cudaFuncSetAttribute(dense_gemv_kernel<W, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); return launch_k(dense_gemv_kernel<W, 1>, dim3(grid, groups), dim3(THREADS), smem, st, pdl, p);
    case 2: cudaFuncSetAttribute(dense_gemv_kernel<W, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); return launch_k(dense_gemv_kernel<W, 2>, dim3(grid, groups), dim3(THREADS), smem, st, pdl, p);
    case 3: cudaFuncSetAttribute(dense_gemv_kernel<W, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); return launch_k(dense_gemv_kernel<W, 3>, dim3(grid, groups), dim3(THREADS), smem, st, pdl, p);
    default: cudaFuncSetAttribute(dense_gemv_kernel<W, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); return launch_k(dense_gemv_kernel<W, 4>, dim3(grid, groups), dim3(THREADS), smem, st, pdl, p);
  }
}
template <typename W>
cudaError_t launch_dense(const DenseParams& p0, int grid, size_t smem, cudaStream_t st, bool pdl) {
  DenseParams p = p0;
  const int full = p.m / MAX_M, rem = p.m % MAX_M;
  const size_t xsz = p.x_f16 ? 2 : 4, ysz = p.y_f16 ? 2 : 4;
  if (full) {
    cudaError_t e = launch_dense_m<W>(p, MAX_M, full, grid, smem, st, pdl);
    if (e != cudaSuccess) return e;
    p.x = (const char*)p.x + (size_t)full * MAX_M * p.n_in * xsz;
    p.y = (char*)p.y + (size_t)full * MAX_M * p.n_out * ysz;
    if (p.residual) p.residual = (const char*)p.residual + (size_t)full * MAX_M * p.n_out * ysz;
  }
  return rem ? launch_dense_m<W>(p, rem, 1, grid, smem, st, pdl && !full) : cudaSuccess;
}

// out[i] = silu(gate[i]) * up[i]: the SwiGLU product behind two separate dense Linears (tinygrad/llm/model.py:137)
__global__ void silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float g = gate[i];
    out[i] = (g / (1.f + __expf(-g))) * up[i];
  }
}

}  // namespace

extern "C" int b200q_silu_mul(const float* gate, const float* up, float* out, int64_t n, int flags, void* stream) {
  if (!gate || !up || !out || n < 0) return B200Q_ERR_BAD_ARG;
  if (n == 0) return B200Q_OK;
  const int64_t blocks = (n + 255) / 256;
  B200Q_CHECK_CUDA(launch_k(silu_mul_kernel, dim3((unsigned)(blocks < 1024 ? blocks : 1024)), dim3(256), 0, (cudaStream_t)stream, (flags & B200Q_FLAG_PDL) != 0,
                            gate, up, out, n));
  return B200Q_OK;
}

extern "C" int b200q_gemv_dense(const void* w, int w_dtype, int n_out, int n_in, int m, const void* x, int x_dtype, const void* norm_weight,
                                float norm_eps, const void* bias, const void* residual, void* y, int y_dtype, int flags, void* stream) {
  if (!w || !x || !y || n_out <= 0 || n_in <= 0 || m <= 0) return B200Q_ERR_BAD_ARG;
  if (w_dtype != B200Q_F16 && w_dtype != B200Q_F32 && w_dtype != B200Q_BF16) return B200Q_ERR_BAD_ARG;
  if ((x_dtype != B200Q_F16 && x_dtype != B200Q_F32) || (y_dtype != B200Q_F16 && y_dtype != B200Q_F32)) return B200Q_ERR_BAD_ARG;
  if (n_in % 8) return B200Q_ERR_BAD_SHAPE;                                // 16-byte loads of 8 fp16 weights
  const size_t smem = (size_t)(m < MAX_M ? m : MAX_M) * n_in * sizeof(float);
  if (smem > 200 * 1024) return B200Q_ERR_TOO_LARGE;
  if (((uintptr_t)w & 15) || ((uintptr_t)x & 3)) return B200Q_ERR_MISALIGNED;
  const int n_sm = b200q_sm_count();
  if (n_sm <= 0) return B200Q_ERR_CUDA;
  DenseParams p;
  p.w = w; p.x = x; p.norm_w = (const __half*)norm_weight; p.bias = (const __half*)bias; p.residual = residual; p.y = y;
  p.n_out = n_out; p.n_in = n_in; p.m = m; p.eps = norm_eps; p.x_f16 = x_dtype == B200Q_F16; p.y_f16 = y_dtype == B200Q_F16;
  const int per_sm = smem > 96 * 1024 ? 1 : smem > 48 * 1024 ? 2 : 4;
  const int grid = min(ceil_div(n_out, WARPS), m > MAX_M ? 8 : n_sm * per_sm);      // many row groups already fill the GPU
  const bool pdl = flags & B200Q_FLAG_PDL;
  cudaError_t e = w_dtype == B200Q_F16 ? launch_dense<__half>(p, grid, smem, (cudaStream_t)stream, pdl)
                : w_dtype == B200Q_BF16 ? launch_dense<__nv_bfloat16>(p, grid, smem, (cudaStream_t)stream, pdl)
                                        : launch_dense<float>(p, grid, smem, (cudaStream_t)stream, pdl);
  B200Q_CHECK_CUDA(e);
  return B200Q_OK;
}
