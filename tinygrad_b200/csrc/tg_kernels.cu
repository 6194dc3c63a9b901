// Entry kernels for launch by tinygrad's OWN runtime (the in-graph seam: Tensor.custom_kernel with a prebuilt PROGRAM,
// tinygrad/tensor.py:390-396, tinygrad/uop/ops.py:1189-1192; precedent extra/gemm/moe_gemm.py:30-48).
//
// tinygrad's CUDA launcher passes one 8-byte device pointer per tensor, in call order, then 32-bit variables, and launches
// with the dynamic shared-memory size its CUDAProgram carries (0 unless patched): tinygrad/runtime/ops_cuda.py:18-24,37-65.
// So these kernels take pointers only, read their sizes from a small int32 tensor (`meta`), use static shared memory below
// 48 KB, and report nothing back (bad sizes make them return without touching memory).  They are compiled to a cubin, not
// linked into libb200q.so; tinygrad_b200/tg_op.py wraps the cubin as Ops.PROGRAM.
//
// b200q_tg_gemv_<type>: y[m, n_out] fp32 = x[m, n_in] fp32 . W^T for W in the packed tile layout of b200q_repack -- `Linear.__call__`
// on a GGUF weight (tinygrad/nn/__init__.py:177).  meta = {n_out, n_in, m}.  Launch: block 256, grid (ceil(ceil(n_out / 16) / 8), m).
// One warp per row tile; the tile arithmetic is the library GEMV's (qgemv_core.cuh).
#include "common.cuh"
#include "actquant.cuh"
#include "qgemv_core.cuh"

namespace {

constexpr int TG_THREADS = 256, TG_WARPS = TG_THREADS / 32;
constexpr int TG_CHUNK_GROUPS = 112;      // column groups (of 128 inputs) staged per pass: 112 * 320 B = 35 KB of static shared memory

template <int QT>
__device__ __forceinline__ void tg_gemv(float* __restrict__ y, const float* __restrict__ x, const uint8_t* __restrict__ w, const int* __restrict__ meta) {
  constexpr int TB = tile_bytes(QT);
  __shared__ __align__(16) unsigned char record[TG_CHUNK_GROUPS * XQ_GROUP_BYTES];
  __shared__ uint4 zero;
  const int n_out = meta[0], n_in = meta[1], m_rows = meta[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3, m = blockIdx.y;
  if (n_out <= 0 || n_in <= 0 || (n_in & 31) || m >= m_rows) return;
  const int kgroups = (n_in + GROUP_ELEMS - 1) / GROUP_ELEMS, n_row_tiles = (n_out + TILE_ROWS - 1) / TILE_ROWS;
  const int rt = blockIdx.x * TG_WARPS + warp;
  if (tid == 0) zero = make_uint4(0, 0, 0, 0);
  const bool diag = (t == (g & 3));
  float acc0 = 0.f, acc1 = 0.f;
  for (int k0 = 0; k0 < kgroups; k0 += TG_CHUNK_GROUPS) {
    const int kg = min(TG_CHUNK_GROUPS, kgroups - k0);
    __syncthreads();                               // the previous chunk's record is no longer read
    const XqDst dst(record, kg);
    for (int b = tid >> 3; b < kg * 4; b += TG_THREADS / 8) {      // 8 threads per block of 32 inputs
      const int k = (k0 * 4 + b) * 32 + 4 * (tid & 7);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < n_in) v = *reinterpret_cast<const float4*>(x + (size_t)m * n_in + k);
      quant_block_8x4(v, tid & 7, b, dst);
    }
    __syncthreads();
    if (rt < n_row_tiles) {
      const uint4* xq = reinterpret_cast<const uint4*>(record);
      const float4* xsc = reinterpret_cast<const float4*>(record + (size_t)kg * 256);
      const uint8_t* tile = w + ((size_t)rt * kgroups + k0) * TB;
      for (int j = 0; j < kg; j++) {
        const uint4 bq0 = diag ? xq[(j * 2 + 0) * 8 + g] : zero, bq1 = diag ? xq[(j * 2 + 1) * 8 + g] : zero;
        const float4 st = xsc[(j * 2 + (t >> 1)) * 2 + (t & 1)];
        tile_mac<QT>(tile + (size_t)j * TB, lane, bq0, bq1, st, acc0, acc1);
      }
    }
  }
  if (rt >= n_row_tiles) return;
  acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1); acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
  acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
  if (t == 0) {
    const int r0 = rt * 16 + g, r1 = r0 + 8;
    if (r0 < n_out) y[(size_t)m * n_out + r0] = acc0;
    if (r1 < n_out) y[(size_t)m * n_out + r1] = acc1;
  }
}

}  // namespace

extern "C" __global__ void __launch_bounds__(256) b200q_tg_gemv_q4_0(float* y, const float* x, const unsigned char* w, const int* meta) {
  tg_gemv<B200Q_Q4_0>(y, x, w, meta);
}
extern "C" __global__ void __launch_bounds__(256) b200q_tg_gemv_q8_0(float* y, const float* x, const unsigned char* w, const int* meta) {
  tg_gemv<B200Q_Q8_0>(y, x, w, meta);
}

// The same kernels through the library, with the launch geometry tinygrad_b200/tg_op.py gives tinygrad: lets the parity tests run
// exactly the code tinygrad's runtime would launch, on a machine without tinygrad.
extern "C" int b200q_tg_gemv(int qtype, float* y, const float* x, const void* w_packed, const int32_t* meta_dev, int n_out, int m, void* stream) {
  if (!y || !x || !w_packed || !meta_dev || n_out <= 0 || m <= 0 || m > 65535) return B200Q_ERR_BAD_ARG;
  if (qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0) return B200Q_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)w_packed) & 15) return B200Q_ERR_MISALIGNED;
  const dim3 grid(ceil_div(ceil_div(n_out, TILE_ROWS), TG_WARPS), m), block(TG_THREADS);
  if (qtype == B200Q_Q4_0) b200q_tg_gemv_q4_0<<<grid, block, 0, (cudaStream_t)stream>>>(y, x, (const unsigned char*)w_packed, meta_dev);
  else b200q_tg_gemv_q8_0<<<grid, block, 0, (cudaStream_t)stream>>>(y, x, (const unsigned char*)w_packed, meta_dev);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
