// Grouped (per-expert) MXFP8 GEMM:  C[M, N] (bf16) = A_q[M, K] (e4m3) x B_q[e(row)][N, K]^T (e4m3),
// both operands scaled by one E8M0 exponent per 32 along K, fp32 accumulation.
// Rows of A are grouped by expert: group e = rows off[e] .. off[e+1], every group a multiple of 256 rows.
// Semantics: extra/gemm/moe_gemm.py:112-134 over the kernel contract of extra/thunder/amd/grouped_mxfp8_gemm.cpp:32-158
// (the reference computation it is tested against: dequantised operands matmul, test/backend/test_asm_gemm.py:289-292,306).
//
// This version runs the contraction on fp8 mma.sync (m16n8k32, one MMA = exactly one scale block along K) and applies
// the two block scales to each MMA's partial product in fp32.  128 x 128 x 128 tiles, 8 warps (2 x 4), 3-stage cp.async
// pipeline, shared-memory rows padded to 144 bytes (conflict-free 32-bit fragment loads).
#include "common.cuh"
#include <cuda_bf16.h>

namespace {

constexpr int BM = 128, BN = 128, BK = 128, STAGES = 3, ROWB = BK + 16;     // padded row bytes
constexpr int STAGE_BYTES = (BM + BN) * ROWB + (BM + BN) * 4;               // tiles + one u32 of 4 scale bytes per row
constexpr int THREADS = 256;

__device__ __forceinline__ void cp16(void* s, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(s)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp4(void* s, const void* g) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(s)), "l"(g) : "memory");
}
__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ float e8_scale(uint32_t packed, int kb) { return __uint_as_float(((packed >> (8 * kb)) & 0xFFu) << 23); }  // 2^(e8-127)

__global__ void __launch_bounds__(THREADS) grouped_mxfp8_gemm_kernel(const uint8_t* __restrict__ a_q, const uint8_t* __restrict__ a_e8,
                                                                     const uint8_t* __restrict__ b_q, const uint8_t* __restrict__ b_e8,
                                                                     const int32_t* __restrict__ off, int n_experts, int m_total, int n, int k,
                                                                     __nv_bfloat16* __restrict__ c) {
  extern __shared__ __align__(16) unsigned char sm[];
  __shared__ int s_expert;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (tid == 0) {
    int e = -1;
    for (int i = 0; i < n_experts; i++) if (m0 >= off[i] && m0 < off[i + 1]) { e = i; break; }
    s_expert = e;
  }
  __syncthreads();
  const int expert = s_expert;
  if (expert < 0) return;                       // tile past the last group: nothing routed there
  const int kb_total = k >> 5;
  const uint8_t* bq = b_q + (size_t)expert * n * k;
  const uint8_t* be = b_e8 + (size_t)expert * n * kb_total;
  const int ktiles = k / BK;

  auto load_stage = [&](int stage, int kt) {
    unsigned char* sA = sm + stage * STAGE_BYTES;
    unsigned char* sB = sA + BM * ROWB;
    uint32_t* sSA = reinterpret_cast<uint32_t*>(sB + BN * ROWB);
    uint32_t* sSB = sSA + BM;
    for (int i = tid; i < BM * (BK / 16); i += THREADS) {
      const int r = i >> 3, ch = i & 7;
      cp16(sA + r * ROWB + ch * 16, a_q + (size_t)(m0 + r) * k + kt * BK + ch * 16);
      cp16(sB + r * ROWB + ch * 16, bq + (size_t)(n0 + r) * k + kt * BK + ch * 16);
    }
    if (tid < BM) cp4(sSA + tid, a_e8 + (size_t)(m0 + tid) * kb_total + kt * 4);
    else cp4(sSB + (tid - BM), be + (size_t)(n0 + tid - BM) * kb_total + kt * 4);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int l = 0; l < 4; l++) acc[i][j][l] = 0.f;

  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  for (int s = 0; s < STAGES - 1; s++) { if (s < ktiles) load_stage(s, s); else asm volatile("cp.async.commit_group;" ::: "memory"); }
  for (int kt = 0; kt < ktiles; kt++) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    if (kt + STAGES - 1 < ktiles) load_stage((kt + STAGES - 1) % STAGES, kt + STAGES - 1);
    else asm volatile("cp.async.commit_group;" ::: "memory");
    const unsigned char* sA = sm + (kt % STAGES) * STAGE_BYTES;
    const unsigned char* sB = sA + BM * ROWB;
    const uint32_t* sSA = reinterpret_cast<const uint32_t*>(sB + BN * ROWB);
    const uint32_t* sSB = sSA + BM;
    uint32_t pa[4][2], pb[4][2];               // packed scale bytes of this thread's rows / columns
#pragma unroll
    for (int i = 0; i < 4; i++) { pa[i][0] = sSA[wm + i * 16 + g]; pa[i][1] = sSA[wm + i * 16 + g + 8]; }
#pragma unroll
    for (int j = 0; j < 4; j++) { pb[j][0] = sSB[wn + j * 8 + 2 * t]; pb[j][1] = sSB[wn + j * 8 + 2 * t + 1]; }
#pragma unroll
    for (int kb = 0; kb < 4; kb++) {
      uint32_t af[4][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const unsigned char* p = sA + (wm + i * 16 + g) * ROWB + kb * 32 + 4 * t;
        af[i][0] = *reinterpret_cast<const uint32_t*>(p);
        af[i][1] = *reinterpret_cast<const uint32_t*>(p + 8 * ROWB);
        af[i][2] = *reinterpret_cast<const uint32_t*>(p + 16);
        af[i][3] = *reinterpret_cast<const uint32_t*>(p + 8 * ROWB + 16);
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const unsigned char* p = sB + (wn + j * 8 + g) * ROWB + kb * 32 + 4 * t;
        bf[j][0] = *reinterpret_cast<const uint32_t*>(p);
        bf[j][1] = *reinterpret_cast<const uint32_t*>(p + 16);
      }
      float sa[4][2], sb[4][2];
#pragma unroll
      for (int i = 0; i < 4; i++) { sa[i][0] = e8_scale(pa[i][0], kb); sa[i][1] = e8_scale(pa[i][1], kb); }
#pragma unroll
      for (int j = 0; j < 4; j++) { sb[j][0] = e8_scale(pb[j][0], kb); sb[j][1] = e8_scale(pb[j][1], kb); }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float d[4];
          mma_e4m3(d, af[i][0], af[i][1], af[i][2], af[i][3], bf[j][0], bf[j][1]);
          acc[i][j][0] = fmaf(d[0], sa[i][0] * sb[j][0], acc[i][j][0]);
          acc[i][j][1] = fmaf(d[1], sa[i][0] * sb[j][1], acc[i][j][1]);
          acc[i][j][2] = fmaf(d[2], sa[i][1] * sb[j][0], acc[i][j][2]);
          acc[i][j][3] = fmaf(d[3], sa[i][1] * sb[j][1], acc[i][j][3]);
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int row = m0 + wm + i * 16 + g, col = n0 + wn + j * 8 + 2 * t;
      *reinterpret_cast<__nv_bfloat162*>(c + (size_t)row * n + col) = __floats2bfloat162_rn(acc[i][j][0], acc[i][j][1]);
      *reinterpret_cast<__nv_bfloat162*>(c + (size_t)(row + 8) * n + col) = __floats2bfloat162_rn(acc[i][j][2], acc[i][j][3]);
    }
}

}  // namespace

extern "C" int b200q_grouped_mxfp8_gemm(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                                        int m_total, int n, int k, void* c_bf16, void* stream) {
  if (!a_q || !a_e8 || !b_q || !b_e8 || !off || !c_bf16 || n_experts <= 0 || m_total <= 0 || n <= 0 || k <= 0) return B200Q_ERR_BAD_ARG;
  if (m_total % 256 || n % BN || k % BK) return B200Q_ERR_BAD_SHAPE;       // the reference asks M % 256 == N % 256 == K % 128 == 0 (moe_gemm.py:120)
  if (((uintptr_t)a_q | (uintptr_t)b_q | (uintptr_t)c_bf16) & 15 || ((uintptr_t)a_e8 | (uintptr_t)b_e8) & 3) return B200Q_ERR_MISALIGNED;
  static bool attr = false;
  if (!attr) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(grouped_mxfp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STAGES * STAGE_BYTES));
    attr = true;
  }
  dim3 grid(n / BN, m_total / BM);
  grouped_mxfp8_gemm_kernel<<<grid, THREADS, STAGES * STAGE_BYTES, (cudaStream_t)stream>>>(
      (const uint8_t*)a_q, (const uint8_t*)a_e8, (const uint8_t*)b_q, (const uint8_t*)b_e8, off, n_experts, m_total, n, k, (__nv_bfloat16*)c_bf16);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
