// Grouped (per-expert) MXFP8 GEMM on the 5th-generation tensor cores:
//   C[M, N] (bf16) = A_q[M, K] (e4m3) x B_q[e(row)][N, K]^T (e4m3), one E8M0 scale per 32 along K on both operands, fp32 accumulation.
// Rows of A are grouped by expert: group e = rows off[e] .. off[e+1], every group a multiple of 256 rows.
// Semantics: extra/gemm/moe_gemm.py:112-134 over the kernel contract of extra/thunder/amd/grouped_mxfp8_gemm.cpp:32-158
// (the reference computation it is tested against: dequantised operands matmul, test/backend/test_asm_gemm.py:289-292,306).
//
// One CTA computes a 128 x 256 tile with tcgen05.mma kind::mxf8f6f4.block_scale (scale_vec::1X): the tensor core applies both
// block scales itself.  Operands are staged by cp.async into a 4-stage ring of shared-memory tiles in the canonical K-major
// no-swizzle layout (8 rows x 16 bytes core matrices; one MMA covers K = 32 = one scale block), accumulators live in tensor
// memory (256 columns), the scale bytes of a K step (4 blocks = one 32-bit word per row) are written to tensor memory with
// tcgen05.st in the layout the MMA reads: row r -> lane r % 32 of every 32-lane sub-partition, column r / 32, byte = K block.
// MMA completion reaches the CTA through tcgen05.commit on an mbarrier per ring stage; every wait is bounded.
#include "common.cuh"
#include <cuda_bf16.h>

namespace {

constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4, THREADS = 256;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;     // 48 KB
constexpr int TMEM_COLS = 512;            // 256 accumulator columns + scale columns, rounded up to a power of two
constexpr int SFA_COL = 256, SFB_COL = 288;   // two buffers of 4 (A) / 8 (B) columns each
constexpr int SPIN = 1 << 22;

__device__ int g_mx_status = 0;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp16(uint32_t s, const void* g) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(g) : "memory"); }
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;      // core matrices adjacent in K
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;      // core matrices adjacent in M / N
  d |= (uint64_t)1 << 46;
  return d;
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < SPIN; i++) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  atomicExch(&g_mx_status, 1);
  return false;
}
// byte (r, k) of an R-row fp8 tile: core (r/8, k/16)
__device__ __forceinline__ uint32_t off8(int r, int k, int rows) { return (k >> 4) * (rows * 16) + (r >> 3) * 128 + (r & 7) * 16 + (k & 15); }

__global__ void __launch_bounds__(THREADS) grouped_mxfp8_tc_kernel(const uint8_t* __restrict__ a_q, const uint8_t* __restrict__ a_e8,
                                                                   const uint8_t* __restrict__ b_q, const uint8_t* __restrict__ b_e8,
                                                                   const int32_t* __restrict__ off, int n_experts, int n, int k,
                                                                   __nv_bfloat16* __restrict__ c) {
  extern __shared__ __align__(128) unsigned char sm[];
  __shared__ __align__(8) uint64_t bars[STAGES];
  __shared__ uint32_t tmem_base;
  __shared__ int s_expert;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (tid == 0) {
    int e = -1;
    for (int i = 0; i < n_experts; i++) if (m0 >= off[i] && m0 < off[i + 1]) { e = i; break; }
    s_expert = e;
    for (int s = 0; s < STAGES; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bars[s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int expert = s_expert;
  if (expert < 0) return;                          // tile past the last group (before any tensor memory is taken)
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t taddr = tmem_base;
  const int kb_total = k >> 5, ktiles = k / BK;
  const uint8_t* bq = b_q + (size_t)expert * n * k;
  const uint8_t* be = b_e8 + (size_t)expert * n * kb_total;
  const uint32_t sm0 = s32(sm);

  auto load_stage = [&](int slot, int kt) {
    const uint32_t sA = sm0 + slot * STAGE_BYTES, sB = sA + A_BYTES;
    for (int i = tid; i < BM * (BK / 16); i += THREADS) {
      const int r = i >> 3, kc = (i & 7) * 16;
      cp16(sA + off8(r, kc, BM), a_q + (size_t)(m0 + r) * k + kt * BK + kc);
    }
    for (int i = tid; i < BN * (BK / 16); i += THREADS) {
      const int r = i >> 3, kc = (i & 7) * 16;
      cp16(sB + off8(r, kc, BN), bq + (size_t)(n0 + r) * k + kt * BK + kc);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // scale words of a K step for the rows this lane serves: A rows lane + 32 j (j < 4), B rows lane + 32 j (j < 8)
  auto load_scales = [&](int kt, uint32_t (&wa)[4], uint32_t (&wb)[8]) {
#pragma unroll
    for (int j = 0; j < 4; j++) wa[j] = *reinterpret_cast<const uint32_t*>(a_e8 + (size_t)(m0 + lane + 32 * j) * kb_total + kt * 4);
#pragma unroll
    for (int j = 0; j < 8; j++) wb[j] = *reinterpret_cast<const uint32_t*>(be + (size_t)(n0 + lane + 32 * j) * kb_total + kt * 4);
  };

  for (int s = 0; s < STAGES - 1; s++) { if (s < ktiles) load_stage(s, s); else asm volatile("cp.async.commit_group;" ::: "memory"); }
  uint32_t wa[4], wb[8];
  load_scales(0, wa, wb);
  bool ok = true;
  for (int kt = 0; kt < ktiles && ok; kt++) {
    const int slot = kt % STAGES, sfbuf = kt & 1;
    // the scale buffer written now was last read by the MMAs of step kt-2: they must be done
    if (kt >= 2 && !wait_bar(s32(&bars[(kt - 2) % STAGES]), ((kt - 2) / STAGES) & 1)) { ok = false; break; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp < 4) {     // one writer per 32-lane sub-partition: every sub-partition holds the full table
      const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
      asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};"
                   ::"r"(taddr + lane_base + SFA_COL + sfbuf * 4), "r"(wa[0]), "r"(wa[1]), "r"(wa[2]), "r"(wa[3]) : "memory");
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                   ::"r"(taddr + lane_base + SFB_COL + sfbuf * 8), "r"(wb[0]), "r"(wb[1]), "r"(wb[2]), "r"(wb[3]), "r"(wb[4]), "r"(wb[5]), "r"(wb[6]),
                     "r"(wb[7]) : "memory");
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    if (kt + 1 < ktiles) load_scales(kt + 1, wa, wb);
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");     // this thread's copies of stage kt have landed
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sA = sm0 + slot * STAGE_BYTES, sB = sA + A_BYTES;
#pragma unroll
      for (int kb = 0; kb < 4; kb++) {
        const uint64_t da = make_desc(sA + kb * 2 * (BM * 16), BM * 16, 128), db = make_desc(sB + kb * 2 * (BN * 16), BN * 16, 128);
        // block-scaled instruction descriptor: B scale id [4,6), E4M3 x E4M3, N>>3 [17,23), E8M0 scales (bit 23), M>>7 [27,29), A scale id [29,31)
        const uint32_t idesc = ((uint32_t)kb << 4) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) | ((uint32_t)(BM >> 7) << 27) | ((uint32_t)kb << 29);
        const uint32_t acc = (kt > 0 || kb > 0) ? 1u : 0u;
        asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %6, 0;\n"
                     "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}"
                     ::"r"(taddr), "l"(da), "l"(db), "r"(idesc), "r"(taddr + SFA_COL + sfbuf * 4), "r"(taddr + SFB_COL + sfbuf * 8), "r"(acc) : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&bars[slot])) : "memory");
    }
    // refill the slot of step kt-1 with step kt+STAGES-1 once its MMAs have read it
    const int nk = kt + STAGES - 1;
    if (nk < ktiles) {
      if (kt >= 1 && !wait_bar(s32(&bars[(kt - 1) % STAGES]), ((kt - 1) / STAGES) & 1)) { ok = false; break; }
      load_stage(nk % STAGES, nk);
    } else {
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (ok) ok = wait_bar(s32(&bars[(ktiles - 1) % STAGES]), ((ktiles - 1) / STAGES) & 1);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok) {
    // accumulator row r = TMEM lane r; warps w and w+4 share a sub-partition and split the 256 columns
    const int row = m0 + (warp & 3) * 32 + lane;
    const int cbase = (warp >> 2) * (BN / 2);
#pragma unroll 1
    for (int j0 = 0; j0 < BN / 2; j0 += 32) {
      uint32_t v[32];
      const uint32_t ta = taddr + ((uint32_t)((warp & 3) * 32) << 16) + cbase + j0;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                     "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                     "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                     "=r"(v[31])
                   : "r"(ta));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      __nv_bfloat16* out = c + (size_t)row * n + n0 + cbase + j0;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 pk;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int q = 0; q < 4; q++) h[q] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * q]), __uint_as_float(v[j + 2 * q + 1]));
        *reinterpret_cast<uint4*>(out + j) = pk;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(TMEM_COLS) : "memory");
}

}  // namespace

extern "C" int b200q_mx_status_read_clear(int* status) {
  if (!status) return B200Q_ERR_BAD_ARG;
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_mx_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_mx_status, &zero, sizeof(int)));
  return B200Q_OK;
}

extern "C" int b200q_grouped_mxfp8_gemm(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                                        int m_total, int n, int k, void* c_bf16, void* stream) {
  if (!a_q || !a_e8 || !b_q || !b_e8 || !off || !c_bf16 || n_experts <= 0 || m_total <= 0 || n <= 0 || k <= 0) return B200Q_ERR_BAD_ARG;
  if (m_total % 256 || n % BN || k % BK) return B200Q_ERR_BAD_SHAPE;       // the reference asks M % 256 == N % 256 == K % 128 == 0 (moe_gemm.py:120)
  if (((uintptr_t)a_q | (uintptr_t)b_q | (uintptr_t)c_bf16) & 15 || ((uintptr_t)a_e8 | (uintptr_t)b_e8) & 3) return B200Q_ERR_MISALIGNED;
  static bool attr = false;
  if (!attr) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(grouped_mxfp8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STAGES * STAGE_BYTES));
    attr = true;
  }
  dim3 grid(n / BN, m_total / BM);
  grouped_mxfp8_tc_kernel<<<grid, THREADS, STAGES * STAGE_BYTES, (cudaStream_t)stream>>>(
      (const uint8_t*)a_q, (const uint8_t*)a_e8, (const uint8_t*)b_q, (const uint8_t*)b_e8, off, n_experts, n, k, (__nv_bfloat16*)c_bf16);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
