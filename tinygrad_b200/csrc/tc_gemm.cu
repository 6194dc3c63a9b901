// Prefill / batched linear on the 5th-generation tensor cores:  C[M, N] (fp32) = A[M, K] (fp16) x W[N, K]^T,
// W either fp16 or GGUF Q4_0 / Q8_0 blocks in the packed tile layout (dequantised to fp16 on the way into shared memory).
// Replaces `Linear.__call__` for T > 1 (tinygrad/nn/__init__.py:177; prefill chunks of tinygrad/llm/model.py:464-481).
//
// One CTA computes a 128 x BN tile: operands are staged in shared memory in the canonical K-major, no-swizzle layout
// (8 x 16-byte core matrices), one elected thread issues tcgen05.mma (kind::f16, fp32 accumulation) into tensor memory,
// completion is signalled through tcgen05.commit to an mbarrier, and the accumulator is read back with tcgen05.ld.
// Every mbarrier wait is bounded (status word on expiry); TMEM is always released before the CTA returns.
#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64;      // tile; BK = 4 MMAs of K = 16
constexpr int GEMM_THREADS = 128;
constexpr int SPIN = 1 << 22;

__device__ int g_tc_status = 0;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor, K-major, no swizzle: core matrix = 8 rows x 16 bytes, stored as 128 contiguous bytes;
// LBO = byte distance between core matrices adjacent in K, SBO = between core matrices adjacent in M/N.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
  return d;                                     // base offset 0, layout type 0 (no swizzle)
}
// instruction descriptor, kind::f16: fp16 x fp16 -> fp32, both operands K-major
__device__ __forceinline__ uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < SPIN; i++) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  atomicExch(&g_tc_status, 1);
  return false;
}

// element (r, k) of an R-row tile: core (r/8, k/8) at (k/8) * (R*16) + (r/8) * 128, inside the core (r%8)*16 + (k%8)*2 bytes
__device__ __forceinline__ uint32_t tile_off(int r, int k, int rows) { return (k >> 3) * (rows * 16) + (r >> 3) * 128 + (r & 7) * 16 + (k & 7) * 2; }

__global__ void __launch_bounds__(GEMM_THREADS) tc_gemm_f16_kernel(const __half* __restrict__ a, const __half* __restrict__ w, float* __restrict__ c,
                                                                    int m, int n, int k) {
  __shared__ __align__(128) unsigned char sA[BM * BK * 2];
  __shared__ __align__(128) unsigned char sB[BN * BK * 2];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_base)), "r"(BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t taddr = tmem_base;
  const uint32_t idesc = make_idesc(BM, BN);
  bool ok = true;
  uint32_t phase = 0;
  for (int k0 = 0; k0 < k; k0 += BK) {
    // stage A (BM x BK) and W (BN x BK), 16 bytes (8 halfs) per thread per step; rows past the edge are zero
    for (int i = tid; i < BM * (BK / 8); i += GEMM_THREADS) {
      const int r = i / (BK / 8), kc = (i % (BK / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m0 + r < m) v = *reinterpret_cast<const uint4*>(a + (size_t)(m0 + r) * k + k0 + kc);
      *reinterpret_cast<uint4*>(sA + tile_off(r, kc, BM)) = v;
    }
    for (int i = tid; i < BN * (BK / 8); i += GEMM_THREADS) {
      const int r = i / (BK / 8), kc = (i % (BK / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (n0 + r < n) v = *reinterpret_cast<const uint4*>(w + (size_t)(n0 + r) * k + k0 + kc);
      *reinterpret_cast<uint4*>(sB + tile_off(r, kc, BN)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic-proxy writes -> visible to the tensor core's reads
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int kk = 0; kk < BK / 16; kk++) {
        const uint64_t da = make_desc(s32(sA) + kk * 2 * (BM * 16), BM * 16, 128);
        const uint64_t db = make_desc(s32(sB) + kk * 2 * (BN * 16), BN * 16, 128);
        const uint32_t acc = (k0 > 0 || kk > 0) ? 1u : 0u;
        asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                     ::"r"(taddr), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&bar)) : "memory");
    }
    // the MMAs read shared memory asynchronously: wait for them before the next tile overwrites it
    if (!wait_bar(s32(&bar), phase)) { ok = false; break; }
    phase ^= 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  if (ok) {
    // accumulator: row r of the tile = TMEM lane r, column j = TMEM column j; warp w reads its 32 lanes
    const int row = m0 + warp * 32 + (tid & 31);
#pragma unroll 1
    for (int j0 = 0; j0 < BN; j0 += 32) {
      uint32_t v[32];
      const uint32_t ta = taddr + ((uint32_t)(warp * 32) << 16) + j0;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                     "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                     "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                     "=r"(v[31])
                   : "r"(ta));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (row < m) {
#pragma unroll
        for (int j = 0; j < 32; j++) if (n0 + j0 + j < n) c[(size_t)row * n + n0 + j0 + j] = __uint_as_float(v[j]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(BN) : "memory");
}

}  // namespace

extern "C" int b200q_tc_status_read_clear(int* status) {
  if (!status) return B200Q_ERR_BAD_ARG;
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_tc_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
  return B200Q_OK;
}

extern "C" int b200q_gemm_f16(const void* a_f16, const void* w_f16, float* c, int m, int n, int k, void* stream) {
  if (!a_f16 || !w_f16 || !c || m <= 0 || n <= 0 || k <= 0) return B200Q_ERR_BAD_ARG;
  if (k % BK) return B200Q_ERR_BAD_SHAPE;
  if (((uintptr_t)a_f16 | (uintptr_t)w_f16) & 15) return B200Q_ERR_MISALIGNED;
  dim3 grid(ceil_div(n, BN), ceil_div(m, BM));
  tc_gemm_f16_kernel<<<grid, GEMM_THREADS, 0, (cudaStream_t)stream>>>((const __half*)a_f16, (const __half*)w_f16, c, m, n, k);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
