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
constexpr int QGEMM_THREADS = 512;      // the dequant GEMM stages with 16 warps: unpacking the weights is its ALU-heavy part
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

// ---------------------------------------------------------------------------------------------------------------
// Quantised weights: W arrives as packed Q4_0 / Q8_0 tiles (include/b200q.h) and is dequantised to fp16 on its way into
// shared memory: (q - 8) * d or q * d as one fp16 multiply of two exactly representable factors, i.e. the same value as
// the reference's materialised fp16 weight (tinygrad/llm/gguf.py:46,56 then .cast('float16'), tinygrad/llm/model.py:376).
// K order inside every 8-element core is [0,2,1,3,4,6,5,7] for both operands (that is how the nibble / byte unpack
// delivers pairs); a contraction does not care as long as A and W agree.
constexpr int QBK = 128;                          // one packed column group per K step
constexpr int QGEMM_SMEM = 2 * (BM + BN) * QBK * 2;     // activations and weights, each as a high and a low fp16 half: 128 KB

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) { uint32_t d; asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) { uint32_t d; asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t h2fma(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { uint32_t d; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel)); return d; }

// q * d for four pairs: the fp16 product (hi, = the reference's materialised fp16 weight) and its exact remainder
// lo = q * d - hi (one fused multiply-add: the remainder has at most 8 significant bits, so it is exact).  hi + lo is the
// fp32 value the reference's fused kernels use when the activations are fp32 (tinygrad/codegen/late/coalesce.py:100).
__device__ __forceinline__ uint4 hi_lo(const uint32_t (&r)[4], uint32_t d2, uint4& lo) {
  const uint4 hi = make_uint4(h2mul(r[0], d2), h2mul(r[1], d2), h2mul(r[2], d2), h2mul(r[3], d2));
  lo = make_uint4(h2fma(r[0], d2, hi.x ^ 0x80008000u), h2fma(r[1], d2, hi.y ^ 0x80008000u), h2fma(r[2], d2, hi.z ^ 0x80008000u),
                  h2fma(r[3], d2, hi.w ^ 0x80008000u));
  return hi;
}
// 8 nibbles of two words (bytes 0..7 of a 16-byte half) -> one core row of 8 fp16 weights, low (HI = false) or high nibbles
template <bool HI>
__device__ __forceinline__ uint4 q4_core(uint32_t wa, uint32_t wb, uint32_t d2, uint4& lo) {
  const uint32_t MAGIC = 0x64006400u;
  uint32_t r[4];
  const uint32_t w[2] = {wa, wb};
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const uint32_t v = w[i] >> 8;
    if (!HI) {   // (1024 + n) - 1032 = n - 8
      r[2 * i] = h2sub(lop3_and_or(w[i], 0x000F000Fu, MAGIC), 0x64086408u);
      r[2 * i + 1] = h2sub(lop3_and_or(v, 0x000F000Fu, MAGIC), 0x64086408u);
    } else {     // (1024 + 16 n) / 16 - 72 = n - 8
      r[2 * i] = h2fma(lop3_and_or(w[i], 0x00F000F0u, MAGIC), 0x2C002C00u, 0xD480D480u);
      r[2 * i + 1] = h2fma(lop3_and_or(v, 0x00F000F0u, MAGIC), 0x2C002C00u, 0xD480D480u);
    }
  }
  return hi_lo(r, d2, lo);
}
// 8 int8 of two words -> one core row of 8 fp16 weights
__device__ __forceinline__ uint4 q8_core(uint32_t wa, uint32_t wb, uint32_t d2, uint4& lo) {
  const uint32_t HIB = 0x64646464u, SUB = 0x64806480u;     // 0x64bb = 1024 + (b ^ 0x80) = 1152 + b
  const uint32_t xa = wa ^ 0x80808080u, xb = wb ^ 0x80808080u;
  const uint32_t r[4] = {h2sub(prmt(xa, HIB, 0x4240u), SUB), h2sub(prmt(xa, HIB, 0x4341u), SUB), h2sub(prmt(xb, HIB, 0x4240u), SUB),
                         h2sub(prmt(xb, HIB, 0x4341u), SUB)};
  return hi_lo(r, d2, lo);
}

struct QGemmParams {
  const uint8_t* w; const void* x; const __half* bias; const void* residual; void* y;
  int m, n_out, n_in, kgroups, n_row_tiles, x_f16, y_f16, silu_mul;
};

template <int QT>
__global__ void __launch_bounds__(QGEMM_THREADS) tc_qgemm_kernel(const QGemmParams p) {
  extern __shared__ __align__(128) unsigned char qsm[];
  unsigned char* sA = qsm;
  unsigned char* sB = qsm + BM * QBK * 2;
  // fp32 activations: x = hi + lo and w = hi + lo (all fp16), y = xh wh + xl wh + xh wl: what the reference's fused fp32 kernels
  // compute (fp32 x times the unrounded dequantised weight) to about 2^-22.  fp16 activations: hi halves only (fp16-rounded weight).
  unsigned char* sA2 = sB + BN * QBK * 2;
  unsigned char* sB2 = sA2 + BM * QBK * 2;
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base;
  constexpr int TB = tile_bytes(QT);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int m0 = blockIdx.y * BM, rt0 = blockIdx.x * (BN / 16);
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_base)), "r"(BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < QGEMM_SMEM / 16; i += QGEMM_THREADS) reinterpret_cast<uint4*>(qsm)[i] = make_uint4(0, 0, 0, 0);   // rows past m / n stay zero
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t taddr = tmem_base;
  const uint32_t idesc = make_idesc(BM, BN);
  const int m_valid = min(BM, p.m - m0);
  bool ok = true;
  uint32_t phase = 0;
  // Software pipeline over the K groups: the global loads of group kg+1 (activations and packed weights, into registers) are
  // issued right after the MMAs of group kg and complete while the tensor core works; conversion + shared-memory stores follow
  // the wait for those MMAs (the operand tiles are single-buffered: 128 KB of fp16 hi / lo halves).
  constexpr int A_ITEMS = BM * (QBK / 8) / QGEMM_THREADS;          // 8-element activation chunks per thread (4)
  static_assert(BM * (QBK / 8) % QGEMM_THREADS == 0 && (BN / 16) * 64 == QGEMM_THREADS, "one weight (row, block) pair per thread");
  float4 xa[A_ITEMS][2];                                            // fp32: 8 values; fp16: the 16 raw bytes in xa[.][0]
  uint4 wq0 = make_uint4(0, 0, 0, 0), wq1 = make_uint4(0, 0, 0, 0);
  uint32_t wd2 = 0;
  const int w_tl = tid >> 6, w_h = (tid >> 5) & 1, w_l = tid & 31, w_g = w_l >> 2, w_t = w_l & 3;
  const bool w_on = rt0 + w_tl < p.n_row_tiles;
  auto load_regs = [&](int kg) {
#pragma unroll
    for (int j = 0; j < A_ITEMS; j++) {
      const int i = tid + j * QGEMM_THREADS, r = i / (QBK / 8), k = kg * QBK + (i % (QBK / 8)) * 8;
      xa[j][0] = xa[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < m_valid && k < p.n_in) {
        if (p.x_f16) xa[j][0] = *reinterpret_cast<const float4*>(reinterpret_cast<const __half*>(p.x) + (size_t)(m0 + r) * p.n_in + k);
        else {
          const float* src = reinterpret_cast<const float*>(p.x) + (size_t)(m0 + r) * p.n_in + k;
          xa[j][0] = *reinterpret_cast<const float4*>(src); xa[j][1] = *reinterpret_cast<const float4*>(src + 4);
        }
      }
    }
    if (w_on) {
      const uint8_t* tile = p.w + ((size_t)(rt0 + w_tl) * p.kgroups + kg) * TB;
      const unsigned short dbits = reinterpret_cast<const unsigned short*>(tile + (TB - 128))[(2 * w_g + (w_t >> 1)) * 4 + w_h * 2 + (w_t & 1)];
      wd2 = (uint32_t)dbits | ((uint32_t)dbits << 16);
      if (QT == B200Q_Q4_0) wq0 = ldg_stream(reinterpret_cast<const uint4*>(tile) + w_h * 32 + w_l);
      else { wq0 = ldg_stream(reinterpret_cast<const uint4*>(tile) + (2 * w_h) * 32 + w_l); wq1 = ldg_stream(reinterpret_cast<const uint4*>(tile) + (2 * w_h + 1) * 32 + w_l); }
    }
  };
  load_regs(0);
  for (int kg = 0; kg < p.kgroups; kg++) {
    // activations: rows m0 .. m0+m_valid, columns kg*128 .. +128, as fp16 in the cores' element order (rows past m stay zero)
#pragma unroll
    for (int j = 0; j < A_ITEMS; j++) {
      const int i = tid + j * QGEMM_THREADS, r = i / (QBK / 8), kc = (i % (QBK / 8)) * 8;
      if (r >= m_valid) continue;
      float f[8];
      if (p.x_f16) {
        const __half2* h = reinterpret_cast<const __half2*>(&xa[j][0]);
#pragma unroll
        for (int q = 0; q < 4; q++) { const float2 t2 = __half22float2(h[q]); f[2 * q] = t2.x; f[2 * q + 1] = t2.y; }
      } else {
        f[0] = xa[j][0].x; f[1] = xa[j][0].y; f[2] = xa[j][0].z; f[3] = xa[j][0].w; f[4] = xa[j][1].x; f[5] = xa[j][1].y; f[6] = xa[j][1].z; f[7] = xa[j][1].w;
      }
      __half2 o[4] = {__floats2half2_rn(f[0], f[2]), __floats2half2_rn(f[1], f[3]), __floats2half2_rn(f[4], f[6]), __floats2half2_rn(f[5], f[7])};
      *reinterpret_cast<uint4*>(sA + tile_off(r, kc, BM)) = *reinterpret_cast<const uint4*>(o);
      if (!p.x_f16) {
        const float2 h0 = __half22float2(o[0]), h1 = __half22float2(o[1]), h2 = __half22float2(o[2]), h3 = __half22float2(o[3]);
        __half2 lo2[4] = {__floats2half2_rn(f[0] - h0.x, f[2] - h0.y), __floats2half2_rn(f[1] - h1.x, f[3] - h1.y),
                          __floats2half2_rn(f[4] - h2.x, f[6] - h2.y), __floats2half2_rn(f[5] - h3.x, f[7] - h3.y)};
        *reinterpret_cast<uint4*>(sA2 + tile_off(r, kc, BM)) = *reinterpret_cast<const uint4*>(lo2);
      }
    }
    // weights: 8 packed tiles (16 rows x 4 blocks each); this thread's (row, block) pair
    if (w_on) {
      const int r = w_tl * 16 + w_h * 8 + w_g, t = w_t;
      const uint32_t d2 = wd2;
      uint4 lo[4];
      if (QT == B200Q_Q4_0) {
        // element e < 16 = low nibble of byte e, e >= 16 = high nibble of byte e - 16: cores 0,1 low, cores 2,3 high
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32, BN)) = q4_core<false>(wq0.x, wq0.y, d2, lo[0]);
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32 + 8, BN)) = q4_core<false>(wq0.z, wq0.w, d2, lo[1]);
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32 + 16, BN)) = q4_core<true>(wq0.x, wq0.y, d2, lo[2]);
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32 + 24, BN)) = q4_core<true>(wq0.z, wq0.w, d2, lo[3]);
      } else {
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32, BN)) = q8_core(wq0.x, wq0.y, d2, lo[0]);
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32 + 8, BN)) = q8_core(wq0.z, wq0.w, d2, lo[1]);
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32 + 16, BN)) = q8_core(wq1.x, wq1.y, d2, lo[2]);
        *reinterpret_cast<uint4*>(sB + tile_off(r, t * 32 + 24, BN)) = q8_core(wq1.z, wq1.w, d2, lo[3]);
      }
      if (!p.x_f16) {
#pragma unroll
        for (int c = 0; c < 4; c++) *reinterpret_cast<uint4*>(sB2 + tile_off(r, t * 32 + 8 * c, BN)) = lo[c];
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int kk = 0; kk < QBK / 16; kk++) {
        const uint64_t da = make_desc(s32(sA) + kk * 2 * (BM * 16), BM * 16, 128);
        const uint64_t db = make_desc(s32(sB) + kk * 2 * (BN * 16), BN * 16, 128);
        const uint32_t acc = (kg > 0 || kk > 0) ? 1u : 0u;
        asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                     ::"r"(taddr), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
        if (!p.x_f16) {
          const uint64_t da2 = make_desc(s32(sA2) + kk * 2 * (BM * 16), BM * 16, 128);
          const uint64_t db2 = make_desc(s32(sB2) + kk * 2 * (BN * 16), BN * 16, 128);
          asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                       ::"r"(taddr), "l"(da2), "l"(db), "r"(idesc), "r"(1u) : "memory");
          asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                       ::"r"(taddr), "l"(da), "l"(db2), "r"(idesc), "r"(1u) : "memory");
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&bar)) : "memory");
    }
    if (kg + 1 < p.kgroups) load_regs(kg + 1);
    // one thread polls the MMA-completion barrier, the others sleep in the block barrier (512 pollers cost issue slots); all
    // threads leave together if the wait ran out
    bool mma_done = true;
    if (tid == 0) mma_done = wait_bar(s32(&bar), phase);
    if (!__syncthreads_and(mma_done)) { ok = false; break; }
    phase ^= 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  if (ok) {
    // 16 warps: warp % 4 is its tensor-memory sub-partition (32 rows), warp / 4 its quarter of the 128 columns
    const int sub = warp & 3;
    const int row = m0 + sub * 32 + (tid & 31);
#pragma unroll 1
    for (int j0 = (warp >> 2) * 32; j0 < (warp >> 2) * 32 + 32; j0 += 32) {
      uint32_t v[32];
      const uint32_t ta = taddr + ((uint32_t)(sub * 32) << 16) + j0;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                     "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                     "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                     "=r"(v[31])
                   : "r"(ta));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (row < p.m && p.silu_mul) {
        // gate / up rows interleaved 8 + 8 per 16-row tile: 32 columns = 2 tiles -> 16 activations silu(gate) * up
#pragma unroll
        for (int t2 = 0; t2 < 2; t2++)
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int acol = (rt0 + j0 / 16 + t2) * 8 + j;
            if (acol < p.n_out / 2) {
              const float gte = __uint_as_float(v[t2 * 16 + j]), up = __uint_as_float(v[t2 * 16 + 8 + j]);
              const float o = (gte / (1.f + expf(-gte))) * up;
              if (p.y_f16) reinterpret_cast<__half*>(p.y)[(size_t)row * (p.n_out / 2) + acol] = __float2half_rn(o);
              else reinterpret_cast<float*>(p.y)[(size_t)row * (p.n_out / 2) + acol] = o;
            }
          }
      } else if (row < p.m) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
          const int col = rt0 * 16 + j0 + j;
          if (col < p.n_out) {
            float o = __uint_as_float(v[j]);
            if (p.bias) o += __half2float(p.bias[col]);
            const size_t at = (size_t)row * p.n_out + col;
            if (p.residual) o += p.y_f16 ? __half2float(reinterpret_cast<const __half*>(p.residual)[at]) : reinterpret_cast<const float*>(p.residual)[at];
            if (p.y_f16) reinterpret_cast<__half*>(p.y)[at] = __float2half_rn(o);
            else reinterpret_cast<float*>(p.y)[at] = o;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(BN) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// Few activation rows (batched decode, m <= 32): the weight-streaming shape.  Operands swap roles: the 128 weight rows of a
// tile are the MMA's M, the (up to 32) activation rows its N, so the tensor core does 128 x 32 x 16 per instruction instead of
// 128 x 128 x 16 on mostly zero rows; the K range is split over blockIdx.y so that layers with few row tiles still fill the GPU;
// the operand stage is 80 KB (weights hi / lo 64 KB + activations hi / lo 16 KB), double-buffered, so unpacking group kg+1 runs
// under the MMAs of group kg.  Every CTA writes its fp32 partial [split][act row][weight row] to a workspace; a second kernel
// sums the splits in a fixed order and applies bias / residual / SwiGLU (deterministic: no floating-point atomics).
constexpr int SK_N = 32;                                        // activation rows per MMA (N)
constexpr int SK_STAGE = 2 * (BN + SK_N) * QBK * 2;             // weights 128 rows + activations 32 rows, hi and lo: 80 KB
constexpr int SK_SMEM = 2 * SK_STAGE;
__host__ __device__ constexpr int sk_raw_stages(int qtype) { return qtype == B200Q_Q4_0 ? 6 : 3; }   // K groups of packed tiles in flight: 54 KB / 51 KB
__host__ __device__ constexpr int sk_smem_total(int qtype) { return SK_SMEM + sk_raw_stages(qtype) * (BN / 16) * tile_bytes(qtype); }

struct SkinnyParams {
  const uint8_t* w; const void* x; float* part;
  int m, n_out, n_in, kgroups, n_row_tiles, x_f16, groups_per_split;
};

template <int QT>
__global__ void __launch_bounds__(QGEMM_THREADS) tc_qgemm_skinny_kernel(const SkinnyParams p) {
  extern __shared__ __align__(128) unsigned char ssm[];
  __shared__ __align__(8) uint64_t bars[2], raw_full[8];
  __shared__ uint32_t tmem_base;
  constexpr int TB = tile_bytes(QT), RAW_STAGES = sk_raw_stages(QT), RAW_STAGE = (BN / 16) * TB;
  unsigned char* raw = ssm + SK_SMEM;                            // ring of packed weight tiles as they sit in HBM, filled by bulk copies
  const int tid = threadIdx.x, warp = tid >> 5;
  const int rt0 = blockIdx.x * (BN / 16), split = blockIdx.y;
  const int kg0 = split * p.groups_per_split, kg1 = min(p.kgroups, kg0 + p.groups_per_split);
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_base)), "r"(SK_N) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bars[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bars[1])));
    for (int i = 0; i < RAW_STAGES; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&raw_full[i])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < SK_SMEM / 16; i += QGEMM_THREADS) reinterpret_cast<uint4*>(ssm)[i] = make_uint4(0, 0, 0, 0);   // rows past m / n_out stay zero
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t taddr = tmem_base;
  const uint32_t idesc = make_idesc(BN, SK_N);                   // M = 128 weight rows, N = 32 activation rows
  // this thread's pieces: one (weight row, block) pair, and one 8-value chunk of the activations (32 rows x 16 chunks = 512)
  const int w_tl = tid >> 6, w_h = (tid >> 5) & 1, w_l = tid & 31, w_g = w_l >> 2, w_t = w_l & 3;
  const bool w_on = rt0 + w_tl < p.n_row_tiles;
  const int a_r = tid >> 4, a_kc = (tid & 15) * 8;
  float4 xa0, xa1;
  uint4 wq0 = make_uint4(0, 0, 0, 0), wq1 = make_uint4(0, 0, 0, 0);
  uint32_t wd2 = 0;
  auto load_regs = [&](int kg) {
    xa0 = xa1 = make_float4(0.f, 0.f, 0.f, 0.f);
    const int k = kg * QBK + a_kc;
    if (a_r < p.m && k < p.n_in) {
      if (p.x_f16) xa0 = *reinterpret_cast<const float4*>(reinterpret_cast<const __half*>(p.x) + (size_t)a_r * p.n_in + k);
      else {
        const float* src = reinterpret_cast<const float*>(p.x) + (size_t)a_r * p.n_in + k;
        xa0 = *reinterpret_cast<const float4*>(src); xa1 = *reinterpret_cast<const float4*>(src + 4);
      }
    }
  };
  // The weight stream: thread 0 keeps RAW_STAGES K groups of packed tiles in flight (one bulk copy per row tile, completion counted in
  // bytes on the slot's mbarrier), which is what hides the HBM latency; a slot is refilled right after the block-wide barrier that
  // follows its last read.
  const int n_tiles_here = min(BN / 16, p.n_row_tiles - rt0);
  auto issue_raw = [&](int it) {
    const int slot = it % RAW_STAGES, kg = kg0 + it;
    const uint32_t bar = s32(&raw_full[slot]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(n_tiles_here * TB)) : "memory");
    for (int tl = 0; tl < n_tiles_here; tl++)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(s32(raw + slot * RAW_STAGE + tl * TB)), "l"(p.w + ((size_t)(rt0 + tl) * p.kgroups + kg) * TB), "r"((uint32_t)TB), "r"(bar) : "memory");
  };
  bool ok = true;
  const int n_it = kg1 - kg0;
  if (tid == 0) for (int it = 0; it < RAW_STAGES && it < n_it; it++) issue_raw(it);
  if (kg0 < kg1) load_regs(kg0);
  for (int kg = kg0, it = 0; kg < kg1; kg++, it++) {
    const int st = it & 1;
    unsigned char* sW = ssm + st * SK_STAGE;                    // weights hi
    unsigned char* sW2 = sW + BN * QBK * 2;                     // weights lo
    unsigned char* sX = sW2 + BN * QBK * 2;                     // activations hi
    unsigned char* sX2 = sX + SK_N * QBK * 2;                   // activations lo
    // a wait that ran out makes the whole CTA leave at the block-wide barrier below (never a thread on its own)
    bool good = it < 2 || wait_bar(s32(&bars[st]), ((it >> 1) - 1) & 1);                          // the MMAs that read this stage are done
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    good = good && wait_bar(s32(&raw_full[it % RAW_STAGES]), (it / RAW_STAGES) & 1);                // this group's packed tiles have landed
    if (w_on && good) {
      const unsigned char* tile = raw + (it % RAW_STAGES) * RAW_STAGE + w_tl * TB;
      const unsigned short dbits = reinterpret_cast<const unsigned short*>(tile + (TB - 128))[(2 * w_g + (w_t >> 1)) * 4 + w_h * 2 + (w_t & 1)];
      wd2 = (uint32_t)dbits | ((uint32_t)dbits << 16);
      if (QT == B200Q_Q4_0) wq0 = reinterpret_cast<const uint4*>(tile)[w_h * 32 + w_l];
      else { wq0 = reinterpret_cast<const uint4*>(tile)[(2 * w_h) * 32 + w_l]; wq1 = reinterpret_cast<const uint4*>(tile)[(2 * w_h + 1) * 32 + w_l]; }
    }
    if (a_r < p.m && good) {
      float f[8];
      if (p.x_f16) {
        const __half2* h = reinterpret_cast<const __half2*>(&xa0);
#pragma unroll
        for (int q = 0; q < 4; q++) { const float2 t2 = __half22float2(h[q]); f[2 * q] = t2.x; f[2 * q + 1] = t2.y; }
      } else { f[0] = xa0.x; f[1] = xa0.y; f[2] = xa0.z; f[3] = xa0.w; f[4] = xa1.x; f[5] = xa1.y; f[6] = xa1.z; f[7] = xa1.w; }
      __half2 o[4] = {__floats2half2_rn(f[0], f[2]), __floats2half2_rn(f[1], f[3]), __floats2half2_rn(f[4], f[6]), __floats2half2_rn(f[5], f[7])};
      *reinterpret_cast<uint4*>(sX + tile_off(a_r, a_kc, SK_N)) = *reinterpret_cast<const uint4*>(o);
      if (!p.x_f16) {
        const float2 h0 = __half22float2(o[0]), h1 = __half22float2(o[1]), h2 = __half22float2(o[2]), h3 = __half22float2(o[3]);
        __half2 lo2[4] = {__floats2half2_rn(f[0] - h0.x, f[2] - h0.y), __floats2half2_rn(f[1] - h1.x, f[3] - h1.y),
                          __floats2half2_rn(f[4] - h2.x, f[6] - h2.y), __floats2half2_rn(f[5] - h3.x, f[7] - h3.y)};
        *reinterpret_cast<uint4*>(sX2 + tile_off(a_r, a_kc, SK_N)) = *reinterpret_cast<const uint4*>(lo2);
      }
    }
    if (w_on && good) {
      const int r = w_tl * 16 + w_h * 8 + w_g, t = w_t;
      uint4 lo[4];
      if (QT == B200Q_Q4_0) {
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32, BN)) = q4_core<false>(wq0.x, wq0.y, wd2, lo[0]);
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32 + 8, BN)) = q4_core<false>(wq0.z, wq0.w, wd2, lo[1]);
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32 + 16, BN)) = q4_core<true>(wq0.x, wq0.y, wd2, lo[2]);
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32 + 24, BN)) = q4_core<true>(wq0.z, wq0.w, wd2, lo[3]);
      } else {
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32, BN)) = q8_core(wq0.x, wq0.y, wd2, lo[0]);
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32 + 8, BN)) = q8_core(wq0.z, wq0.w, wd2, lo[1]);
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32 + 16, BN)) = q8_core(wq1.x, wq1.y, wd2, lo[2]);
        *reinterpret_cast<uint4*>(sW + tile_off(r, t * 32 + 24, BN)) = q8_core(wq1.z, wq1.w, wd2, lo[3]);
      }
      if (!p.x_f16) {
#pragma unroll
        for (int c = 0; c < 4; c++) *reinterpret_cast<uint4*>(sW2 + tile_off(r, t * 32 + 8 * c, BN)) = lo[c];
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (!__syncthreads_and(good)) {
      ok = false;
      if (tid == 0)        // bulk copies still in flight must land before the CTA gives up its shared memory
        for (int j = it; j < n_it && j < it + RAW_STAGES; j++) wait_bar(s32(&raw_full[j % RAW_STAGES]), (j / RAW_STAGES) & 1);
      break;
    }
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      // descriptors of K step kk = the stage's base descriptor + the step's byte offset >> 4 in the address field
      const uint64_t dw0 = make_desc(s32(sW), BN * 16, 128), dx0 = make_desc(s32(sX), SK_N * 16, 128);
      const uint64_t dwl0 = make_desc(s32(sW2), BN * 16, 128), dxl0 = make_desc(s32(sX2), SK_N * 16, 128);
      for (int kk = 0; kk < QBK / 16; kk++) {
        const uint64_t dw = dw0 + (uint64_t)((kk * 2 * (BN * 16)) >> 4), dx = dx0 + (uint64_t)((kk * 2 * (SK_N * 16)) >> 4);
        const uint32_t acc = (it > 0 || kk > 0) ? 1u : 0u;
        asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                     ::"r"(taddr), "l"(dw), "l"(dx), "r"(idesc), "r"(acc) : "memory");
        if (!p.x_f16) {
          const uint64_t dw2 = dwl0 + (uint64_t)((kk * 2 * (BN * 16)) >> 4), dx2 = dxl0 + (uint64_t)((kk * 2 * (SK_N * 16)) >> 4);
          asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                       ::"r"(taddr), "l"(dw), "l"(dx2), "r"(idesc), "r"(1u) : "memory");
          asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                       ::"r"(taddr), "l"(dw2), "l"(dx), "r"(idesc), "r"(1u) : "memory");
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&bars[st])) : "memory");
      if (it + RAW_STAGES < n_it) issue_raw(it + RAW_STAGES);     // every thread has read this slot (the barrier above)
    }
    if (kg + 1 < kg1) load_regs(kg + 1);
  }
  // the last commit covers every MMA issued before it
  if (n_it > 0) {     // also on the way out after a failed wait: MMAs that were issued must be done before tensor memory is freed
    const bool done = wait_bar(s32(&bars[(n_it - 1) & 1]), ((n_it - 1) >> 1) & 1);
    ok = ok && done;
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok && warp < 4) {
    // accumulator row = weight row (tensor-memory lane), column = activation row
    uint32_t v[32];
    const uint32_t ta = taddr + ((uint32_t)(warp * 32) << 16);
    if (n_it > 0) {
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                     "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                     "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                     "=r"(v[31])
                   : "r"(ta));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++) v[j] = 0u;
    }
    const int col = rt0 * 16 + tid;                              // weight row = output column of y
    if (col < p.n_out) {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (j < p.m) p.part[((size_t)split * p.m + j) * p.n_out + col] = __uint_as_float(v[j]);       // consecutive lanes: consecutive addresses
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(SK_N) : "memory");
}

// y = sum over splits (fixed order) + bias + residual, or the SwiGLU product of interleaved gate / up columns
__global__ void skinny_reduce_kernel(const float* __restrict__ part, int n_splits, int m, int n_out, const __half* __restrict__ bias,
                                     const void* __restrict__ residual, void* __restrict__ y, int y_f16, int silu_mul) {
  const int n_y = silu_mul ? n_out / 2 : n_out;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)m * n_y) return;
  const int row = (int)(i / n_y), c = (int)(i - (size_t)row * n_y);
  auto total = [&](int col) { float s = 0.f; for (int z = 0; z < n_splits; z++) s += part[((size_t)z * m + row) * n_out + col]; return s; };
  float o;
  if (silu_mul) {
    const int col = (c >> 3) * 16 + (c & 7);                     // 8 gate rows then 8 up rows per 16-row tile
    const float g = total(col), u = total(col + 8);
    o = (g / (1.f + expf(-g))) * u;
  } else {
    o = total(c);
    if (bias) o += __half2float(bias[c]);
    if (residual) o += y_f16 ? __half2float(reinterpret_cast<const __half*>(residual)[i]) : reinterpret_cast<const float*>(residual)[i];
  }
  if (y_f16) reinterpret_cast<__half*>(y)[i] = __float2half_rn(o); else reinterpret_cast<float*>(y)[i] = o;
}


// ---------------------------------------------------------------------------------------------------------------
// Pipelined dequant GEMM (prompt chunks).  The kernel above converts the same activation rows once per column tile and moves all its
// warps in lock-step through convert -> unpack -> barrier -> MMA -> wait.  Here the activations are split ONCE per GEMM into fp16
// hi / lo tiles laid out as the tensor core reads them (split_rows_kernel: per 128 rows x 128 columns one 32 KB tile per half, in a
// workspace), so a CTA brings its A operand in by bulk copies; a stage is 64 columns of K (A hi / lo 32 KB by bulk copy, W hi / lo
// 32 KB unpacked by the 512 threads, 16 weights each); the weight slots are double-buffered (the MMAs of a step run while the threads unpack
// the next one) and the activation copies run two steps ahead in a ring of four slots; weight words are fetched two steps ahead too.
constexpr int P_BK = 64, P_A_SLOTS = 4;               // K columns per step; activation slots (copies run two steps ahead); two weight slots
constexpr int P_HALF = BM * P_BK * 2;                 // 16 KB: one operand half (hi or lo) of a step
constexpr int P_SMEM = (P_A_SLOTS + 2) * 2 * P_HALF;  // 4 x (A hi, A lo) + 2 x (W hi, W lo) = 192 KB
constexpr int WS_TILE = BM * QBK * 2;                 // 32 KB: 128 rows x 128 columns of fp16 in core-matrix order

template <typename T>
__global__ void __launch_bounds__(QGEMM_THREADS) split_rows_kernel(const T* __restrict__ x, int m, int n_in, int kgroups, unsigned char* __restrict__ ws,
                                                                   int with_lo) {
  const int kg = blockIdx.x, mt = blockIdx.y, tid = threadIdx.x;
  unsigned char* hi = ws + ((size_t)(mt * kgroups + kg) * 2) * WS_TILE;
  unsigned char* lo = hi + WS_TILE;
#pragma unroll
  for (int j = 0; j < BM * (QBK / 8) / QGEMM_THREADS; j++) {
    const int i = tid + j * QGEMM_THREADS, r = i / (QBK / 8), kc = (i % (QBK / 8)) * 8, row = mt * BM + r, k = kg * QBK + kc;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (row < m && k < n_in) {
      if (sizeof(T) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(x) + (size_t)row * n_in + k);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int q = 0; q < 4; q++) { const float2 t2 = __half22float2(h[q]); f[2 * q] = t2.x; f[2 * q + 1] = t2.y; }
      } else {
        const float* src = reinterpret_cast<const float*>(x) + (size_t)row * n_in + k;
        const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
      }
    }
    // element order inside a core: [0,2,1,3,4,6,5,7], the order the weight unpack delivers
    __half2 o[4] = {__floats2half2_rn(f[0], f[2]), __floats2half2_rn(f[1], f[3]), __floats2half2_rn(f[4], f[6]), __floats2half2_rn(f[5], f[7])};
    *reinterpret_cast<uint4*>(hi + tile_off(r, kc, BM)) = *reinterpret_cast<const uint4*>(o);
    if (with_lo) {
      const float2 h0 = __half22float2(o[0]), h1 = __half22float2(o[1]), h2 = __half22float2(o[2]), h3 = __half22float2(o[3]);
      __half2 lo2[4] = {__floats2half2_rn(f[0] - h0.x, f[2] - h0.y), __floats2half2_rn(f[1] - h1.x, f[3] - h1.y),
                        __floats2half2_rn(f[4] - h2.x, f[6] - h2.y), __floats2half2_rn(f[5] - h3.x, f[7] - h3.y)};
      *reinterpret_cast<uint4*>(lo + tile_off(r, kc, BM)) = *reinterpret_cast<const uint4*>(lo2);
    }
  }
}

__device__ __forceinline__ void p_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int QT>
__global__ void __launch_bounds__(QGEMM_THREADS) tc_qgemm_pipe_kernel(const QGemmParams p, const unsigned char* __restrict__ ws) {
  extern __shared__ __align__(128) unsigned char psm[];
  __shared__ __align__(8) uint64_t full[P_A_SLOTS], empty[2], done;
  __shared__ uint32_t tmem_base;
  constexpr int TB = tile_bytes(QT);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int mt = blockIdx.y, m0 = mt * BM, rt0 = blockIdx.x * (BN / 16);
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_base)), "r"(BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int i = 0; i < P_A_SLOTS; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&full[i])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&empty[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&empty[1])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&done)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < P_SMEM / 16; i += QGEMM_THREADS) reinterpret_cast<uint4*>(psm)[i] = make_uint4(0, 0, 0, 0);   // weight rows past n_out stay zero
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t taddr = tmem_base;
  const uint32_t idesc = make_idesc(BM, BN);
  const int n_steps = 2 * p.kgroups;
  const uint32_t a_bytes = p.x_f16 ? P_HALF : 2 * P_HALF;
  unsigned char* const b_ring = psm + P_A_SLOTS * 2 * P_HALF;
  // this thread's 16 weights of a step: row r of the 128, block b of the step's two, half h of the block's 32 (8 quant bytes)
  const int r = tid >> 2, b = (tid >> 1) & 1, h = tid & 1;
  const int w_tl = r >> 4, h8 = (r >> 3) & 1, g = r & 7;
  const bool w_on = rt0 + w_tl < p.n_row_tiles;
  struct WRegs { uint2 q4; uint4 q8; uint32_t d2; };
  WRegs wa = {make_uint2(0, 0), make_uint4(0, 0, 0, 0), 0u}, wb = wa;      // weights of the step in hand and of the one after it
  auto load_regs = [&](int step, WRegs& w) {
    if (!w_on || step >= n_steps) return;
    const int t = (step & 1) * 2 + b;
    const uint8_t* tile = p.w + ((size_t)(rt0 + w_tl) * p.kgroups + (step >> 1)) * TB;
    const unsigned short dbits = reinterpret_cast<const unsigned short*>(tile + (TB - 128))[(2 * g + (t >> 1)) * 4 + h8 * 2 + (t & 1)];
    w.d2 = (uint32_t)dbits | ((uint32_t)dbits << 16);
    if (QT == B200Q_Q4_0) w.q4 = ldg_stream(reinterpret_cast<const uint2*>(tile) + (h8 * 32 + g * 4 + t) * 2 + h);
    else w.q8 = ldg_stream(reinterpret_cast<const uint4*>(tile) + (2 * h8 + h) * 32 + g * 4 + t);
  };
  auto issue_a = [&](int step) {       // thread 0: the activation halves of `step` into its slot of the A ring
    const int slot = step % P_A_SLOTS;
    const uint32_t fb = s32(&full[slot]), dst = s32(psm + slot * 2 * P_HALF);
    const unsigned char* src = ws + ((size_t)(mt * p.kgroups + (step >> 1)) * 2) * WS_TILE + (step & 1) * P_HALF;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(a_bytes) : "memory");
    p_bulk_g2s(dst, src, P_HALF, fb);
    if (!p.x_f16) p_bulk_g2s(dst + P_HALF, src + WS_TILE, P_HALF, fb);
  };
  bool ok = true;
  int a_issued = 0;                    // thread 0: highest step whose activation copy is out
  load_regs(0, wa); load_regs(1, wb);
  if (tid == 0) { issue_a(0); if (n_steps > 1) { issue_a(1); a_issued = 1; } }
  // One step: (1) the MMAs of step - 2 are done -> their W slot (this step's) and their A slot (step + 2's) are free; (2) thread 0 sends
  // for the activations of step + 2; (3) everybody unpacks this step's weights and asks for those of step + 2; (4) thread 0 issues the MMAs.
  auto do_step = [&](int step, WRegs& w) -> bool {
    if (step >= 2) {
      bool free_ok = true;
      if (tid == 0) free_ok = wait_bar(s32(&empty[step & 1]), ((step - 2) >> 1) & 1);
      if (!__syncthreads_and(free_ok)) return false;
    }
    if (tid == 0 && step + 2 < n_steps) { issue_a(step + 2); a_issued = step + 2; }
    unsigned char* sBh = b_ring + (step & 1) * 2 * P_HALF;
    unsigned char* sBl = sBh + P_HALF;
    if (w_on) {
      uint4 lo0, lo1, c0, c1;
      int k0, k1;
      if (QT == B200Q_Q4_0) {      // low nibbles: elements 8h .. 8h+7, high nibbles: 16 + 8h ..
        c0 = q4_core<false>(w.q4.x, w.q4.y, w.d2, lo0); c1 = q4_core<true>(w.q4.x, w.q4.y, w.d2, lo1);
        k0 = b * 32 + 8 * h; k1 = k0 + 16;
      } else {                     // bytes 16h .. 16h+15
        c0 = q8_core(w.q8.x, w.q8.y, w.d2, lo0); c1 = q8_core(w.q8.z, w.q8.w, w.d2, lo1);
        k0 = b * 32 + 16 * h; k1 = k0 + 8;
      }
      *reinterpret_cast<uint4*>(sBh + tile_off(r, k0, BN)) = c0;
      *reinterpret_cast<uint4*>(sBh + tile_off(r, k1, BN)) = c1;
      if (!p.x_f16) {
        *reinterpret_cast<uint4*>(sBl + tile_off(r, k0, BN)) = lo0;
        *reinterpret_cast<uint4*>(sBl + tile_off(r, k1, BN)) = lo1;
      }
    }
    load_regs(step + 2, w);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      const int slot = step % P_A_SLOTS;
      if (wait_bar(s32(&full[slot]), (step / P_A_SLOTS) & 1)) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sA = s32(psm + slot * 2 * P_HALF), sA2 = sA + P_HALF, sB = s32(sBh), sB2 = sB + P_HALF;
#pragma unroll
        for (int kk = 0; kk < P_BK / 16; kk++) {
          const uint64_t da = make_desc(sA + kk * 2 * (BM * 16), BM * 16, 128), db = make_desc(sB + kk * 2 * (BN * 16), BN * 16, 128);
          const uint32_t acc = (step > 0 || kk > 0) ? 1u : 0u;
          asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                       ::"r"(taddr), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
          if (!p.x_f16) {
            const uint64_t da2 = make_desc(sA2 + kk * 2 * (BM * 16), BM * 16, 128), db2 = make_desc(sB2 + kk * 2 * (BN * 16), BN * 16, 128);
            asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                         ::"r"(taddr), "l"(da2), "l"(db), "r"(idesc), "r"(1u) : "memory");
            asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                         ::"r"(taddr), "l"(da), "l"(db2), "r"(idesc), "r"(1u) : "memory");
          }
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&empty[step & 1])) : "memory");
        if (step == n_steps - 1) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&done)) : "memory");
      }
    }
    return true;
  };
  for (int step = 0; step < n_steps && ok; step += 2) {      // n_steps is even: two steps per K group
    ok = do_step(step, wa);
    if (ok) ok = do_step(step + 1, wb);
  }
  // all MMAs done (or a wait ran out: then every copy and MMA issued so far is drained before the tensor memory goes back)
  bool fin = true;
  if (tid == 0) {
    if (ok) fin = wait_bar(s32(&done), 0);       // the last step's copies were waited for before its MMAs were issued
    if (!ok) {      // left the loop early: drain the MMAs issued so far and the (at most two) activation copies still in flight
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&done)) : "memory");
      wait_bar(s32(&done), 0);
      for (int st = max(0, a_issued - 2); st <= a_issued; st++) wait_bar(s32(&full[st % P_A_SLOTS]), (st / P_A_SLOTS) & 1);
    }
  }
  ok = __syncthreads_and(ok && fin);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok) {
    const int sub = warp & 3;
    const int row = m0 + sub * 32 + (tid & 31);
    const int j0 = (warp >> 2) * 32;
    uint32_t v[32];
    const uint32_t ta = taddr + ((uint32_t)(sub * 32) << 16) + j0;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                   "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                   "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                   "=r"(v[31])
                 : "r"(ta));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (row < p.m && p.silu_mul) {
#pragma unroll
      for (int t2 = 0; t2 < 2; t2++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int acol = (rt0 + j0 / 16 + t2) * 8 + j;
          if (acol < p.n_out / 2) {
            const float gte = __uint_as_float(v[t2 * 16 + j]), up = __uint_as_float(v[t2 * 16 + 8 + j]);
            const float o = (gte / (1.f + expf(-gte))) * up;
            if (p.y_f16) reinterpret_cast<__half*>(p.y)[(size_t)row * (p.n_out / 2) + acol] = __float2half_rn(o);
            else reinterpret_cast<float*>(p.y)[(size_t)row * (p.n_out / 2) + acol] = o;
          }
        }
    } else if (row < p.m) {
#pragma unroll
      for (int j = 0; j < 32; j++) {
        const int col = rt0 * 16 + j0 + j;
        if (col < p.n_out) {
          float o = __uint_as_float(v[j]);
          if (p.bias) o += __half2float(p.bias[col]);
          const size_t at = (size_t)row * p.n_out + col;
          if (p.residual) o += p.y_f16 ? __half2float(reinterpret_cast<const __half*>(p.residual)[at]) : reinterpret_cast<const float*>(p.residual)[at];
          if (p.y_f16) reinterpret_cast<__half*>(p.y)[at] = __float2half_rn(o);
          else reinterpret_cast<float*>(p.y)[at] = o;
        }
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

extern "C" int b200q_qgemm(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue,
                           void* y, int y_dtype, int m, int n_out, int n_in, void* stream) {
  if (!w_packed || !x || !y || m <= 0 || n_out <= 0 || n_in <= 0) return B200Q_ERR_BAD_ARG;
  if (epilogue != B200Q_EPI_LINEAR && epilogue != B200Q_EPI_SILU_MUL) return B200Q_ERR_BAD_ARG;
  if (epilogue == B200Q_EPI_SILU_MUL && (bias_f16 || residual || n_out % 16)) return B200Q_ERR_BAD_ARG;
  if (qtype == B200Q_Q6_K) return B200Q_ERR_UNSUPPORTED;
  if (qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0) return B200Q_ERR_BAD_ARG;
  if ((x_dtype != B200Q_F32 && x_dtype != B200Q_F16) || (y_dtype != B200Q_F32 && y_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (n_in % 32) return B200Q_ERR_BAD_SHAPE;
  if (((uintptr_t)w_packed | (uintptr_t)x) & 15) return B200Q_ERR_MISALIGNED;
  QGemmParams p;
  p.w = (const uint8_t*)w_packed; p.x = x; p.bias = (const __half*)bias_f16; p.residual = residual; p.y = y;
  p.silu_mul = epilogue == B200Q_EPI_SILU_MUL;
  p.m = m; p.n_out = n_out; p.n_in = n_in; p.kgroups = ceil_div(n_in, GROUP_ELEMS); p.n_row_tiles = ceil_div(n_out, TILE_ROWS);
  p.x_f16 = x_dtype == B200Q_F16; p.y_f16 = y_dtype == B200Q_F16;
  dim3 grid(ceil_div(p.n_row_tiles, BN / 16), ceil_div(m, BM));
  static PerDeviceFlag attr;
  const int dev = b200q_current_device();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!attr.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(tc_qgemm_kernel<B200Q_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, QGEMM_SMEM));
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(tc_qgemm_kernel<B200Q_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, QGEMM_SMEM));
    attr.set(dev);
  }
  if (qtype == B200Q_Q4_0) tc_qgemm_kernel<B200Q_Q4_0><<<grid, QGEMM_THREADS, QGEMM_SMEM, (cudaStream_t)stream>>>(p);
  else tc_qgemm_kernel<B200Q_Q8_0><<<grid, QGEMM_THREADS, QGEMM_SMEM, (cudaStream_t)stream>>>(p);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" size_t b200q_qgemm_workspace_bytes(int m, int n_in) {
  if (m <= 0 || n_in <= 0) return 0;
  return (size_t)ceil_div(m, BM) * ceil_div(n_in, GROUP_ELEMS) * 2 * WS_TILE;
}

extern "C" int b200q_qgemm_ws(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue,
                              void* y, int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes, void* stream) {
  if (!w_packed || !x || !y || !workspace || m <= 0 || n_out <= 0 || n_in <= 0) return B200Q_ERR_BAD_ARG;
  if (epilogue != B200Q_EPI_LINEAR && epilogue != B200Q_EPI_SILU_MUL) return B200Q_ERR_BAD_ARG;
  if (epilogue == B200Q_EPI_SILU_MUL && (bias_f16 || residual || n_out % 16)) return B200Q_ERR_BAD_ARG;
  if (qtype == B200Q_Q6_K) return B200Q_ERR_UNSUPPORTED;
  if (qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0) return B200Q_ERR_BAD_ARG;
  if ((x_dtype != B200Q_F32 && x_dtype != B200Q_F16) || (y_dtype != B200Q_F32 && y_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (n_in % 32) return B200Q_ERR_BAD_SHAPE;
  if (((uintptr_t)w_packed | (uintptr_t)x | (uintptr_t)workspace) & 15) return B200Q_ERR_MISALIGNED;
  if (workspace_bytes < b200q_qgemm_workspace_bytes(m, n_in)) return B200Q_ERR_TOO_LARGE;
  QGemmParams p;
  p.w = (const uint8_t*)w_packed; p.x = x; p.bias = (const __half*)bias_f16; p.residual = residual; p.y = y;
  p.silu_mul = epilogue == B200Q_EPI_SILU_MUL;
  p.m = m; p.n_out = n_out; p.n_in = n_in; p.kgroups = ceil_div(n_in, GROUP_ELEMS); p.n_row_tiles = ceil_div(n_out, TILE_ROWS);
  p.x_f16 = x_dtype == B200Q_F16; p.y_f16 = y_dtype == B200Q_F16;
  static PerDeviceFlag attr;
  const int dev = b200q_current_device();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!attr.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(tc_qgemm_pipe_kernel<B200Q_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(tc_qgemm_pipe_kernel<B200Q_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM));
    attr.set(dev);
  }
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 sgrid(p.kgroups, ceil_div(m, BM));
  if (p.x_f16) split_rows_kernel<__half><<<sgrid, QGEMM_THREADS, 0, st>>>((const __half*)x, m, n_in, p.kgroups, (unsigned char*)workspace, 0);
  else split_rows_kernel<float><<<sgrid, QGEMM_THREADS, 0, st>>>((const float*)x, m, n_in, p.kgroups, (unsigned char*)workspace, 1);
  const dim3 grid(ceil_div(p.n_row_tiles, BN / 16), ceil_div(m, BM));
  if (qtype == B200Q_Q4_0) tc_qgemm_pipe_kernel<B200Q_Q4_0><<<grid, QGEMM_THREADS, P_SMEM, st>>>(p, (const unsigned char*)workspace);
  else tc_qgemm_pipe_kernel<B200Q_Q8_0><<<grid, QGEMM_THREADS, P_SMEM, st>>>(p, (const unsigned char*)workspace);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

static int skinny_splits(int n_row_tiles, int kgroups, int n_sm) {
  const int tiles = ceil_div(n_row_tiles, BN / 16);
  int splits = ceil_div(2 * n_sm, tiles);                         // about two CTAs per SM over the whole launch
  const int max_splits = kgroups / 4 > 0 ? kgroups / 4 : 1;       // at least 4 K groups per CTA
  if (splits > max_splits) splits = max_splits;
  return splits < 1 ? 1 : splits;
}

static int sm_count_cached() { return b200q_sm_count(); }

extern "C" size_t b200q_qgemm_skinny_workspace_bytes(int m, int n_out, int n_in) {
  if (m <= 0 || n_out <= 0 || n_in <= 0) return 0;
  const int n_sm = sm_count_cached();
  if (!n_sm) return 0;
  const int kgroups = ceil_div(n_in, GROUP_ELEMS);
  const int gps = ceil_div(kgroups, skinny_splits(ceil_div(n_out, TILE_ROWS), kgroups, n_sm));
  return (size_t)ceil_div(kgroups, gps) * m * n_out * sizeof(float);
}

extern "C" int b200q_qgemm_skinny(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue,
                                  void* y, int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes, void* stream) {
  if (!w_packed || !x || !y || !workspace || m <= 0 || n_out <= 0 || n_in <= 0) return B200Q_ERR_BAD_ARG;
  if (m > SK_N) return B200Q_ERR_UNSUPPORTED;
  if (qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0) return B200Q_ERR_BAD_ARG;
  if ((x_dtype != B200Q_F32 && x_dtype != B200Q_F16) || (y_dtype != B200Q_F32 && y_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (epilogue != B200Q_EPI_LINEAR && epilogue != B200Q_EPI_SILU_MUL) return B200Q_ERR_BAD_ARG;
  if (epilogue == B200Q_EPI_SILU_MUL && (bias_f16 || residual || n_out % 16)) return B200Q_ERR_BAD_ARG;
  if (n_in % 32) return B200Q_ERR_BAD_SHAPE;
  if (((uintptr_t)w_packed | (uintptr_t)x | (uintptr_t)workspace) & 15) return B200Q_ERR_MISALIGNED;
  const int n_sm = sm_count_cached();
  if (!n_sm) return B200Q_ERR_CUDA;
  static PerDeviceFlag attr;
  const int dev = b200q_current_device();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!attr.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(tc_qgemm_skinny_kernel<B200Q_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, sk_smem_total(B200Q_Q4_0)));
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(tc_qgemm_skinny_kernel<B200Q_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, sk_smem_total(B200Q_Q8_0)));
    attr.set(dev);
  }
  SkinnyParams p;
  p.w = (const uint8_t*)w_packed; p.x = x; p.part = (float*)workspace;
  p.m = m; p.n_out = n_out; p.n_in = n_in; p.kgroups = ceil_div(n_in, GROUP_ELEMS); p.n_row_tiles = ceil_div(n_out, TILE_ROWS);
  p.x_f16 = x_dtype == B200Q_F16;
  int splits = skinny_splits(p.n_row_tiles, p.kgroups, n_sm);
  p.groups_per_split = ceil_div(p.kgroups, splits);
  splits = ceil_div(p.kgroups, p.groups_per_split);              // no empty split
  if ((size_t)splits * m * n_out * sizeof(float) > workspace_bytes) return B200Q_ERR_TOO_LARGE;
  dim3 grid(ceil_div(p.n_row_tiles, BN / 16), splits);
  if (qtype == B200Q_Q4_0) tc_qgemm_skinny_kernel<B200Q_Q4_0><<<grid, QGEMM_THREADS, sk_smem_total(B200Q_Q4_0), (cudaStream_t)stream>>>(p);
  else tc_qgemm_skinny_kernel<B200Q_Q8_0><<<grid, QGEMM_THREADS, sk_smem_total(B200Q_Q8_0), (cudaStream_t)stream>>>(p);
  B200Q_CHECK_CUDA(cudaGetLastError());
  const size_t n_y = (size_t)m * (epilogue == B200Q_EPI_SILU_MUL ? n_out / 2 : n_out);
  skinny_reduce_kernel<<<(unsigned)((n_y + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)workspace, splits, m, n_out, (const __half*)bias_f16,
                                                                                         residual, y, y_dtype == B200Q_F16, epilogue == B200Q_EPI_SILU_MUL);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
