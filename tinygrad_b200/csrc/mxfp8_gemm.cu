// Grouped (per-expert) MXFP8 GEMM on the 5th-generation tensor cores:
//   C[M, N] (bf16) = A_q[M, K] (e4m3) x B_q[e(row)][N, K]^T (e4m3), one E8M0 scale per 32 along K on both operands, fp32 accumulation.
// Rows of A are grouped by expert: group e = rows off[e] .. off[e+1], every group a multiple of 256 rows.
// Semantics: extra/gemm/moe_gemm.py:112-134 over the kernel contract of extra/thunder/amd/grouped_mxfp8_gemm.cpp:32-158
// (the reference computation it is tested against: dequantised operands matmul, test/backend/test_asm_gemm.py:289-292,306).
//
// Persistent, warp-specialised kernel, one CTA per SM, 128 x 256 output tiles, tiles of the used rows (off[E]) dealt round-robin:
//   warps 4-7  loaders: cp.async the A (128 x 128 B) and B (256 x 128 B) tiles of a K step into a 4-stage ring (K-major, 128-byte
//              swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7)) together with the step's E8M0 scale words (one 32-bit
//              word = 4 K blocks per row, stored as 32 x 16 B chunks: row r -> chunk r % 32, word r / 32); each thread's copies
//              arrive on the stage's "full" mbarrier when they land;
//   warp 8     one thread moves the scale chunks to tensor memory with tcgen05.cp 32x128b.warpx4 (row r -> lane r % 32 of every
//              32-lane sub-partition, column r / 32: the layout the MMA reads), issues tcgen05.mma kind::mxf8f6f4.block_scale
//              (scale_vec::1X, 128 x 256 x 32 per instruction, the tensor core applies both block scales), four per K step, and
//              commits each step to the stage's "empty" mbarrier;
//   warps 0-3, 9-20  epilogue: tcgen05.ld the fp32 accumulator (256 tensor-memory columns; four warps per 32-lane sub-partition,
//              64 columns each) into registers, release the accumulator, then round to bf16 and store (or SwiGLU + requantise).
// Loaders run ahead across tile boundaries; the accumulator (one buffer: 2 x 256 columns + the scale columns do not fit the 512 of
// tensor memory) is handed back after one tensor-memory round trip, the epilogue's arithmetic and stores overlap the next tile's MMAs.
// Every mbarrier wait is bounded; a wait that runs out raises a status word and makes every role leave.
#include "common.cuh"
#include "mxq.cuh"
#include <cuda.h>
#include <cuda_bf16.h>

#ifndef B200Q_MX_TMA
#define B200Q_MX_TMA 1      // 1: the A / B tiles of a K step arrive by two tensor-map (TMA) copies; 0: by 16-byte cp.async of 128 threads
#endif

namespace {

#ifndef B200Q_MX_STAGES
#define B200Q_MX_STAGES 3
#endif
constexpr int BM = 128, BN = 256, BK = 128, STAGES = B200Q_MX_STAGES;
constexpr int EPI_WARPS = 4, LOAD_WARPS = 4, EPI_Q = 4;      // epilogue: warps 0-3 and 9-20, EPI_Q warps per 32-lane sub-partition (64 columns each)
constexpr int THREADS = (EPI_Q * EPI_WARPS + LOAD_WARPS + 1) * 32;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, SF_BYTES = 2048;                    // scale chunks: A 512 B, B 2 x 512 B
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_BYTES;                               // 50 KB, a multiple of 1024
#ifndef B200Q_MX_STAGED_EPI
#define B200Q_MX_STAGED_EPI 2     // bf16 epilogue: 0 = each thread stores its own row (16-byte pieces of 32 different rows per instruction); 1 = through
#endif                            // 4 KB of shared memory per warp, stores of whole 128-byte row segments; 2 = the same, stored by one tensor-map copy
constexpr int EPI_STAGE_BYTES = B200Q_MX_STAGED_EPI ? 16 * 4096 : 0;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + EPI_STAGE_BYTES;               // + room to align the ring to 1024 B
constexpr int TMEM_COLS = 512;            // 256 accumulator columns + scale columns, rounded up to a power of two
constexpr int SFA_COL = 256, SFB_COL = 256 + 4 * STAGES;   // per stage 4 columns (A: 128 rows) and 8 columns (B: 256 rows)
constexpr int MAX_EXPERTS = 1024;
constexpr int SPIN = 1 << 22;

__device__ int g_mx_status = 0;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp16(uint32_t s, const void* g) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(g) : "memory"); }
__device__ __forceinline__ void cp4(uint32_t s, const void* g) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(g) : "memory"); }
__device__ __forceinline__ uint64_t desc_plain(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;      // core matrices adjacent in K
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;      // core matrices adjacent in M / N
  d |= (uint64_t)1 << 46;
  return d;
}
// K-major, 128-byte swizzle: 8-row groups 1024 B apart; a K offset inside the 128-byte row is added to the start address
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < SPIN; i++) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 255) == 255 && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicExch(&g_mx_status, 1);
  return false;
}
__device__ __forceinline__ void arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

// 32 consecutive accumulator columns of this thread's row (tensor-memory lane) -> registers; the caller waits (tcgen05.wait::ld)
__device__ __forceinline__ void tmem_ld32(uint32_t ta, uint32_t (&v)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                 "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                 "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
                 "=r"(v[31])
               : "r"(ta));
}
__device__ __forceinline__ void bf16_store32(const uint32_t (&v)[32], __nv_bfloat16* dst) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 pk;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int q = 0; q < 4; q++) h[q] = __floats2bfloat162_rn(__uint_as_float(v[j + 2 * q]), __uint_as_float(v[j + 2 * q + 1]));
    *reinterpret_cast<uint4*>(dst + j) = pk;
  }
}
// one MX block of the activation: gate / up accumulators of 32 columns -> silu(gate) * up -> E4M3 codes + block exponent at [row, col..col+31]
__device__ __forceinline__ void swiglu_quant_store(const uint32_t (&vg)[32], const uint32_t (&vu)[32], uint8_t* act_q, uint8_t* act_e8, size_t row, int f,
                                                   int col) {
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vg[j]))), u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(vu[j])));
    v[j] = __bfloat162float(__float2bfloat16_rn((g / (1.f + expf(-g))) * u));
    amax = fmaxf(amax, fabsf(v[j]));
  }
  const uint8_t e = mx_scale_exponent(amax);
  uint2 pk[4];
#pragma unroll
  for (int q = 0; q < 4; q++) {
    const float v8[8] = {v[8 * q], v[8 * q + 1], v[8 * q + 2], v[8 * q + 3], v[8 * q + 4], v[8 * q + 5], v[8 * q + 6], v[8 * q + 7]};
    pk[q] = mx_quant8(v8, e);
  }
  uint4* dst = reinterpret_cast<uint4*>(act_q + row * f + col);
  dst[0] = make_uint4(pk[0].x, pk[0].y, pk[1].x, pk[1].y);
  dst[1] = make_uint4(pk[2].x, pk[2].y, pk[3].x, pk[3].y);
  act_e8[row * (f >> 5) + (col >> 5)] = e;
}

__global__ void __launch_bounds__(THREADS, 1) grouped_mxfp8_tc_kernel(const uint8_t* __restrict__ a_q, const uint8_t* __restrict__ a_e8,
                                                                      const uint8_t* __restrict__ b_q, const uint8_t* __restrict__ b_e8,
                                                                      const int32_t* __restrict__ off, int n_experts, int m_total, int n, int k,
                                                                      __nv_bfloat16* __restrict__ c, uint8_t* __restrict__ act_q,
                                                                      uint8_t* __restrict__ act_e8, const __grid_constant__ CUtensorMap tm_a,
                                                                      const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_c,
                                                                      int c_f32) {
  extern __shared__ unsigned char sm_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc_full, bar_acc_empty, bar_drain;
  __shared__ uint32_t tmem_base;
  __shared__ int s_abort;
  __shared__ int s_off[MAX_EXPERTS + 1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&bar_full[s])), "r"(LOAD_WARPS * 32 + B200Q_MX_TMA));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar_empty[s])));
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar_acc_full)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&bar_acc_empty)), "r"(EPI_Q * EPI_WARPS * 32));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar_drain)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_abort = 0;
  }
  for (int i = tid; i <= n_experts; i += THREADS) s_off[i] = off[i];
  if (warp == EPI_WARPS + LOAD_WARPS) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t taddr = tmem_base;
  volatile int* abort_flag = &s_abort;
  const int kb_total = k >> 5, ktiles = k / BK;
  const int m_used = min(max(s_off[n_experts], 0), m_total);
  const int tiles_n = n / BN, n_tiles = (m_used / BM) * tiles_n;
  const uint32_t ring = (s32(sm_raw) + 1023u) & ~1023u;

  if (warp >= EPI_WARPS && warp < EPI_WARPS + LOAD_WARPS) {
    // ---------------------------------------------------------------- loaders
    const int lt = tid - EPI_WARPS * 32;            // 0..127
    const int r0 = lt >> 3, ch = lt & 7;            // this thread copies chunk ch of rows r0 + 16 j
    const uint32_t t_off = (uint32_t)(r0 * 128 + ((ch ^ (r0 & 7)) << 4));
    const uint32_t sf_off = (uint32_t)((lt & 31) * 16 + (lt >> 5) * 4);      // scale word of row lt (A), rows lt and lt + 128 (B)
    int b_row0 = 0;       // first row of the tile's B operand inside [n_experts * n, k]
    auto tile_ptrs = [&](int t, const uint8_t*& ap, const uint8_t*& bp, const uint8_t*& ae, const uint8_t*& be) {
      const int m0 = (t / tiles_n) * BM, n0 = (t % tiles_n) * BN;
      int lo = 0, hi = n_experts - 1;
      while (lo < hi) { const int mid = (lo + hi) >> 1; if (s_off[mid + 1] <= m0) lo = mid + 1; else hi = mid; }
      ap = a_q + (size_t)(m0 + r0) * k + ch * 16;
      bp = b_q + ((size_t)lo * n + n0 + r0) * k + ch * 16;
      ae = a_e8 + (size_t)(m0 + lt) * kb_total;
      be = b_e8 + ((size_t)lo * n + n0 + lt) * kb_total;
      b_row0 = lo * n + n0;
    };
    uint32_t g = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
      const uint8_t *ap, *bp, *ae, *be;
      tile_ptrs(t, ap, bp, ae, be);
      for (int kt = 0; kt < ktiles; kt++, g++) {
        const uint32_t slot = g % STAGES;
        if (g >= STAGES && !wait_bar(s32(&bar_empty[slot]), ((g / STAGES) - 1) & 1, abort_flag)) { ok = false; break; }
        const uint32_t sA = ring + slot * STAGE_BYTES, sB = sA + A_BYTES, sF = sB + B_BYTES;
        const uint8_t* pa = ap + kt * BK;
        const uint8_t* pb = bp + kt * BK;
#if B200Q_MX_TMA
        if (lt == 0) {
          // the 128-byte-swizzle tiled copy writes exactly the layout above (chunk c of row r at c ^ (r & 7)); no multicast
          const uint32_t fb = s32(&bar_full[slot]);
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(A_BYTES + B_BYTES) : "memory");
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(sA), "l"(&tm_a), "r"(kt * BK), "r"((t / tiles_n) * BM), "r"(fb) : "memory");
          asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                       ::"r"(sB), "l"(&tm_b), "r"(kt * BK), "r"(b_row0), "r"(fb) : "memory");
        }
        (void)pa; (void)pb; (void)t_off;
#else
#pragma unroll
        for (int j = 0; j < BM / 16; j++) cp16(sA + t_off + j * 2048, pa + (size_t)(16 * j) * k);
#pragma unroll
        for (int j = 0; j < BN / 16; j++) cp16(sB + t_off + j * 2048, pb + (size_t)(16 * j) * k);
#endif
        cp4(sF + sf_off, ae + kt * 4);
        cp4(sF + 512 + sf_off, be + kt * 4);
        cp4(sF + 1024 + sf_off, be + (size_t)128 * kb_total + kt * 4);
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(s32(&bar_full[slot])) : "memory");
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
#if B200Q_MX_TMA
    // nothing of this thread's tensor-map copies may still be landing when the CTA leaves (they are all consumed unless a wait ran out)
    if (lt == 0)
      for (uint32_t j = g > STAGES ? g - STAGES : 0; j < g; j++) {
        const uint32_t fb = s32(&bar_full[j % STAGES]), par = (j / STAGES) & 1;
        for (int i = 0; i < SPIN; i++) {
          uint32_t done;
          asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(done) : "r"(fb), "r"(par) : "memory");
          if (done) break;
        }
      }
#endif
  } else if (warp == EPI_WARPS + LOAD_WARPS) {
    // ---------------------------------------------------------------- MMA issue (one thread)
    if (lane == 0) {
      uint32_t g = 0, tile_i = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, tile_i++) {
        if (tile_i > 0 && !wait_bar(s32(&bar_acc_empty), (tile_i - 1) & 1, abort_flag)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kt = 0; kt < ktiles; kt++, g++) {
          const uint32_t slot = g % STAGES;
          if (!wait_bar(s32(&bar_full[slot]), (g / STAGES) & 1, abort_flag)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          const uint32_t sA = ring + slot * STAGE_BYTES, sB = sA + A_BYTES, sF = sB + B_BYTES;
          // scale chunks -> tensor memory (32 lanes x 16 B, replicated into the four sub-partitions); ordered before the MMAs below
          asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr + SFA_COL + slot * 4), "l"(desc_plain(sF, 128, 128)) : "memory");
          asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr + SFB_COL + slot * 8), "l"(desc_plain(sF + 512, 128, 128)) : "memory");
          asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr + SFB_COL + slot * 8 + 4), "l"(desc_plain(sF + 1024, 128, 128)) : "memory");
#pragma unroll
          for (int kb = 0; kb < 4; kb++) {
            const uint64_t da = desc_sw128(sA + kb * 32), db = desc_sw128(sB + kb * 32);
            // block-scaled instruction descriptor: B scale id [4,6), E4M3 x E4M3, N>>3 [17,23), E8M0 scales (bit 23), M>>7 [27,29), A scale id [29,31)
            const uint32_t idesc = ((uint32_t)kb << 4) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) | ((uint32_t)(BM >> 7) << 27) | ((uint32_t)kb << 29);
            const uint32_t acc = (kt > 0 || kb > 0) ? 1u : 0u;
            asm volatile("{\n.reg .pred p;\nsetp.ne.u32 p, %6, 0;\n"
                         "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}"
                         ::"r"(taddr), "l"(da), "l"(db), "r"(idesc), "r"(taddr + SFA_COL + slot * 4), "r"(taddr + SFB_COL + slot * 8), "r"(acc) : "memory");
          }
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&bar_empty[slot])) : "memory");
        }
        if (ok) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&bar_acc_full)) : "memory");
      }
      if (!ok) {     // leave nothing in flight before the tensor memory is given back
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(&bar_drain)) : "memory");
        for (int i = 0; i < SPIN; i++) {
          uint32_t done;
          asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(done) : "r"(s32(&bar_drain)) : "memory");
          if (done) break;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: accumulator row r = tensor-memory lane r
    // Four warps per 32-lane sub-partition (a warp reaches only the lanes of sub-partition warp % 4), 64 columns each.  A warp brings
    // its columns into registers with two loads in flight and ONE wait, releases the accumulator, and only then does its arithmetic
    // and stores: the next tile's MMAs wait for one tensor-memory round trip, not for the epilogue.
    const int sub = warp & 3, cq = warp < EPI_WARPS ? 0 : 1 + (warp - (EPI_WARPS + LOAD_WARPS + 1)) / 4;      // column quarter 0..3
    uint32_t tile_i = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, tile_i++) {
      if (!wait_bar(s32(&bar_acc_full), tile_i & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m0 = (t / tiles_n) * BM, n0 = (t % tiles_n) * BN;
      const uint32_t ta = taddr + ((uint32_t)(sub * 32) << 16);
      const size_t row = (size_t)(m0 + sub * 32 + lane);
      uint32_t v0[32], v1[32];
      if (act_q) {
        // Fused activation between the expert GEMMs: the B rows of this tile are 128 gate rows followed by the 128 matching up rows
        // (the caller interleaves them so), so accumulator columns c and 128 + c belong together.  A thread holds 32 consecutive
        // outputs of its row = one MX block: bf16-round gate and up (what the unfused path stores), silu(gate) * up in fp32,
        // bf16-round, block exponent from the amax, E4M3 codes -- the arithmetic of swiglu_quant_kernel, with no trip through HBM.
        tmem_ld32(ta + cq * 32, v0); tmem_ld32(ta + BN / 2 + cq * 32, v1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        arrive(s32(&bar_acc_empty));
        swiglu_quant_store(v0, v1, act_q, act_e8, row, n >> 1, (n0 >> 1) + cq * 32);
        continue;
      }
      tmem_ld32(ta + cq * 64, v0); tmem_ld32(ta + cq * 64 + 32, v1);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      arrive(s32(&bar_acc_empty));
      if (c_f32) {      // unrounded sums (the per-tensor FP8 linear scales them afterwards): each thread stores its own row
        float4* o4 = reinterpret_cast<float4*>(reinterpret_cast<float*>(c) + row * n + n0 + cq * 64);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          o4[j] = make_float4(__uint_as_float(v0[4 * j]), __uint_as_float(v0[4 * j + 1]), __uint_as_float(v0[4 * j + 2]), __uint_as_float(v0[4 * j + 3]));
          o4[8 + j] = make_float4(__uint_as_float(v1[4 * j]), __uint_as_float(v1[4 * j + 1]), __uint_as_float(v1[4 * j + 2]), __uint_as_float(v1[4 * j + 3]));
        }
        continue;
      }
      __nv_bfloat16* out_row = c + row * n + n0 + cq * 64;
#if B200Q_MX_STAGED_EPI
      {
        // row `lane`, 64 columns = eight 16-byte packets -> this warp's staging rows (packet p of row r at p ^ (r & 7): conflict-free
        // both ways) -> read back four rows x 128 contiguous bytes per instruction and store those
        unsigned char* stg = sm_raw + (ring - s32(sm_raw)) + STAGES * STAGE_BYTES + (warp < EPI_WARPS ? warp : warp - (LOAD_WARPS + 1)) * 4096;
#pragma unroll
        for (int p8 = 0; p8 < 8; p8++) {
          uint4 pk;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const int j = p8 * 8 + 2 * q;
            h[q] = j < 32 ? __floats2bfloat162_rn(__uint_as_float(v0[j]), __uint_as_float(v0[j + 1]))
                          : __floats2bfloat162_rn(__uint_as_float(v1[j - 32]), __uint_as_float(v1[j - 31]));
          }
          *reinterpret_cast<uint4*>(stg + lane * 128 + ((p8 ^ (lane & 7)) << 4)) = pk;
        }
#if B200Q_MX_STAGED_EPI == 2
        // the staging rows are in the 128-byte-swizzle layout a tiled tensor-map store reads: one copy per warp and tile
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                       ::"l"(&tm_c), "r"(n0 + cq * 64), "r"(m0 + sub * 32), "r"(s32(stg)) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the rows may be overwritten for the next tile
        }
        __syncwarp();
#else
        __syncwarp();
        __nv_bfloat16* out_tile = c + (size_t)(m0 + sub * 32) * n + n0 + cq * 64;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int r = 4 * i + (lane >> 3), p8 = lane & 7;
          const uint4 pk = *reinterpret_cast<const uint4*>(stg + r * 128 + ((p8 ^ (r & 7)) << 4));
          *reinterpret_cast<uint4*>(out_tile + (size_t)r * n + p8 * 8) = pk;
        }
        __syncwarp();
#endif
        (void)out_row;
      }
#elif !defined(B200Q_MX_EXP_NOSTORE)
      bf16_store32(v0, out_row); bf16_store32(v1, out_row + 32);
#else
      if (v0[0] == 0x12345678u && v1[5] == 0x9abcdef0u) bf16_store32(v0, out_row);
#endif
    }
#if B200Q_MX_STAGED_EPI == 2
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // this warp's stores have left before the CTA does
#endif
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == EPI_WARPS + LOAD_WARPS) {
    __syncwarp();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

extern "C" int b200q_mx_status_read_clear(int* status) {
  if (!status) return B200Q_ERR_BAD_ARG;
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_mx_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_mx_status, &zero, sizeof(int)));
  int ep = 0;
  const int rc = b200q_ep_status_take(&ep);       // the exchange kernels around the expert GEMMs report through the same word
  if (rc) return rc;
  if (*status == 0) *status = ep;
  return B200Q_OK;
}

// [rows, k] bytes, row-major -> tiled tensor map with boxes of `box_rows` rows x 128 bytes in the 128-byte-swizzle shared-memory layout.
// The encoder is a driver entry point; it is looked up through the runtime so that the library links against cudart only.
static int make_map(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t k, uint32_t box_rows, bool bf16 = false) {
  typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static encode_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    B200Q_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (!p || q != cudaDriverEntryPointSuccess) return B200Q_ERR_UNSUPPORTED;
    fn = (encode_fn)p;
  }
  // bf16: `k` counts elements, a box row is 64 of them (128 bytes); else bytes, a box row is BK = 128 of them
  const cuuint64_t dims[2] = {k, rows}, strides[1] = {bf16 ? 2 * k : k};
  const cuuint32_t box[2] = {(cuuint32_t)(bf16 ? 64 : BK), box_rows}, estr[2] = {1, 1};
  const CUresult r = fn(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200Q_OK : B200Q_ERR_BAD_ARG;
}

static int grouped_launch(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts, int m_total, int n, int k,
                          void* c_bf16, void* act_q, void* act_e8, void* stream, bool c_f32 = false) {
  if (!a_q || !a_e8 || !b_q || !b_e8 || !off || (!c_bf16 && !act_q) || n_experts <= 0 || m_total <= 0 || n <= 0 || k <= 0) return B200Q_ERR_BAD_ARG;
  if (act_q && (!act_e8 || (((uintptr_t)act_q) & 15))) return B200Q_ERR_BAD_ARG;
  if (m_total % 256 || n % BN || k % BK) return B200Q_ERR_BAD_SHAPE;       // the reference asks M % 256 == N % 256 == K % 128 == 0 (moe_gemm.py:120)
  if (n_experts > MAX_EXPERTS) return B200Q_ERR_UNSUPPORTED;
  if (((uintptr_t)a_q | (uintptr_t)b_q | (uintptr_t)c_bf16) & 15 || ((uintptr_t)a_e8 | (uintptr_t)b_e8) & 3) return B200Q_ERR_MISALIGNED;
  static PerDeviceFlag attr_set;
  const int dev = b200q_current_device(), n_sm = b200q_sm_count();
  if (dev < 0 || n_sm <= 0) return B200Q_ERR_CUDA;
  if (!attr_set.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(grouped_mxfp8_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_set.set(dev);
  }
  const long long tiles = (long long)(m_total / BM) * (n / BN);
  const int grid = (int)(tiles < n_sm ? tiles : n_sm);
  alignas(64) CUtensorMap tm_a, tm_b, tm_c;
  memset(&tm_a, 0, sizeof(tm_a)); memset(&tm_b, 0, sizeof(tm_b)); memset(&tm_c, 0, sizeof(tm_c));
#if B200Q_MX_STAGED_EPI == 2
  if (c_bf16 && !c_f32) { const int rcc = make_map(&tm_c, c_bf16, (uint64_t)m_total, (uint64_t)n, 32, true); if (rcc != B200Q_OK) return rcc; }
#endif
#if B200Q_MX_TMA
  int rc = make_map(&tm_a, a_q, (uint64_t)m_total, (uint64_t)k, BM);
  if (rc == B200Q_OK) rc = make_map(&tm_b, b_q, (uint64_t)n_experts * n, (uint64_t)k, BN);
  if (rc != B200Q_OK) return rc;
#endif
  grouped_mxfp8_tc_kernel<<<grid, THREADS, SMEM_BYTES, (cudaStream_t)stream>>>((const uint8_t*)a_q, (const uint8_t*)a_e8, (const uint8_t*)b_q, (const uint8_t*)b_e8, off,
                                                            n_experts, m_total, n, k, (__nv_bfloat16*)c_bf16, (uint8_t*)act_q, (uint8_t*)act_e8, tm_a, tm_b, tm_c, c_f32 ? 1 : 0);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_grouped_mxfp8_gemm(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                                        int m_total, int n, int k, void* c_bf16, void* stream) {
  if (!c_bf16) return B200Q_ERR_BAD_ARG;
  return grouped_launch(a_q, a_e8, b_q, b_e8, off, n_experts, m_total, n, k, c_bf16, nullptr, nullptr, stream);
}

extern "C" int b200q_grouped_mxfp8_gemm_f32(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                                            int m_total, int n, int k, float* c_f32, void* stream) {
  if (!c_f32) return B200Q_ERR_BAD_ARG;
  return grouped_launch(a_q, a_e8, b_q, b_e8, off, n_experts, m_total, n, k, c_f32, nullptr, nullptr, stream, true);
}

extern "C" int b200q_grouped_mxfp8_gemm_swiglu(const void* a_q, const void* a_e8, const void* b_q, const void* b_e8, const int32_t* off, int n_experts,
                                               int m_total, int n, int k, void* act_q, void* act_e8, void* stream) {
  if (!act_q || !act_e8) return B200Q_ERR_BAD_ARG;
  return grouped_launch(a_q, a_e8, b_q, b_e8, off, n_experts, m_total, n, k, nullptr, act_q, act_e8, stream);
}
