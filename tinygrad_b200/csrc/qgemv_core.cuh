// Device pieces shared by the quantised-GEMV kernels (the per-launch GEMV and the whole-step decode kernel):
// mbarrier / bulk-copy primitives with bounded waits, and the multiply-accumulate of one packed weight tile
// (16 rows x 128 columns of Q4_0 / Q8_0) against a quantised activation record (actquant.cuh) on int8 tensor-core MMAs.
#pragma once
#include "common.cuh"

namespace {

constexpr int SPIN_LIMIT = 1 << 20;
__device__ int g_status = 0;                     // sticky, one per translation unit: 1 = a bounded wait ran out

// ---- mbarrier / bulk-copy primitives -------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Suspends the thread for a bounded time.  With the time hint the waiting warps come back less often and leave the issue slots to the
// warps that have a tile (measured: 1.8 % on the decode step; 500 ns .. 20 us all the same).
#ifndef B200Q_MBAR_HINT_NS
#define B200Q_MBAR_HINT_NS 2000
#endif
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
#if B200Q_MBAR_HINT_NS > 0
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity), "r"(B200Q_MBAR_HINT_NS) : "memory");
#else
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
#endif
  return ok != 0;
}
// Bounded wait: false (and the status word set) if the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < SPIN_LIMIT; i++) {
    if (mbar_try(bar, parity)) return true;
    if (i > 1024) __nanosleep(128);      // (sleeping after every failed try measured 0.7 % slower)
  }
  atomicExch(&g_status, 1);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// ---- tensor-core pieces ---------------------------------------------------------------
// first MMA of a tile: accumulator input is zero (no register clears)
template <int QT> __device__ __forceinline__ void imma0(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (QT == B200Q_Q4_0)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
template <int QT> __device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void imma<B200Q_Q4_0>(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void imma<B200Q_Q8_0>(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One weight tile (16 rows x 4 blocks) against the staged activation digits.
// bq: the lane's 8 B-operand words for its block (zeros unless the lane feeds this tile's diagonal),
// st: {scale_A, offset_A, scale_B, offset_B} of the lane's two accumulator columns.
template <int QT>
__device__ __forceinline__ void tile_mac(const uint8_t* tile, int lane, const uint4& bq0, const uint4& bq1, const float4& st, float& acc0, float& acc1) {
  const uint4* tp = reinterpret_cast<const uint4*>(tile);
  int c[4];
  uint2 sc;
  if (QT == B200Q_Q4_0) {
    // byte i of a block's 16 quant bytes = element i (low nibble) | element i+16 (high nibble)
    const uint4 r0 = tp[lane], r1 = tp[32 + lane];      // rows g and g+8
    sc = *(reinterpret_cast<const uint2*>(tile + 1024) + (2 * (lane >> 2) + (lane & 1)));
    const uint32_t M = 0x0F0F0F0Fu;
    imma0<QT>(c, r0.x & M, r1.x & M, (r0.x >> 4) & M, (r1.x >> 4) & M, bq0.x, bq0.y);
    imma<QT>(c, r0.y & M, r1.y & M, (r0.y >> 4) & M, (r1.y >> 4) & M, bq0.z, bq0.w);
    imma<QT>(c, r0.z & M, r1.z & M, (r0.z >> 4) & M, (r1.z >> 4) & M, bq1.x, bq1.y);
    imma<QT>(c, r0.w & M, r1.w & M, (r0.w >> 4) & M, (r1.w >> 4) & M, bq1.z, bq1.w);
  } else {
    const uint4 r0 = tp[lane], r1 = tp[32 + lane], r2 = tp[64 + lane], r3 = tp[96 + lane];   // row g: r0,r1; row g+8: r2,r3
    sc = *(reinterpret_cast<const uint2*>(tile + 2048) + (2 * (lane >> 2) + (lane & 1)));
    // same B word order as Q4_0: MMA j pairs elements 4j..4j+3 with 16+4j..16+4j+3
    imma0<QT>(c, r0.x, r2.x, r1.x, r3.x, bq0.x, bq0.y);
    imma<QT>(c, r0.y, r2.y, r1.y, r3.y, bq0.z, bq0.w);
    imma<QT>(c, r0.z, r2.z, r1.z, r3.z, bq1.x, bq1.y);
    imma<QT>(c, r0.w, r2.w, r1.w, r3.w, bq1.z, bq1.w);
  }
  const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&sc.x)), d1 = __half22float2(*reinterpret_cast<const __half2*>(&sc.y));
  const float oa = QT == B200Q_Q4_0 ? st.y : 0.f, ob = QT == B200Q_Q4_0 ? st.w : 0.f;   // only Q4_0 stores value + 8
  const float f0 = (float)c[0], f1 = (float)c[1], f2 = (float)c[2], f3 = (float)c[3];
  const float v0 = fmaf(f0, st.x, -oa), v1 = fmaf(f1, st.z, -ob);
  const float v2 = fmaf(f2, st.x, -oa), v3 = fmaf(f3, st.z, -ob);
  acc0 = fmaf(v0, d0.x, fmaf(v1, d0.y, acc0));
  acc1 = fmaf(v2, d1.x, fmaf(v3, d1.y, acc1));
}

// One Q6_K weight tile (16 rows x 128 columns = half a super-block per row) against the same activation digits.
// Tile bytes: uint4 L[2][32] low nibbles of the 6-bit quants (lane (g, t) of half h: row 8h + g, block t; byte i = element i | element
// i + 16 << 4), uint2 H[2][32] their high 2 bits (.x byte k: bits 2m, 2m+1 = element 4m + k, m = 0..3; .y the same for elements
// 16..31), int8 SC[16][8] sub-block scales (sub-block = 2 * block + half of the block), fp16 D[16] super-block scales.
// The quants stay unsigned (0..63) in the MMA; `sub` = the four offsets {block A first half, second half, block B first, second} of
// the lane's two columns (zero on the lanes that hold the low digits).  Weight value = d * scale * (q - 32)
// (tinygrad/llm/gguf.py:68-72).
__device__ __forceinline__ void tile_mac_q6k(const uint8_t* tile, int lane, const uint4& bq0, const uint4& bq1, const float4& st, const float4& sub,
                                             float& acc0, float& acc1) {
  const uint4* lp = reinterpret_cast<const uint4*>(tile);
  const uint2* hp = reinterpret_cast<const uint2*>(tile + 1024);
  const uint4 l0 = lp[lane], l1 = lp[32 + lane];      // rows g and g + 8
  const uint2 h0 = hp[lane], h1 = hp[32 + lane];
  const int g = lane >> 2, t = lane & 3;
  const uint32_t s0 = *reinterpret_cast<const uint32_t*>(tile + 1536 + g * 8 + (t & 1) * 4);
  const uint32_t s1 = *reinterpret_cast<const uint32_t*>(tile + 1536 + (g + 8) * 8 + (t & 1) * 4);
  const __half* dp = reinterpret_cast<const __half*>(tile + 1664);
  const float d0 = __half2float(dp[g]), d1 = __half2float(dp[g + 8]);
  const uint32_t M = 0x0F0F0F0Fu, H = 0x30303030u;
  int c0[4], c1[4];
  // first halves of the blocks (elements 0..15): two MMAs into c0; second halves into c1
  imma0<B200Q_Q4_0>(c0, (l0.x & M) | ((h0.x << 4) & H), (l1.x & M) | ((h1.x << 4) & H), (l0.y & M) | ((h0.x << 2) & H), (l1.y & M) | ((h1.x << 2) & H),
                    bq0.x, bq0.z);
  imma<B200Q_Q4_0>(c0, (l0.z & M) | (h0.x & H), (l1.z & M) | (h1.x & H), (l0.w & M) | ((h0.x >> 2) & H), (l1.w & M) | ((h1.x >> 2) & H), bq1.x, bq1.z);
  imma0<B200Q_Q4_0>(c1, ((l0.x >> 4) & M) | ((h0.y << 4) & H), ((l1.x >> 4) & M) | ((h1.y << 4) & H), ((l0.y >> 4) & M) | ((h0.y << 2) & H),
                    ((l1.y >> 4) & M) | ((h1.y << 2) & H), bq0.y, bq0.w);
  imma<B200Q_Q4_0>(c1, ((l0.z >> 4) & M) | (h0.y & H), ((l1.z >> 4) & M) | (h1.y & H), ((l0.w >> 4) & M) | ((h0.y >> 2) & H),
                   ((l1.w >> 4) & M) | ((h1.y >> 2) & H), bq1.y, bq1.w);
  // columns of this lane: blocks A = 2 * (t & 1) and B = A + 1 (high digits on t < 2, low digits on t >= 2)
  const float a0 = fmaf((float)c0[0], st.x, -sub.x), a1 = fmaf((float)c1[0], st.x, -sub.y);      // row g, block A, halves 0 / 1
  const float b0 = fmaf((float)c0[1], st.z, -sub.z), b1 = fmaf((float)c1[1], st.z, -sub.w);      // row g, block B
  const float e0 = fmaf((float)c0[2], st.x, -sub.x), e1 = fmaf((float)c1[2], st.x, -sub.y);      // row g + 8
  const float f0 = fmaf((float)c0[3], st.z, -sub.z), f1 = fmaf((float)c1[3], st.z, -sub.w);
  const float v0 = fmaf(a0, (float)(int8_t)(s0 & 0xFF), fmaf(a1, (float)(int8_t)((s0 >> 8) & 0xFF), fmaf(b0, (float)(int8_t)((s0 >> 16) & 0xFF),
                        b1 * (float)(int8_t)(s0 >> 24))));
  const float v1 = fmaf(e0, (float)(int8_t)(s1 & 0xFF), fmaf(e1, (float)(int8_t)((s1 >> 8) & 0xFF), fmaf(f0, (float)(int8_t)((s1 >> 16) & 0xFF),
                        f1 * (float)(int8_t)(s1 >> 24))));
  acc0 = fmaf(v0, d0, acc0);
  acc1 = fmaf(v1, d1, acc1);
}

}  // namespace
