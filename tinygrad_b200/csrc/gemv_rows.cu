// Weight-dequant-fused linear for a FEW activation rows (batched decode: up to 8 sequences per pass), on the int8 tensor cores.
//
// Replaces `Linear.__call__` on a GGUF weight when the model runs B sequences in lock-step (tokens [B, 1], tinygrad/llm/model.py:358-367).
// The one-row GEMV (gemv.cu) spends one MMA column per (quant block, digit); here the 8 MMA columns are 8 activation ROWS: for every
// quant block of a 16 x 128 weight tile one m16n8k32 MMA per activation digit (high / low 7 bits of a 15-bit integer) yields the exact
// integer dot products of 16 weight rows with 8 activation rows, which are scaled by (activation scale x fp16 weight scale) and added
// up in fp32 -- the weights are streamed ONCE for all 8 rows.  A weight tile keeps (row, block) pairs per lane, an MMA wants one
// block across the quad's lanes: a 4 x 4 word transpose inside each quad (four shuffles) bridges the two.
//
// Pre-pass (rows_record_kernel): the activation rows are quantised once (per block of 32: fp32 scale, 15-bit integers split in two int8
// digits) into the B-operand order of the MMA, per K chunk of 32 column groups.  Main kernel: grid (CTAs over row tiles, K chunks);
// a CTA brings its chunk's record into shared memory by bulk copies, then streams its row tiles' chunk of weights through a ring of
// bulk-copied stages (one stage = one tile's chunk), 16 consumer warps, 2 column groups per warp and stage; four finisher warps add the
// consumers' partial sums of a tile in a fixed order while the consumers are on the next tile, and apply the epilogue (one K chunk) or
// leave partial sums in a workspace [chunk][row][n_out] that a last kernel adds in a fixed order with bias / residual / SwiGLU (no
// floating-point atomics: bit-reproducible).  Every mbarrier wait is bounded (status word on expiry, see gemv.cu).
#include "common.cuh"
#include "qgemv_core.cuh"

namespace {

#ifndef B200Q_R_WARPS
#define B200Q_R_WARPS 16
#endif
#ifndef B200Q_R_CG
#define B200Q_R_CG 32
#endif
#ifndef B200Q_R_NS4
#define B200Q_R_NS4 3
#endif
#ifndef B200Q_R_NS8
#define B200Q_R_NS8 2
#endif
constexpr int R_FIN = 4;                                        // finisher warps: 128 outputs (16 weight rows x 8 activation rows) per row tile
constexpr int R_WARPS = B200Q_R_WARPS, R_THREADS = R_WARPS * 32 + 32 + R_FIN * 32;      // consumers + the producer warp + the finishers
constexpr int R_CG = B200Q_R_CG;                                // column groups (of 128 inputs) per K chunk = per ring stage
__host__ __device__ constexpr int rows_ns(int qtype) { return qtype == B200Q_Q4_0 ? B200Q_R_NS4 : B200Q_R_NS8; }      // ring depth (a stage is 36 KB of Q4_0, 68 KB of Q8_0)
constexpr int R_TOK = 8;                                        // activation rows per pass = MMA columns
constexpr int REC_GROUP = 32 * 64;                              // record bytes per column group: 32 lanes x 16 words
constexpr int SC_GROUP = R_TOK * 4 * 8;                         // scale bytes per column group: [row][block]{scale, offset}

#ifdef B200Q_ROWS_PROF
// experiment builds only: per CTA {start, record in, end (globaltimer ns), clocks waiting for weights, computing, in the cross-warp sum, producer waiting for a free slot, stages}
__device__ unsigned long long g_rows_prof[1024 * 8];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define RSTAMP(i, v) do { if (lane == 0) g_rows_prof[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + (i)] = (v); } while (0)
#endif

struct RowsParams {
  const uint8_t* w; const unsigned char* record; float* part;
  int m, n_out, kgroups, n_row_tiles, n_chunks;
  // one K chunk: the epilogue runs in the streaming kernel (no partial sums, no third launch)
  const __half* bias; const void* residual; void* y; int y_f16, silu_mul;
};

// ---- pre-pass: x [m, n_in] -> per chunk c and group j:  words [c][j][b][lane = 4 * row + t][{hi0, hi1, lo0, lo1}]  (row < 8: zero rows
// past m), hi0 / lo0 = the digits of elements 4t..4t+3 of block b, hi1 / lo1 = of elements 16+4t..16+4t+3 (the k order of m16n8k32's B
// fragment); then  float2 [c][j][row][b] = {scale, 8 * scale * sum(q)}  (the second removes Q4_0's offset of 8).  One warp per (row, block).
template <typename T>
__global__ void __launch_bounds__(256) rows_record_kernel(const T* __restrict__ x, int m, int n_in, int kgroups, unsigned char* __restrict__ record,
                                                          const __half* __restrict__ norm_w, float norm_eps) {
  // a CTA = 8 warps on 8 consecutive blocks of ONE activation row, so that the row's RMS (norm_w: RMSNorm folded into the quantisation,
  // x * rsqrt(mean(x^2) + eps) * w as tinygrad/llm/model.py:159 applies before every Linear of a block) is computed once per CTA
  __shared__ float s_ss[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x % R_TOK, bi = (blockIdx.x / R_TOK) * 8 + warp;      // block index along K
  pdl_wait();
  pdl_launch_dependents();
  float sc = 1.f;
  if (norm_w) {                                                  // fp32 rows only (checked by the host)
    float ss = 0.f;
    if (row < m) {
      const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)row * n_in);
      for (int i = threadIdx.x; i < n_in / 4; i += 256) { const float4 v4 = xr[i]; ss += v4.x * v4.x + v4.y * v4.y + v4.z * v4.z + v4.w * v4.w; }
    }
    ss = warp_sum(ss);
    if (lane == 0) s_ss[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += s_ss[i];
    sc = 1.0f / sqrtf(tot / (float)n_in + norm_eps);
  }
  if (bi >= kgroups * 4) return;
  const int blk = bi & 3, j = bi >> 2;
  const int k = j * GROUP_ELEMS + blk * 32 + lane;
  float v = 0.f;
  if (row < m && k < n_in) {
    v = sizeof(T) == 2 ? __half2float(reinterpret_cast<const __half*>(x)[(size_t)row * n_in + k]) : reinterpret_cast<const float*>(x)[(size_t)row * n_in + k];
    if (norm_w) v = v * sc * __half2float(norm_w[k]);
  }
  const float amax = warp_max(fabsf(v));
  const bool live = amax > 0.f && amax < INFINITY;
  const float inv = live ? 16256.f / amax : 0.f, s = live ? amax / 16256.f : 0.f;
  const int q = __float2int_rn(v * inv);
  int qsum = q;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
  const int h = (q + 64) >> 7;
  const uint32_t hb = h & 0xFF, lb = (q - (h << 7)) & 0xFF;
  const uint32_t hiw = hb | (__shfl_down_sync(0xffffffffu, hb, 1) << 8) | (__shfl_down_sync(0xffffffffu, hb, 2) << 16) | (__shfl_down_sync(0xffffffffu, hb, 3) << 24);
  const uint32_t low = lb | (__shfl_down_sync(0xffffffffu, lb, 1) << 8) | (__shfl_down_sync(0xffffffffu, lb, 2) << 16) | (__shfl_down_sync(0xffffffffu, lb, 3) << 24);
  const int chunk = j / R_CG, jj = j % R_CG;
  const int cg = min(R_CG, kgroups - chunk * R_CG);              // groups of this chunk
  unsigned char* base = record + (size_t)chunk * R_CG * (REC_GROUP + SC_GROUP);     // chunk c: its words, then its scales
  if ((lane & 3) == 0) {
    const int e4 = lane >> 2, t = e4 & 3, half = e4 >> 2;        // elements 4 e4 .. 4 e4 + 3
    uint32_t* wp = reinterpret_cast<uint32_t*>(base + (size_t)jj * REC_GROUP) + (blk * 32 + row * 4 + t) * 4;
    wp[half] = hiw; wp[2 + half] = low;
  }
  if (lane == 0) {
    float2* sp = reinterpret_cast<float2*>(base + (size_t)cg * REC_GROUP + (size_t)jj * SC_GROUP) + row * 4 + blk;
    *sp = make_float2(s, 8.f * s * (float)qsum);
  }
}

// 4 x 4 word transpose inside a quad: lane t ends up with word t of lanes 0, 1, 2, 3 (out.x .. out.w).  Two butterfly steps (2 x 2
// words between lanes t and t ^ 1, then 2 x 2 pairs between t and t ^ 2): four shuffles and twelve selects on two lane-constant bits.
__device__ __forceinline__ uint4 quad_transpose(const uint4 r, int t) {
  const bool b0 = (t & 1) != 0, b1 = (t & 2) != 0;
  uint32_t s0 = b0 ? r.x : r.y, s1 = b0 ? r.z : r.w;             // odd lanes give away words 0, 2; even lanes words 1, 3
  s0 = __shfl_xor_sync(0xffffffffu, s0, 1); s1 = __shfl_xor_sync(0xffffffffu, s1, 1);
  const uint32_t x = b0 ? s0 : r.x, y = b0 ? r.y : s0, z = b0 ? s1 : r.z, w = b0 ? r.w : s1;
  uint32_t u0 = b1 ? x : z, u1 = b1 ? y : w;                     // lanes 2, 3 give away the first pair, lanes 0, 1 the second
  u0 = __shfl_xor_sync(0xffffffffu, u0, 2); u1 = __shfl_xor_sync(0xffffffffu, u1, 2);
  uint4 o;
  o.x = b1 ? u0 : x; o.y = b1 ? u1 : y; o.z = b1 ? z : u0; o.w = b1 ? w : u1;
  return o;
}

__device__ __forceinline__ void imma_u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// One weight tile (16 rows x 4 blocks) against 8 activation rows.  xw: this lane's 16 record words of the column group, xs: the
// {scale, offset} pairs of the lane's two activation rows (2t, 2t + 1) for the 4 blocks.  acc: rows g / g + 8 x activation rows 2t / 2t + 1.
template <int QT>
__device__ __forceinline__ void tile_mac_rows(const uint8_t* tile, int lane, const uint4 (&xw)[4], const float4 (&xs)[4], float (&acc)[4]) {
  const int g = lane >> 2, t = lane & 3;
  const uint4* tp = reinterpret_cast<const uint4*>(tile);
  const uint32_t M = 0x0F0F0F0Fu;
  uint32_t a[4][4];      // [block][a0..a3]
  if (QT == B200Q_Q4_0) {
    const uint4 w0 = quad_transpose(tp[lane], t), w1 = quad_transpose(tp[32 + lane], t);      // rows g, g + 8: word t of blocks 0..3
    const uint32_t r0[4] = {w0.x, w0.y, w0.z, w0.w}, r1[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int b = 0; b < 4; b++) { a[b][0] = r0[b] & M; a[b][1] = r1[b] & M; a[b][2] = (r0[b] >> 4) & M; a[b][3] = (r1[b] >> 4) & M; }
  } else {
    const uint4 w0 = quad_transpose(tp[lane], t), w2 = quad_transpose(tp[32 + lane], t);      // row g: elements 0..15, 16..31 of the lane's block
    const uint4 w1 = quad_transpose(tp[64 + lane], t), w3 = quad_transpose(tp[96 + lane], t); // row g + 8
    const uint32_t r0[4] = {w0.x, w0.y, w0.z, w0.w}, r2[4] = {w2.x, w2.y, w2.z, w2.w}, r1[4] = {w1.x, w1.y, w1.z, w1.w}, r3[4] = {w3.x, w3.y, w3.z, w3.w};
#pragma unroll
    for (int b = 0; b < 4; b++) { a[b][0] = r0[b]; a[b][1] = r1[b]; a[b][2] = r2[b]; a[b][3] = r3[b]; }
  }
  // fp16 weight scales: entry 2g + p holds {block 2p row g, block 2p+1 row g, block 2p row g+8, block 2p+1 row g+8}
  const uint2* sp = reinterpret_cast<const uint2*>(tile + (QT == B200Q_Q4_0 ? 1024 : 2048));
  const uint2 s01 = sp[2 * g], s23 = sp[2 * g + 1];
  const float2 d01a = __half22float2(*reinterpret_cast<const __half2*>(&s01.x)), d01b = __half22float2(*reinterpret_cast<const __half2*>(&s01.y));
  const float2 d23a = __half22float2(*reinterpret_cast<const __half2*>(&s23.x)), d23b = __half22float2(*reinterpret_cast<const __half2*>(&s23.y));
  const float da[4] = {d01a.x, d01a.y, d23a.x, d23a.y}, db[4] = {d01b.x, d01b.y, d23b.x, d23b.y};      // rows g and g + 8
  const uint32_t xwv[16] = {xw[0].x, xw[0].y, xw[0].z, xw[0].w, xw[1].x, xw[1].y, xw[1].z, xw[1].w, xw[2].x, xw[2].y, xw[2].z, xw[2].w,
                            xw[3].x, xw[3].y, xw[3].z, xw[3].w};
  // xs: [0] = row 2t blocks 0,1 {s, o, s, o}; [1] = row 2t blocks 2,3; [2], [3] = the same for row 2t + 1
  const float se[4] = {xs[0].x, xs[0].z, xs[1].x, xs[1].z}, oe[4] = {xs[0].y, xs[0].w, xs[1].y, xs[1].w};
  const float so[4] = {xs[2].x, xs[2].z, xs[3].x, xs[3].z}, oo[4] = {xs[2].y, xs[2].w, xs[3].y, xs[3].w};
#pragma unroll
  for (int b = 0; b < 4; b++) {
    int ch[4], cl[4];
    if (QT == B200Q_Q4_0) {
      imma_u8(ch, a[b][0], a[b][1], a[b][2], a[b][3], xwv[b * 4 + 0], xwv[b * 4 + 1]);
      imma_u8(cl, a[b][0], a[b][1], a[b][2], a[b][3], xwv[b * 4 + 2], xwv[b * 4 + 3]);
    } else {
      imma_s8(ch, a[b][0], a[b][1], a[b][2], a[b][3], xwv[b * 4 + 0], xwv[b * 4 + 1]);
      imma_s8(cl, a[b][0], a[b][1], a[b][2], a[b][3], xwv[b * 4 + 2], xwv[b * 4 + 3]);
    }
    const float oe_b = QT == B200Q_Q4_0 ? oe[b] : 0.f, oo_b = QT == B200Q_Q4_0 ? oo[b] : 0.f;      // only Q4_0 stores value + 8
    const float v0 = fmaf((float)(ch[0] * 128 + cl[0]), se[b], -oe_b), v1 = fmaf((float)(ch[1] * 128 + cl[1]), so[b], -oo_b);
    const float v2 = fmaf((float)(ch[2] * 128 + cl[2]), se[b], -oe_b), v3 = fmaf((float)(ch[3] * 128 + cl[3]), so[b], -oo_b);
    acc[0] = fmaf(v0, da[b], acc[0]); acc[1] = fmaf(v1, da[b], acc[1]);
    acc[2] = fmaf(v2, db[b], acc[2]); acc[3] = fmaf(v3, db[b], acc[3]);
  }
}

__device__ __forceinline__ void rows_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(R_WARPS * 32) : "memory"); }

template <int QT>
__global__ void __launch_bounds__(R_THREADS, 1) qgemv_rows_kernel(const RowsParams p) {
  constexpr int TB = tile_bytes(QT), STAGE = R_CG * TB, R_NS = rows_ns(QT);
  extern __shared__ __align__(128) unsigned char rsm[];
  unsigned char* ring = rsm;
  unsigned char* rec = rsm + R_NS * STAGE;                       // words of the chunk's groups, then their scales
  float* red = reinterpret_cast<float*>(rec + R_CG * (REC_GROUP + SC_GROUP));      // [2][R_WARPS][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * R_WARPS * 128);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 2 * R_NS + 5);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + R_NS), rbar = smem_u32(bars + 2 * R_NS);
  const uint32_t rfull0 = smem_u32(bars + 2 * R_NS + 1), rempty0 = smem_u32(bars + 2 * R_NS + 3);      // the two buffers of `red`
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = blockIdx.y, cg = min(R_CG, p.kgroups - chunk * R_CG);
  if (tid == 0) {
    for (int s = 0; s < R_NS; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, R_WARPS); }
    mbar_init(rbar, 1);
    for (int b = 0; b < 2; b++) { mbar_init(rfull0 + 8 * b, R_WARPS); mbar_init(rempty0 + 8 * b, R_FIN); }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();
  if (warp == R_WARPS) {
    // ------------------------------ producer: weights do not depend on the previous kernel, the record does
    if (lane == 0) {
      int it = 0;
      bool ok = true, rec_issued = false;
#ifdef B200Q_ROWS_PROF
      long long p_wait = 0;
#endif
      auto fetch_record = [&]() {
        pdl_wait();
        const uint32_t bytes = (uint32_t)cg * (REC_GROUP + SC_GROUP);
        const unsigned char* src = p.record + (size_t)chunk * R_CG * (REC_GROUP + SC_GROUP);
        mbar_expect_tx(rbar, bytes);
        for (uint32_t o = 0; o < bytes; o += 8192) bulk_g2s(smem_u32(rec) + o, src + o, min(8192u, bytes - o), rbar);
        rec_issued = true;
      };
      for (int rt = blockIdx.x; rt < p.n_row_tiles && ok; rt += gridDim.x, it++) {
        const int slot = it % R_NS;
        if (it == R_NS && !rec_issued) fetch_record();
#ifdef B200Q_ROWS_PROF
        const long long pc0 = clock64();
#endif
        if (!mbar_wait(empty0 + 8 * slot, ((it / R_NS) & 1) ^ 1)) { ok = false; break; }
#ifdef B200Q_ROWS_PROF
        p_wait += clock64() - pc0;
#endif
        const uint8_t* src = p.w + ((size_t)rt * p.kgroups + (size_t)chunk * R_CG) * TB;
        mbar_expect_tx(full0 + 8 * slot, cg * TB);
        for (int g0 = 0; g0 < cg; g0 += 4) {
          const int gn = min(4, cg - g0);
          bulk_g2s(smem_u32(ring + slot * STAGE + g0 * TB), src + (size_t)g0 * TB, gn * TB, full0 + 8 * slot);
        }
      }
      if (!rec_issued) fetch_record();
      for (int j = max(0, it - R_NS); j < it; j++) mbar_wait(full0 + 8 * (j % R_NS), (j / R_NS) & 1);      // nothing may still be landing at exit
      mbar_wait(rbar, 0);
#ifdef B200Q_ROWS_PROF
      RSTAMP(6, (unsigned long long)p_wait);
#endif
    } else {
      pdl_wait();
    }
    return;
  }
  if (warp > R_WARPS) {
    // -------------------------------- finishers: the cross-warp sum (fixed order) and the epilogue of every row tile, off the consumers' path
    const int fw = warp - R_WARPS - 1;
    pdl_wait();
    int it = 0;
    for (int rt = blockIdx.x; rt < p.n_row_tiles; rt += gridDim.x, it++) {
      const int par = it & 1;
      if (!mbar_wait(rfull0 + 8 * par, (it >> 1) & 1)) { *s_abort = 1; break; }
      const float* rb = red + par * R_WARPS * 128;
      const int o = fw * 32 + lane;                              // output o of the tile: lane' = o / 4, i = o % 4
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < R_WARPS; w++) v += rb[w * 128 + o];
      __syncwarp();
      if (lane == 0) mbar_arrive(rempty0 + 8 * par);             // the buffer may be written again (by the tile after next)
      const int ln = o >> 2, i = o & 3, row = rt * 16 + (ln >> 2) + (i >> 1) * 8, tok = 2 * (ln & 3) + (i & 1);
      if (p.n_chunks > 1) {
        if (row < p.n_out && tok < p.m) p.part[((size_t)chunk * p.m + tok) * p.n_out + row] = v;
      } else if (p.silu_mul) {                                   // rows g / g + 8 of a tile are a gate row and its up row: i and i + 2 of one quad
        const float up = __shfl_down_sync(0xffffffffu, v, 2);
        if (i < 2 && row < p.n_out && tok < p.m) {
          const size_t at = (size_t)tok * (p.n_out >> 1) + rt * 8 + (ln >> 2);
          const float r = (v / (1.f + expf(-v))) * up;
          if (p.y_f16) reinterpret_cast<__half*>(p.y)[at] = __float2half_rn(r); else reinterpret_cast<float*>(p.y)[at] = r;
        }
      } else if (row < p.n_out && tok < p.m) {
        const size_t at = (size_t)tok * p.n_out + row;
        if (p.bias) v += __half2float(p.bias[row]);
        if (p.residual) v += p.y_f16 ? __half2float(reinterpret_cast<const __half*>(p.residual)[at]) : reinterpret_cast<const float*>(p.residual)[at];
        if (p.y_f16) reinterpret_cast<__half*>(p.y)[at] = __float2half_rn(v); else reinterpret_cast<float*>(p.y)[at] = v;
      }
    }
    return;
  }
  // -------------------------------- consumers
  pdl_wait();
  const int g = lane >> 2, t = lane & 3;
#ifdef B200Q_ROWS_PROF
  long long c_wait = 0, c_mac = 0, c_red = 0;
  if (warp == 0) RSTAMP(0, gtime());
#endif
  if (!mbar_wait(rbar, 0)) *s_abort = 1;
  rows_bar_sync();
#ifdef B200Q_ROWS_PROF
  if (warp == 0) RSTAMP(1, gtime());
#endif
  bool live = *s_abort == 0;
  const uint4* recw = reinterpret_cast<const uint4*>(rec);
  const float4* recs = reinterpret_cast<const float4*>(rec + (size_t)cg * REC_GROUP);
  int it = 0, par = 0;
  for (int rt = blockIdx.x; rt < p.n_row_tiles && live; rt += gridDim.x, it++, par ^= 1) {
    const int slot = it % R_NS;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#ifdef B200Q_ROWS_PROF
    const long long k0 = clock64();
#endif
    const bool arrived = mbar_wait(full0 + 8 * slot, (it / R_NS) & 1);
#ifdef B200Q_ROWS_PROF
    const long long k1 = clock64();
#endif
    if (!arrived) { *s_abort = 1; }
    else {
      const uint8_t* stage = ring + slot * STAGE;
#pragma unroll
      for (int u = 0; u < (R_CG + R_WARPS - 1) / R_WARPS; u++) {
        const int jj = warp + u * R_WARPS;
        if (jj < cg) {
          uint4 xw[4];
          float4 xs[4];
#pragma unroll
          for (int i = 0; i < 4; i++) xw[i] = recw[(jj * 4 + i) * 32 + lane];      // block i: 32 consecutive 16-byte words, no bank conflict
          // scales of activation rows 2t and 2t + 1: [row][block]{s, o} = 8 floats per row
          const float4* sc = recs + (size_t)jj * (SC_GROUP / 16);
          xs[0] = sc[(2 * t) * 2]; xs[1] = sc[(2 * t) * 2 + 1]; xs[2] = sc[(2 * t + 1) * 2]; xs[3] = sc[(2 * t + 1) * 2 + 1];
          tile_mac_rows<QT>(stage + jj * TB, lane, xw, xs, acc);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * slot);
    }
#ifdef B200Q_ROWS_PROF
    const long long k2 = clock64();
#endif
    // partial sums to the finishers: rb[warp][lane * 4 + i] in buffer it & 1, free again once tile it - 2 has been summed
    if (it >= 2 && !mbar_wait(rempty0 + 8 * par, ((it >> 1) - 1) & 1)) *s_abort = 1;
    live = *s_abort == 0;
    if (!live) break;
    float* rb = red + par * R_WARPS * 128;
    *reinterpret_cast<float4*>(rb + warp * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncwarp();
    if (lane == 0) mbar_arrive(rfull0 + 8 * par);
#ifdef B200Q_ROWS_PROF
    c_wait += k1 - k0; c_mac += k2 - k1; c_red += clock64() - k2;
#endif
  }
#ifdef B200Q_ROWS_PROF
  if (warp == 0) { RSTAMP(2, gtime()); RSTAMP(3, (unsigned long long)c_wait); RSTAMP(4, (unsigned long long)c_mac); RSTAMP(5, (unsigned long long)c_red); RSTAMP(7, (unsigned long long)it); }
#endif
}

// y = sum over K chunks (fixed order) + bias + residual, or the SwiGLU product of interleaved gate / up columns
__global__ void rows_reduce_kernel(const float* __restrict__ part, int n_chunks, int m, int n_out, const __half* __restrict__ bias,
                                   const void* __restrict__ residual, void* __restrict__ y, int y_f16, int silu_mul) {
  pdl_wait();
  const int n_y = silu_mul ? n_out / 2 : n_out;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)m * n_y) return;
  const int row = (int)(i / n_y), c = (int)(i - (size_t)row * n_y);
  auto total = [&](int col) { float s = 0.f; for (int z = 0; z < n_chunks; z++) s += part[((size_t)z * m + row) * n_out + col]; return s; };
  float o;
  if (silu_mul) {
    const int col = (c >> 3) * 16 + (c & 7);                     // 8 gate rows then 8 up rows per 16-row tile
    const float gte = total(col), up = total(col + 8);
    o = (gte / (1.f + expf(-gte))) * up;
  } else {
    o = total(c);
    if (bias) o += __half2float(bias[c]);
    if (residual) o += y_f16 ? __half2float(reinterpret_cast<const __half*>(residual)[i]) : reinterpret_cast<const float*>(residual)[i];
  }
  if (y_f16) reinterpret_cast<__half*>(y)[i] = __float2half_rn(o); else reinterpret_cast<float*>(y)[i] = o;
}

size_t rows_smem(int qtype) {
  return (size_t)rows_ns(qtype) * R_CG * tile_bytes(qtype) + (size_t)R_CG * (REC_GROUP + SC_GROUP) + 2 * R_WARPS * 128 * sizeof(float) + (2 * rows_ns(qtype) + 5) * sizeof(uint64_t) + 16;
}
size_t rows_record_bytes(int kgroups) { return (size_t)ceil_div(kgroups, R_CG) * R_CG * (REC_GROUP + SC_GROUP); }

}  // namespace

#ifdef B200Q_ROWS_PROF
extern "C" int b200q_rows_prof_read(unsigned long long* out, int n_ctas) {
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_rows_prof, sizeof(unsigned long long) * 8 * (n_ctas < 1024 ? n_ctas : 1024)));
  return B200Q_OK;
}
#endif

extern "C" size_t b200q_qgemv_rows_workspace_bytes(int m, int n_out, int n_in) {
  if (m <= 0 || n_out <= 0 || n_in <= 0) return 0;
  const int kgroups = ceil_div(n_in, GROUP_ELEMS), passes = ceil_div(m, R_TOK);
  return rows_record_bytes(kgroups) + (size_t)ceil_div(kgroups, R_CG) * (size_t)(passes > 1 ? R_TOK : m) * n_out * sizeof(float);
}

extern "C" int b200q_qgemv_rows_norm(int qtype, const void* w_packed, const void* x, int x_dtype, const void* norm_weight_f16, float norm_eps, const void* bias_f16,
                                     const void* residual, int epilogue, void* y, int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes,
                                     void* stream) {
  if (!w_packed || !x || !y || !workspace || m <= 0 || n_out <= 0 || n_in <= 0) return B200Q_ERR_BAD_ARG;
  if (qtype == B200Q_Q6_K) return B200Q_ERR_UNSUPPORTED;
  if (qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0) return B200Q_ERR_BAD_ARG;
  if ((x_dtype != B200Q_F32 && x_dtype != B200Q_F16) || (y_dtype != B200Q_F32 && y_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (epilogue != B200Q_EPI_LINEAR && epilogue != B200Q_EPI_SILU_MUL) return B200Q_ERR_BAD_ARG;
  if (epilogue == B200Q_EPI_SILU_MUL && (bias_f16 || residual || n_out % 16)) return B200Q_ERR_BAD_ARG;
  if (norm_weight_f16 && (x_dtype != B200Q_F32 || n_in % 4)) return B200Q_ERR_BAD_ARG;
  if (n_in % 32) return B200Q_ERR_BAD_SHAPE;
  if (((uintptr_t)w_packed | (uintptr_t)x | (uintptr_t)workspace) & 15) return B200Q_ERR_MISALIGNED;
  if (workspace_bytes < b200q_qgemv_rows_workspace_bytes(m, n_out, n_in)) return B200Q_ERR_TOO_LARGE;
  const int n_sm = b200q_sm_count(), dev = b200q_current_device();
  if (n_sm <= 0 || dev < 0) return B200Q_ERR_CUDA;
  static PerDeviceFlag attr;
  if (!attr.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(qgemv_rows_kernel<B200Q_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rows_smem(B200Q_Q4_0)));
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(qgemv_rows_kernel<B200Q_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rows_smem(B200Q_Q8_0)));
    attr.set(dev);
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int kgroups = ceil_div(n_in, GROUP_ELEMS), n_chunks = ceil_div(kgroups, R_CG), n_row_tiles = ceil_div(n_out, TILE_ROWS);
  unsigned char* record = (unsigned char*)workspace;
  float* part = reinterpret_cast<float*>(record + rows_record_bytes(kgroups));
  const size_t esz = x_dtype == B200Q_F16 ? 2 : 4, ysz = y_dtype == B200Q_F16 ? 2 : 4;
  const int n_y = epilogue == B200Q_EPI_SILU_MUL ? n_out / 2 : n_out;
  for (int r0 = 0; r0 < m; r0 += R_TOK) {                        // 8 activation rows per pass over the weights
    const int mm = min(R_TOK, m - r0);
    const unsigned char* xr = (const unsigned char*)x + (size_t)r0 * n_in * esz;
    const dim3 rec_grid(R_TOK * ceil_div(kgroups * 4, 8));
    if (x_dtype == B200Q_F16)
      B200Q_CHECK_CUDA(launch_k(rows_record_kernel<__half>, rec_grid, dim3(256), (size_t)0, st, true, (const __half*)xr, mm, n_in, kgroups, record, (const __half*)nullptr, 0.f));
    else
      B200Q_CHECK_CUDA(launch_k(rows_record_kernel<float>, rec_grid, dim3(256), (size_t)0, st, true, (const float*)xr, mm, n_in, kgroups, record,
                                (const __half*)norm_weight_f16, norm_eps));
    const unsigned char* res = residual ? (const unsigned char*)residual + (size_t)r0 * n_out * ysz : nullptr;
    void* yr = (void*)((unsigned char*)y + (size_t)r0 * n_y * ysz);
    RowsParams p;
    p.w = (const uint8_t*)w_packed; p.record = record; p.part = part; p.m = mm; p.n_out = n_out; p.kgroups = kgroups; p.n_row_tiles = n_row_tiles;
    p.n_chunks = n_chunks;
    p.bias = (const __half*)bias_f16; p.residual = res; p.y = yr; p.y_f16 = y_dtype == B200Q_F16; p.silu_mul = epilogue == B200Q_EPI_SILU_MUL;
    int gx = n_sm / n_chunks; if (gx < 1) gx = 1; if (gx > n_row_tiles) gx = n_row_tiles;
    const dim3 grid(gx, n_chunks);
    const size_t smem = rows_smem(qtype);
    if (qtype == B200Q_Q4_0) B200Q_CHECK_CUDA(launch_k(qgemv_rows_kernel<B200Q_Q4_0>, grid, dim3(R_THREADS), smem, st, true, p));
    else B200Q_CHECK_CUDA(launch_k(qgemv_rows_kernel<B200Q_Q8_0>, grid, dim3(R_THREADS), smem, st, true, p));
    if (n_chunks > 1) {
      const size_t total = (size_t)mm * n_y;
      B200Q_CHECK_CUDA(launch_k(rows_reduce_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), (size_t)0, st, true, (const float*)part, n_chunks, mm, n_out,
                                (const __half*)bias_f16, (const void*)res, yr, (int)(y_dtype == B200Q_F16), (int)(epilogue == B200Q_EPI_SILU_MUL)));
    }
  }
  return B200Q_OK;
}

extern "C" int b200q_qgemv_rows(int qtype, const void* w_packed, const void* x, int x_dtype, const void* bias_f16, const void* residual, int epilogue,
                                void* y, int y_dtype, int m, int n_out, int n_in, void* workspace, size_t workspace_bytes, void* stream) {
  return b200q_qgemv_rows_norm(qtype, w_packed, x, x_dtype, nullptr, 0.f, bias_f16, residual, epilogue, y, y_dtype, m, n_out, n_in, workspace, workspace_bytes, stream);
}
