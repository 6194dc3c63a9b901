// Weight-dequant-fused GEMV for GGUF Q4_0 / Q8_0 weights (decode: one activation row per CTA row).
//
// Replaces the kernels tinygrad generates for `Linear.__call__` on a lazily dequantised
// GGUF weight (tinygrad/nn/__init__.py:177 over tinygrad/llm/gguf.py:46,56).
//
// Structure of one CTA (8 consumer warps + 1 producer warp, persistent over row tiles):
//  * producer: one thread streams the CTA's weight tiles HBM -> shared memory with bulk
//    async copies (cp.async.bulk + mbarrier transaction counts) through a ring of stages.
//    Weights do not depend on the previous kernel, so under programmatic dependent launch
//    the ring fills while the previous kernel is still running.
//  * consumers: stage the activation row once (optionally times the RMSNorm weight):
//    every block of 32 activations is quantised to a 15-bit integer with a per-block fp32
//    scale and split into two int8 digits (hi*128 + lo).  The weight nibbles / bytes are
//    unpacked with two logic ops per 8 values and fed to int8 tensor-core MMAs
//    (mma.m16n8k32): the 8 accumulator columns are the tile's 4 quant blocks x {hi, lo}
//    digit (B is block-diagonal), so each block's exact integer dot product lands in its
//    own column and is scaled by (activation scale x fp16 weight scale) afterwards; the
//    Q4_0 offset of 8 is removed with the block's activation sum.  The k-reduction runs
//    inside the MMA, then across the 4 lanes of a quad (warp shuffles), then across warps
//    through shared memory in a fixed order: results are bit-reproducible run to run.
// The kernel is HBM-bound; the tensor core only takes the multiply-adds off the issue slots.
// Every mbarrier wait is bounded: on expiry the kernel raises a status word
// (b200q_status_read_clear) and drains its copies instead of spinning.
#include "common.cuh"
#include "actquant.cuh"
#include "qgemv_core.cuh"

namespace {

struct GemvParams {
  const uint8_t* w;
  const void* x;
  const __half* norm_w;
  const __half* bias;
  const float* residual;
  float residual_scale;
  void* y;
  int n_out, n_in, kgroups, n_row_tiles;
  int x_f16, y_f16, epilogue;
  float eps;
  // activation hand-over between kernels (see actquant.cuh)
  const void* xq_in;        // ready-made record of the input row (then x is not read)
  const float* ss_in;       // partial sums of squares of the input row, for the fused RMSNorm
  int ss_count;
  void* xq_out;             // record of the OUTPUT row for the next GEMV
  const __half* out_norm_w; // multiplied into the output before it is quantised (the next GEMV's norm weight)
  float* ss_out;            // one partial sum of squares per 32 outputs
  int unit, n_units;        // row tiles are dealt to CTAs in runs of `unit` (one run = 32 outputs when xq_out is set without a staging row)
  uint32_t* out_stage;      // xq_out with a staging row: tiles go to CTAs one by one; the CTA of a block's last tile collects the 32 outputs
  // tensor / vocabulary parallel: the output row goes, as self-validating words, into slot `peer_rank` of a mailbox on EVERY rank
  // (peer memory over NVLink; see peer.cu), where a small kernel sums the ranks' slots (all-reduce) or copies them (all-gather)
  uint32_t* peer[B200Q_MAX_PEERS];
  int n_peers, peer_rank;
  int prof_id;              // experiment builds only: the launch's slot in the time-stamp table
};

// Tunables (overridable at compile time for experiments).
#ifndef B200Q_CONS_WARPS
#define B200Q_CONS_WARPS 16
#endif
#ifndef B200Q_STAGE_GROUPS
#define B200Q_STAGE_GROUPS 32
#endif
#ifndef B200Q_NS_Q4
#define B200Q_NS_Q4 2
#endif
#ifndef B200Q_CTAS_PER_SM
#define B200Q_CTAS_PER_SM 2
#endif
constexpr int CONS_WARPS = B200Q_CONS_WARPS;
constexpr int CONS_THREADS = CONS_WARPS * 32;
constexpr int NTHREADS = CONS_THREADS + 64;      // + the producer warp + the finisher warp
constexpr int STAGE_GROUPS = B200Q_STAGE_GROUPS; // weight tiles (16 rows x 128 columns) per ring stage
#ifndef B200Q_COPY_GROUPS
#define B200Q_COPY_GROUPS 4
#endif
constexpr int COPY_GROUPS = B200Q_COPY_GROUPS;   // weight tiles per bulk copy

template <int QT> struct Cfg;      // NS: ring depth, SG: weight tiles per stage, XSUB: bytes per column group of per-sub-block offsets behind the record
template <> struct Cfg<B200Q_Q4_0> { static constexpr int NS = B200Q_NS_Q4, SG = STAGE_GROUPS, XSUB = 0; };   // stage = SG x 1152 B
template <> struct Cfg<B200Q_Q8_0> { static constexpr int NS = 2, SG = STAGE_GROUPS, XSUB = 0; };             // stage = SG x 2176 B
template <> struct Cfg<B200Q_Q6_K> { static constexpr int NS = 3, SG = CONS_WARPS, XSUB = 32; };              // stage = SG x 1696 B

#ifdef B200Q_GEMV_PROF
// experiment build only: per-launch time stamps of CTA 0 (entry, dependency resolved, row staged, first stage landed, tiles done, exit)
__device__ unsigned long long g_gemv_prof[4096 * 8];
__device__ unsigned g_gemv_prof_n;
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define PSTAMP(i) do { if (blockIdx.x == 0 && tid == 0) g_gemv_prof[prof_slot * 8 + (i)] = gtime(); } while (0)
#else
#define PSTAMP(i) do {} while (0)
#endif

// words of the hand-over staging row: relaxed, device scope (they are polled across CTAs)
__device__ __forceinline__ void stage_store(uint32_t* p, uint32_t bits) { asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(bits) : "memory"); }
__device__ __forceinline__ uint32_t stage_load(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void cons_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONS_THREADS) : "memory"); }

// Shared-memory plan (dynamic):
//   ring   [NS][STAGE_GROUPS * tile_bytes]        weight tiles as they sit in HBM
//   xq,xsc the activation record of actquant.cuh  (kgroups * 320 bytes)
//   zero   uint4                                  B operand of the lanes off the diagonal
//   red    [2][CONS_WARPS][16] float              cross-warp partial sums, double-buffered over row tiles
//   ssq    [CONS_WARPS] float
//   ubuf   [32] float                             the 32 finished outputs of a run, before they are quantised for the next GEMV
//   bars   full[NS], empty[NS], xbar, red_full[2], red_empty[2]
//   abort  int                                    set by a warp whose wait ran out; the others leave at their next row tile or wait
// Hands the 32 finished outputs of a run to the next GEMV already quantised (block index = run index).
// Kept out of line: it runs once per 32 outputs and must not weigh on the register budget of the MMA loop.
__device__ __noinline__ void emit_output_record(const GemvParams& p, const float* ubuf, int unit, int lane) {
  const float u = ubuf[lane];
  if (p.ss_out) {
    const float s2 = warp_sum(u * u);
    if (lane == 0) p.ss_out[unit] = s2;
  }
  const float uq = p.out_norm_w ? u * __half2float(p.out_norm_w[unit * 32 + lane]) : u;
  quant_block_32x1(uq, lane, unit, XqDst(p.xq_out, p.n_out / GROUP_ELEMS));
}

// The count a finisher made for block `pend_blk` one tile ago has come back in lane 0's `pend_prev`: the last of the block's `per`
// tiles collects the 32 words (bounded polling: they were stored before the counts, so they are on their way), leaves the row and
// the counter empty for the next launch and emits the record.
__device__ __noinline__ void settle_handover(const GemvParams& p, float* ubuf, int& pend_blk, unsigned pend_prev, int per, int lane) {
  if (pend_blk < 0) return;
  const unsigned prev = __shfl_sync(0xffffffffu, pend_prev, 0);
  const int blk = pend_blk;
  pend_blk = -1;
  if (prev != (unsigned)per - 1) return;
  uint32_t* word = p.out_stage + (size_t)blk * 32 + lane;
  uint32_t w = MAILBOX_EMPTY;
  for (int i = 0; i < SPIN_LIMIT; i++) {
    w = stage_load(word);
    if (w != MAILBOX_EMPTY) break;
    if (i > 64) __nanosleep(64);
  }
  const bool all = __all_sync(0xffffffffu, w != MAILBOX_EMPTY);
  if (w != MAILBOX_EMPTY) stage_store(word, MAILBOX_EMPTY);
  if (lane == 0) p.out_stage[p.n_out + blk] = 0;
  if (!all) { if (lane == 0) atomicExch(&g_status, 1); return; }
  ubuf[lane] = __uint_as_float(w);
  __syncwarp();
  emit_output_record(p, ubuf, blk, lane);
  __syncwarp();
}

// XQ_IN / XQ_OUT: compiled-in use of a ready-made input record / production of an output record.
template <int QT, bool XQ_IN, bool XQ_OUT>
__global__ void __launch_bounds__(NTHREADS, B200Q_CTAS_PER_SM) qgemv_kernel(const GemvParams p) {
  constexpr int NS = Cfg<QT>::NS, SG = Cfg<QT>::SG, XSUB = Cfg<QT>::XSUB, TB = tile_bytes(QT), STAGE_BYTES = SG * TB;
  static_assert(!(XQ_IN && XSUB), "a ready-made record carries no per-sub-block sums");
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* ring = smem;
  unsigned char* record = smem + NS * STAGE_BYTES;
  const uint4* xq = reinterpret_cast<const uint4*>(record);
  const float4* xsc = reinterpret_cast<const float4*>(record + (size_t)p.kgroups * 256);
  float* sub16 = reinterpret_cast<float*>(record + (size_t)p.kgroups * XQ_GROUP_BYTES);        // [kgroups][4 blocks][2 halves], Q6_K only
  uint4* zero = reinterpret_cast<uint4*>(record + (size_t)p.kgroups * (XQ_GROUP_BYTES + XSUB));
  float* red = reinterpret_cast<float*>(zero + 1);
  float* ssq = red + 2 * CONS_WARPS * 16;
  float* ubuf = ssq + CONS_WARPS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ubuf + 32);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 2 * NS + 5);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + NS), xbar = smem_u32(bars + 2 * NS);
  const uint32_t rfull0 = smem_u32(bars + 2 * NS + 1), rempty0 = smem_u32(bars + 2 * NS + 3);      // the two buffers of `red`
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int m = blockIdx.y;
  const int stages_per_tile = (p.kgroups + SG - 1) / SG;
#ifdef B200Q_GEMV_PROF
  __shared__ unsigned s_prof_slot;
  if (tid == 0) {
    s_prof_slot = (unsigned)p.prof_id & 4095u;
    if (blockIdx.x == 0) {
      g_gemv_prof[s_prof_slot * 8 + 6] = ((unsigned long long)p.n_out << 32) | (unsigned)p.n_in;
      g_gemv_prof[s_prof_slot * 8 + 0] = gtime();
    }
  }
#endif

  if (tid == 0) {
    for (int s = 0; s < NS; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, CONS_WARPS); }
    mbar_init(xbar, 1);
    for (int b = 0; b < 2; b++) { mbar_init(rfull0 + 8 * b, CONS_WARPS); mbar_init(rempty0 + 8 * b, 1); }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
#ifdef B200Q_GEMV_PROF
  const unsigned prof_slot = s_prof_slot;
#endif
  pdl_launch_dependents();

  if (warp == CONS_WARPS) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      int it = 0;
      bool ok = true, x_issued = false;
      // The first NS fills need no consumer.  After them the consumers must be running, and they start only when the
      // previous kernel has finished: wait for it outside the bounded waits, then fetch the activation record it left.
      auto after_prefetch = [&]() {
        pdl_wait();
        if (XQ_IN) {
          // the record in pieces on one barrier: a single bulk copy is served slowly, several overlap
          const uint32_t bytes = (uint32_t)p.kgroups * XQ_GROUP_BYTES, piece = 8 * XQ_GROUP_BYTES;
          mbar_expect_tx(xbar, bytes);
          for (uint32_t o = 0; o < bytes; o += piece)
            bulk_g2s(smem_u32(record) + o, reinterpret_cast<const unsigned char*>(p.xq_in) + o, min(piece, bytes - o), xbar);
        }
        x_issued = true;
      };
      const int run = XQ_OUT ? p.unit : 1;
      for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x) {
        for (int ti = 0; ti < run && ok; ti++) {
          const int rt = unit * run + ti;
          if (rt >= p.n_row_tiles) break;
          const uint8_t* src = p.w + (size_t)rt * p.kgroups * TB;
          for (int s = 0; s < stages_per_tile; s++, it++) {
            const int slot = it % NS, groups = min(SG, p.kgroups - s * SG);
            if (it == NS && !x_issued) after_prefetch();
            if (!mbar_wait(empty0 + 8 * slot, ((it / NS) & 1) ^ 1)) { ok = false; break; }
            mbar_expect_tx(full0 + 8 * slot, groups * TB);
            // one stage = several bulk copies on the same barrier: a single copy is served slowly, several overlap
            for (int g0 = 0; g0 < groups; g0 += COPY_GROUPS) {
              const int gn = min(COPY_GROUPS, groups - g0);
              bulk_g2s(smem_u32(ring + slot * STAGE_BYTES + g0 * TB), src + (size_t)s * STAGE_BYTES + (size_t)g0 * TB, gn * TB, full0 + 8 * slot);
            }
          }
        }
      }
      if (!x_issued) after_prefetch();
      // nothing may still be landing in this CTA's shared memory when it exits
      for (int j = max(0, it - NS); j < it; j++) mbar_wait(full0 + 8 * (j % NS), (j / NS) & 1);
      if (XQ_IN) mbar_wait(xbar, 0);
    } else {
      pdl_wait();   // keep launch order transitive: this grid is not complete before its predecessor
    }
    return;
  }

  if (warp == CONS_WARPS + 1) {
    // ------------------------------ finisher ------------------------------
    // Takes every row tile's cross-warp sum and epilogue off the consumers: they leave their partial sums in `red` (two buffers,
    // a full / empty barrier pair each) and go on with the next tile; nothing in a tile's MMAs waits for the previous tile's
    // stores, residual loads or hand-over bookkeeping.
    pdl_wait();
    float pre_add = 0.f;
    const int first_rt = blockIdx.x * (XQ_OUT ? p.unit : 1);
    if (lane < 16 && p.epilogue == B200Q_EPI_LINEAR && first_rt * 16 + lane < p.n_out) {      // addends of the first tile: their latency hides behind its MMAs
      if (p.residual) pre_add = p.residual[(size_t)m * p.n_out + first_rt * 16 + lane] * p.residual_scale;
      if (p.bias) pre_add += __half2float(p.bias[first_rt * 16 + lane]);
    }
    float rs = 1.f;
    int n = 0, pend_blk = -1;
    unsigned pend_prev = 0;
    bool ok = true;
    const int run = XQ_OUT ? p.unit : 1;
    for (int unit = blockIdx.x; unit < p.n_units && ok; unit += gridDim.x) {
      for (int ti = 0; ti < run; ti++, n++) {
        const int rt = unit * run + ti;
        if (rt >= p.n_row_tiles) break;
        const int par = n & 1;
        if (!mbar_wait(rfull0 + 8 * par, (n >> 1) & 1)) { *s_abort = 1; ok = false; break; }
        if (n == 0 && p.norm_w) {                                // the consumers left their sums of squares before their first tile
          float tot = 0.f;
#pragma unroll
          for (int w = 0; w < CONS_WARPS; w++) tot += ssq[w];
          rs = rsqrtf(tot / (float)p.n_in + p.eps);
        }
        const float* rb = red + par * CONS_WARPS * 16;
        float v = 0.f;
        if (lane < 16) {
#pragma unroll
          for (int w = 0; w < CONS_WARPS; w++) v += rb[w * 16 + lane];
          v *= rs;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(rempty0 + 8 * par);           // the buffer may be written again (by the tile after next)
        if (p.epilogue == B200Q_EPI_LINEAR) {
          const int row = rt * 16 + lane;
          if (lane < 16 && row < p.n_out) {
            if (rt == first_rt) v += pre_add;
            else {
              if (p.bias) v += __half2float(p.bias[row]);
              if (p.residual) v = fmaf(p.residual[(size_t)m * p.n_out + row], p.residual_scale, v);
            }
            if (p.y) {
              if (p.y_f16) reinterpret_cast<__half*>(p.y)[(size_t)m * p.n_out + row] = __float2half_rn(v);
              else reinterpret_cast<float*>(p.y)[(size_t)m * p.n_out + row] = v;
            }
            if (p.n_peers) {
              const uint32_t bits = mailbox_bits(v);
              for (int d = 0; d < p.n_peers; d++) mailbox_store(p.peer[d] + (size_t)p.peer_rank * p.n_out + row, bits);
            }
          }
          if (XQ_OUT && lane < 16) ubuf[ti * 16 + lane] = v;
        } else {
          const float up = __shfl_down_sync(0xffffffffu, v, 8);     // rows 8..15 of the tile are the `up` rows
          const int row = rt * 8 + lane;
          const float o = (v / (1.f + __expf(-v))) * up;
          if (lane < 8 && row < p.n_out && p.y) {
            if (p.y_f16) reinterpret_cast<__half*>(p.y)[(size_t)m * p.n_out + row] = __float2half_rn(o);
            else reinterpret_cast<float*>(p.y)[(size_t)m * p.n_out + row] = o;
          }
          if (XQ_OUT && lane < 8) ubuf[ti * 8 + lane] = o;
        }
        if (XQ_OUT && p.out_stage) {
          // A block of 32 outputs spans `per` row tiles, which may sit on different CTAs.  Every tile leaves its outputs in the
          // staging row as self-validating words (empty or complete: no flag, no fence) and counts into the block's counter; the
          // one that counts last collects the block and quantises it (the record is a function of the 32 values alone).  The
          // count's answer is looked at one tile later, so its round trip stays off this warp's path, and the collector's wait for
          // words that are still on their way depends on no other CTA's progress.
          const int per = p.epilogue == B200Q_EPI_LINEAR ? 2 : 4, cnt = 32 / per, blk = rt / per, sub = rt - blk * per;
          __syncwarp();
          const float mine = ubuf[lane & 15];                    // ubuf[0 .. cnt) = this tile's outputs
          settle_handover(p, ubuf, pend_blk, pend_prev, per, lane);
          if (lane < cnt) stage_store(p.out_stage + (size_t)blk * 32 + sub * cnt + lane, mailbox_bits(mine));
          if (lane == 0) pend_prev = atomicAdd(p.out_stage + p.n_out + blk, 1u);
          pend_blk = blk;
        } else if (XQ_OUT && ti == run - 1) {
          __syncwarp();
          emit_output_record(p, ubuf, unit, lane);     // the run's 32 outputs are complete
          __syncwarp();
        }
      }
    }
    if (XQ_OUT && p.out_stage) settle_handover(p, ubuf, pend_blk, pend_prev, p.epilogue == B200Q_EPI_LINEAR ? 2 : 4, lane);
#ifdef B200Q_GEMV_PROF
    if (lane == 0) atomicMax(&g_gemv_prof[prof_slot * 8 + 7], gtime());      // the last CTA's exit
#endif
    return;
  }

  // -------------------------------- consumers --------------------------------
  pdl_wait();
  PSTAMP(1);
  const int g = lane >> 2, t = lane & 3;
  if (tid == 0) *zero = make_uint4(0, 0, 0, 0);
  float ss = 0.f;
  if (XQ_IN) {
    // the row arrives quantised (the producer thread copies the record); only the RMSNorm scalar is computed here
    if (p.norm_w) for (int i = tid; i < p.ss_count; i += CONS_THREADS) ss += p.ss_in[i];
  } else {
    // quantise the activation row here: 8 threads per block of 32, 4 elements each.  The loads of PF blocks are issued
    // before any is used, so a batch costs one L2 round trip instead of one per block.
#ifndef B200Q_XPF
#define B200Q_XPF 4
#endif
    constexpr int PF = B200Q_XPF, BSTEP = CONS_THREADS / 8;
    const int nblk_pad = p.kgroups * 4, q = tid & 7;
    const XqDst dst(record, p.kgroups);
    for (int b0 = tid >> 3; b0 < nblk_pad; b0 += PF * BSTEP) {
      float4 v[PF];
      uint2 nw[PF];
#pragma unroll
      for (int u = 0; u < PF; u++) {
        const int k = (b0 + u * BSTEP) * 32 + 4 * q;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        nw[u] = make_uint2(0x3C003C00u, 0x3C003C00u);      // fp16 ones
        if (b0 + u * BSTEP < nblk_pad && k < p.n_in) {
          if (p.x_f16) {
            const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p.x) + (size_t)m * p.n_in + k);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
            v[u] = make_float4(a.x, a.y, c.x, c.y);
          } else {
            v[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + (size_t)m * p.n_in + k);
          }
          if (p.norm_w) nw[u] = *reinterpret_cast<const uint2*>(p.norm_w + k);
        }
      }
#pragma unroll
      for (int u = 0; u < PF; u++) {
        if (b0 + u * BSTEP < nblk_pad) {      // uniform over the 8 lanes of a block (and over the warp: 4 consecutive blocks)
          ss = fmaf(v[u].x, v[u].x, fmaf(v[u].y, v[u].y, fmaf(v[u].z, v[u].z, fmaf(v[u].w, v[u].w, ss))));
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&nw[u].x)), c = __half22float2(*reinterpret_cast<const __half2*>(&nw[u].y));
          quant_block_8x4(make_float4(v[u].x * a.x, v[u].y * a.y, v[u].z * c.x, v[u].w * c.y), q, b0 + u * BSTEP, dst, XSUB ? sub16 : nullptr);
        }
      }
    }
  }
  if (p.norm_w) {
    ss = warp_sum(ss);
    if (lane == 0) ssq[warp] = ss;
  }
  if (XQ_IN && !mbar_wait(xbar, 0)) *s_abort = 1;
  cons_bar_sync();
  PSTAMP(2);
  const bool diag = (t == (g & 3));
  int it = 0, n = 0;
  bool live = *s_abort == 0;
  const int run = XQ_OUT ? p.unit : 1;
  for (int unit = blockIdx.x; unit < p.n_units && live; unit += gridDim.x) {
    for (int ti = 0; ti < run; ti++, n++) {
      const int rt = unit * run + ti;
      if (rt >= p.n_row_tiles) break;
      float acc0 = 0.f, acc1 = 0.f;
      for (int s = 0; s < stages_per_tile; s++, it++) {
        const int slot = it % NS, groups = min(SG, p.kgroups - s * SG);
        if (!mbar_wait(full0 + 8 * slot, (it / NS) & 1)) { *s_abort = 1; break; }
        if (it == 0) PSTAMP(3);
        const uint8_t* stage = ring + slot * STAGE_BYTES;
#pragma unroll
        for (int u = 0; u < SG / CONS_WARPS; u++) {
          const int gi = warp + u * CONS_WARPS;
          if (gi < groups) {
            const int j = s * SG + gi;
            // the address is selected, not the loaded value: `diag ? xq[..] : *zero` compiled to a divergent branch around the loads
            // (5 % of the decode step)
            const uint4* q0 = diag ? xq + (j * 2 + 0) * 8 + g : zero;
            const uint4* q1 = diag ? xq + (j * 2 + 1) * 8 + g : zero;
            const uint4 bq0 = *q0, bq1 = *q1;
            const float4 st = xsc[(j * 2 + (t >> 1)) * 2 + (t & 1)];
            if constexpr (QT == B200Q_Q6_K) {
              // the offsets belong to the high digits only (their columns sit on the lanes t < 2)
              const float4 sub = *(t < 2 ? reinterpret_cast<const float4*>(sub16 + j * 8 + t * 4) : reinterpret_cast<const float4*>(zero));
              tile_mac_q6k(stage + gi * TB, lane, bq0, bq1, st, sub, acc0, acc1);
            } else {
              tile_mac<QT>(stage + gi * TB, lane, bq0, bq1, st, acc0, acc1);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * slot);
      }
      PSTAMP(4);
      // quad lanes hold the columns {blocks 0,1 hi}, {2,3 hi}, {0,1 lo}, {2,3 lo}: add them
      acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1); acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
      acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
      // hand the partial sums to the finisher: buffer n & 1, free again once the finisher has read tile n - 2
      const int par = n & 1;
      if (n >= 2 && !mbar_wait(rempty0 + 8 * par, ((n >> 1) - 1) & 1)) *s_abort = 1;
      live = *s_abort == 0;
      if (!live) break;
      float* rb = red + par * CONS_WARPS * 16;
      if (t == 0) { rb[warp * 16 + g] = acc0; rb[warp * 16 + 8 + g] = acc1; }
      __syncwarp();
      if (lane == 0) mbar_arrive(rfull0 + 8 * par);
    }
  }
  PSTAMP(5);
}

#ifdef B200Q_GEMV_PROF
}  // namespace
extern "C" int b200q_gemv_prof_read(unsigned long long* out, int max_slots, unsigned* n) {
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_gemv_prof, sizeof(unsigned long long) * 8 * (max_slots < 4096 ? max_slots : 4096)));
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(n, g_gemv_prof_n, sizeof(unsigned)));
  return B200Q_OK;
}
extern "C" int b200q_gemv_prof_reset(void) {
  static unsigned long long zeros[4096 * 8];
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_gemv_prof, zeros, sizeof(zeros)));
  return B200Q_OK;
}
int g_gemv_prof_host_counter = 0;
namespace {
#endif

template <int QT, bool XQ_IN, bool XQ_OUT>
int launch_gemv(const b200q_gemv_args* a, const GemvParams& p, cudaStream_t stream) {
  constexpr int NS = Cfg<QT>::NS;
  const size_t smem = (size_t)NS * Cfg<QT>::SG * tile_bytes(QT) + (size_t)p.kgroups * (XQ_GROUP_BYTES + Cfg<QT>::XSUB) + 16 +
                      (2 * CONS_WARPS * 16 + CONS_WARPS + 32) * sizeof(float) + (2 * NS + 5) * sizeof(uint64_t) + 16;
  if (smem > 220 * 1024) return B200Q_ERR_TOO_LARGE;
  auto kern = qgemv_kernel<QT, XQ_IN, XQ_OUT>;
  // per device (and per instantiation): the shared-memory attribute, and the last occupancy answer packed as (smem << 8) | blocks
  static PerDeviceFlag attr_set;
  static std::atomic<long long> occ_cache[B200Q_MAX_DEVICES];
  const int dev = b200q_current_device(), sm_count = b200q_sm_count();
  if (dev < 0 || sm_count <= 0) return B200Q_ERR_CUDA;
  if (!attr_set.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set.set(dev);
  }
  long long oc = occ_cache[dev].load(std::memory_order_relaxed);
  if (oc == 0 || (oc >> 8) != (long long)smem) {
    int occ = 0;
    B200Q_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, NTHREADS, smem));
    if (occ < 1) occ = 1;
    oc = ((long long)smem << 8) | occ;
    occ_cache[dev].store(oc, std::memory_order_relaxed);
  }
  const int max_ctas = a->max_ctas > 0 ? a->max_ctas : (int)(oc & 0xFF) * sm_count;
  int grid_x = p.n_units < max_ctas ? p.n_units : max_ctas;
  // Between one and two units per CTA the fixed deal leaves some CTAs with twice the work of the others: two units for every CTA on
  // fewer CTAs instead (8B QKV, 384 row tiles: 192 CTAs instead of 296 took 4 % off the decode step; with more units per CTA the
  // full grid measured faster than an even deal)
  if (a->max_ctas <= 0 && p.n_units > max_ctas && p.n_units <= 2 * max_ctas) grid_x = (p.n_units + 1) / 2;
#ifdef B200Q_GEMV_PROF
  GemvParams pp = p;
  pp.prof_id = g_gemv_prof_host_counter++;
  B200Q_CHECK_CUDA(launch_k(kern, dim3(grid_x, a->m), dim3(NTHREADS), smem, stream, (a->flags & B200Q_FLAG_PDL) != 0, pp));
  return B200Q_OK;
#endif
  B200Q_CHECK_CUDA(launch_k(kern, dim3(grid_x, a->m), dim3(NTHREADS), smem, stream, (a->flags & B200Q_FLAG_PDL) != 0, p));
  return B200Q_OK;
}

}  // namespace

extern "C" int b200q_status_read_clear(int* status) {
  if (!status) return B200Q_ERR_BAD_ARG;
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
  int dec = 0;
  const int rc = b200q_decode_status_take(&dec);
  if (rc != B200Q_OK) return rc;
  if (dec && !*status) *status = dec;
  int step = 0;
  const int rc2 = b200q_decode_step_status_take(&step);
  if (rc2 != B200Q_OK) return rc2;
  if (step && !*status) *status = step;
  int peer = 0;
  const int rc3 = b200q_peer_status_take(&peer);
  if (rc3 != B200Q_OK) return rc3;
  if (peer && !*status) *status = peer;
  return B200Q_OK;
}

extern "C" size_t b200q_xq_bytes(int n) { return n > 0 ? xq_record_bytes(n) : 0; }

extern "C" int b200q_gemv(const b200q_gemv_args* a, void* stream) {
  if (!a || !a->w_packed || (!a->x && !a->xq_in) || (!a->y && !a->xq_out && !a->n_peers)) return B200Q_ERR_BAD_ARG;
  if (a->qtype != B200Q_Q4_0 && a->qtype != B200Q_Q8_0 && a->qtype != B200Q_Q6_K) return B200Q_ERR_BAD_ARG;
  if (a->n_out <= 0 || a->n_in <= 0 || a->m <= 0 || a->m > 65535) return B200Q_ERR_BAD_ARG;
  if (a->n_in % (a->qtype == B200Q_Q6_K ? 256 : 32)) return B200Q_ERR_BAD_SHAPE;
  // Q6_K: plain linears only, and the kernel quantises the activations itself (it needs sums per 16-element sub-block)
  if (a->qtype == B200Q_Q6_K && (a->epilogue != B200Q_EPI_LINEAR || a->xq_in)) return B200Q_ERR_UNSUPPORTED;
  if ((a->x_dtype != B200Q_F32 && a->x_dtype != B200Q_F16) || (a->y_dtype != B200Q_F32 && a->y_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (a->epilogue != B200Q_EPI_LINEAR && a->epilogue != B200Q_EPI_SILU_MUL) return B200Q_ERR_BAD_ARG;
  if (a->epilogue == B200Q_EPI_SILU_MUL && (a->bias || a->residual)) return B200Q_ERR_UNSUPPORTED;
  if ((uintptr_t)a->w_packed & 15) return B200Q_ERR_MISALIGNED;
  // activation rows are read 4 elements at a time
  if (a->x && ((uintptr_t)a->x & (a->x_dtype == B200Q_F32 ? 15 : 7))) return B200Q_ERR_MISALIGNED;
  if (a->y && ((uintptr_t)a->y & (a->y_dtype == B200Q_F32 ? 3 : 1))) return B200Q_ERR_MISALIGNED;
  if (a->norm_weight && ((uintptr_t)a->norm_weight & 7)) return B200Q_ERR_MISALIGNED;
  if (((uintptr_t)a->xq_in | (uintptr_t)a->xq_out) & 15) return B200Q_ERR_MISALIGNED;
  if ((a->xq_in || a->xq_out) && a->m != 1) return B200Q_ERR_UNSUPPORTED;
  if (a->xq_in && a->norm_weight && (!a->ss_in || a->ss_count <= 0)) return B200Q_ERR_BAD_ARG;   // the norm weight is already inside the record
  if (a->xq_out && a->n_out % GROUP_ELEMS) return B200Q_ERR_BAD_SHAPE;
  if (a->xq_out_stage && (!a->xq_out || ((uintptr_t)a->xq_out_stage & 3))) return B200Q_ERR_BAD_ARG;
  GemvParams p;
  p.w = (const uint8_t*)a->w_packed; p.x = a->x; p.norm_w = (const __half*)a->norm_weight; p.bias = (const __half*)a->bias;
  p.residual = (const float*)a->residual; p.residual_scale = a->residual_scale == 0.f ? 1.f : a->residual_scale; p.y = a->y;
  p.n_out = a->n_out; p.n_in = a->n_in; p.kgroups = ceil_div(a->n_in, GROUP_ELEMS);
  p.n_row_tiles = a->epilogue == B200Q_EPI_SILU_MUL ? ceil_div(a->n_out, 8) : ceil_div(a->n_out, TILE_ROWS);
  p.x_f16 = a->x_dtype == B200Q_F16; p.y_f16 = a->y_dtype == B200Q_F16; p.epilogue = a->epilogue; p.eps = a->norm_eps;
  p.xq_in = a->xq_in; p.ss_in = a->ss_in; p.ss_count = a->ss_count;
  p.xq_out = a->xq_out; p.out_norm_w = (const __half*)a->xq_out_norm_weight; p.ss_out = a->ss_out;
  p.n_peers = 0; p.peer_rank = 0; p.prof_id = 0;
  if (a->n_peers) {
    if (a->n_peers < 0 || a->n_peers > B200Q_MAX_PEERS || a->peer_rank < 0 || a->peer_rank >= a->n_peers || !a->peer_mailboxes) return B200Q_ERR_BAD_ARG;
    if (a->m != 1 || a->epilogue != B200Q_EPI_LINEAR) return B200Q_ERR_UNSUPPORTED;
    for (int d = 0; d < a->n_peers; d++) {
      if (!a->peer_mailboxes[d] || ((uintptr_t)a->peer_mailboxes[d] & 3)) return B200Q_ERR_BAD_ARG;
      p.peer[d] = (uint32_t*)a->peer_mailboxes[d];
    }
    p.n_peers = a->n_peers; p.peer_rank = a->peer_rank;
  }
  p.out_stage = (uint32_t*)a->xq_out_stage;
  p.unit = (a->xq_out && !a->xq_out_stage) ? (a->epilogue == B200Q_EPI_SILU_MUL ? 4 : 2) : 1;
  p.n_units = ceil_div(p.n_row_tiles, p.unit);
  const bool xi = a->xq_in != nullptr, xo = a->xq_out != nullptr;
  if (a->qtype == B200Q_Q4_0) {
    if (xi) return xo ? launch_gemv<B200Q_Q4_0, true, true>(a, p, (cudaStream_t)stream) : launch_gemv<B200Q_Q4_0, true, false>(a, p, (cudaStream_t)stream);
    return xo ? launch_gemv<B200Q_Q4_0, false, true>(a, p, (cudaStream_t)stream) : launch_gemv<B200Q_Q4_0, false, false>(a, p, (cudaStream_t)stream);
  }
  if (a->qtype == B200Q_Q6_K)
    return xo ? launch_gemv<B200Q_Q6_K, false, true>(a, p, (cudaStream_t)stream) : launch_gemv<B200Q_Q6_K, false, false>(a, p, (cudaStream_t)stream);
  if (xi) return xo ? launch_gemv<B200Q_Q8_0, true, true>(a, p, (cudaStream_t)stream) : launch_gemv<B200Q_Q8_0, true, false>(a, p, (cudaStream_t)stream);
  return xo ? launch_gemv<B200Q_Q8_0, false, true>(a, p, (cudaStream_t)stream) : launch_gemv<B200Q_Q8_0, false, false>(a, p, (cudaStream_t)stream);
}
