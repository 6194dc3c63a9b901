// One decode step of a dense GGUF-quantised Transformer as ONE persistent kernel.
//
// Replaces the reference's captured decode graph (tinygrad/llm/model.py:358-364 forward for T == 1, replayed by
// TinyJit -> CUDAGraph, tinygrad/engine/jit.py:241-291): embedding, per block norm + QKV, RoPE + KV append + GQA attention,
// O + residual, norm + gate/up + SwiGLU, down + residual, then final norm, vocabulary head and greedy sample.
//
// Why one kernel: at batch 1 a step streams every weight byte once (HBM-bound) through ~160 dependent stages.  As separate
// launches each stage pays launch + drain + refill, and the weight stream stops at every boundary.  Here one cooperative grid
// (one CTA of 32 warps per SM) walks the stages itself:
//  * every Linear is cut "stream-K" style: its packed weight tiles (16 rows x 128 columns, stored [row tile][column group])
//    are dealt to the CTAs as equal CONTIGUOUS byte ranges, and inside a CTA to its 32 warps as contiguous runs.  A warp streams
//    its run through a private ring of bulk-async copies (cp.async.bulk + mbarrier) and never synchronises with other warps
//    while it multiplies; since weights do not depend on activations, its copies run ahead across stage boundaries, so HBM
//    keeps streaming while the grid synchronises and stages the next activation vector;
//  * partial sums of a row tile meet in shared memory (fixed order), row tiles cut by a CTA boundary are finished by the CTA
//    that holds their first tile (the other side leaves its partial in global memory behind a flag): results are bit-reproducible;
//  * stages are separated by a grid barrier (one atomic counter, bounded spin); attention runs between the QKV and O stages on
//    (KV head, 64-position slice) units, the cache rows of a unit fetched into shared memory before the barrier is awaited.
// The tile arithmetic is the per-launch GEMV's (qgemv_core.cuh): 15-bit quantised activations, exact int8 tensor-core block
// sums, fp32 accumulation across blocks.
// Every wait is bounded; on expiry the kernel raises the status word, tells the other CTAs through an abort word, drains its
// copies and returns.
#include "common.cuh"
#include "actquant.cuh"
#include "qgemv_core.cuh"
#include <math.h>

namespace {

constexpr int DS_WARPS = 32, DS_THREADS = DS_WARPS * 32;
constexpr int DS_MAXT = 4;            // row tiles the run of one warp may touch
constexpr int DS_MAX_TILES = 512;     // row tiles the range of one CTA may touch (finished 64 at a time, one thread per (tile, row))
constexpr int DS_CHUNK = 64;          // positions per attention unit
constexpr int DS_MAX_REP = 8;         // query heads per KV head
constexpr int DS_MAX_DEPTH = 4;       // ring slots per warp
constexpr int DS_SMEM_BUDGET = 226 * 1024;   // dynamic shared memory: the 227 KB a CTA can opt into, less the kernel's static variables
constexpr int DS_GRID_SPIN = 1 << 21; // polls of a grid-level wait before it gives up (each poll is an L2 round trip)

struct DsParams {
  const b200q_decode_layer* layers;
  int n_layers, dim, hidden, n_heads, n_kv, hd, rope_dim, max_ctx, vocab, embd_vocab;
  int q_dim, kv_dim, qkv_rows, n_rep, n_split, wph;
  float eps;
  const __half* embd; const __half* out_norm; const uint8_t* out_w;
  const float* rope;
  int32_t* tokens; int32_t* pos;
  float *x, *qkv, *attn, *act, *logits;
  unsigned* ctrl;          // [0] grid-barrier counter, [1] its value while the grid is idle, [2] abort, [3] flag sequence base
  float* part;             // [row tile][maxc][16] partial sums of row tiles cut by a CTA boundary
  unsigned* pflag;         // [row tile][maxc]     sequence number of the stage whose partial sits there
  int maxc;
  float* attn_part;        // [n_heads][n_split][hd + 4]
  unsigned* attn_cnt;      // [n_kv]
  float* cand_val; int* cand_idx;    // [grid] arg-max candidates
  int with_head, depth;
  int rec_off, attn_off, wred_off, misc_off;     // shared-memory plan (bytes)
  unsigned long long* prof; int prof_n;          // optional: [grid][prof_n] nanosecond stamps of thread 0 at the stage boundaries
};

enum { K_QKV = 0, K_O = 1, K_GU = 2, K_DOWN = 3, K_HEAD = 4 };

struct Stage { const uint8_t* w; int kind, n_out, n_in, KG, R, A; };

__device__ __forceinline__ Stage stage_of(const DsParams& p, int ph) {
  Stage s;
  const int l = ph >> 2;
  s.kind = l < p.n_layers ? (ph & 3) : K_HEAD;
  if (s.kind == K_HEAD) { s.w = p.out_w; s.n_out = p.vocab; s.n_in = p.dim; }
  else {
    const b200q_decode_layer& L = p.layers[l];
    if (s.kind == K_QKV) { s.w = (const uint8_t*)L.qkv; s.n_out = p.qkv_rows; s.n_in = p.dim; }
    else if (s.kind == K_O) { s.w = (const uint8_t*)L.attn_output; s.n_out = p.dim; s.n_in = p.q_dim; }
    else if (s.kind == K_GU) { s.w = (const uint8_t*)L.gate_up; s.n_out = p.hidden; s.n_in = p.dim; }
    else { s.w = (const uint8_t*)L.ffn_down; s.n_out = p.dim; s.n_in = p.hidden; }
  }
  s.KG = (s.n_in + GROUP_ELEMS - 1) / GROUP_ELEMS;
  s.R = s.kind == K_GU ? (s.n_out + 7) / 8 : (s.n_out + TILE_ROWS - 1) / TILE_ROWS;
  s.A = s.R * s.KG;
  return s;
}

// atoms [lo, hi) of part `i` of `n_parts` equal parts of `total`
__device__ __forceinline__ void split_range(int total, int i, int n_parts, int& lo, int& hi) {
  lo = (int)((long long)total * i / n_parts);
  hi = (int)((long long)total * (i + 1) / n_parts);
}

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(unsigned* p, unsigned v) { asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) { asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

// The weight stream of one warp: the atoms of its runs, stage after stage, copied into its ring `depth` slots ahead of use.
struct WStream {
  int ph, a, a_end;          // next atom to issue: stage, index, end of the warp's run in that stage
  const uint8_t* base;       // weights of that stage
  int slot;                  // ring slot the next copy goes to
  int issued;                // copies issued so far
  bool done;
};

template <int QT>
__device__ __forceinline__ void stream_issue(WStream& s, const DsParams& p, int n_ph, int cta, int n_ctas, int warp, int lane, uint32_t ring, uint32_t bars) {
  constexpr int TB = tile_bytes(QT);
  while (!s.done && s.a == s.a_end) {      // this warp's run in the stage is exhausted: go to its run in the next stage
    if (++s.ph >= n_ph) { s.done = true; break; }
    const Stage f = stage_of(p, s.ph);
    int a0, a1, w0, w1;
    split_range(f.A, cta, n_ctas, a0, a1);
    split_range(a1 - a0, warp, DS_WARPS, w0, w1);
    s.a = a0 + w0; s.a_end = a0 + w1; s.base = f.w;
  }
  if (s.done) return;
  if (lane == 0) {
    const uint32_t bar = bars + 8 * s.slot;
    mbar_expect_tx(bar, TB);
    bulk_g2s(ring + s.slot * TB, s.base + (size_t)s.a * TB, TB, bar);
  }
  s.a++; s.issued++;
  if (++s.slot == p.depth) s.slot = 0;
}

// Quantise an activation vector into the record the tile arithmetic reads (actquant.cuh); returns this thread's part of sum(x^2).
// `coherent`: the vector was written by other CTAs of this grid (read it past L1).
template <bool F16>
__device__ __forceinline__ float stage_record(const void* src, int n_in, int kgroups, const __half* norm_w, unsigned char* record, int tid, float* x_copy,
                                              int copy_lo, int copy_hi) {
  constexpr int BSTEP = DS_THREADS / 8;
  const int nblk_pad = kgroups * 4, q = tid & 7;
  const XqDst dst(record, kgroups);
  float ss = 0.f;
  for (int b = tid >> 3; b < nblk_pad; b += BSTEP) {
    const int k = b * 32 + 4 * q;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    uint2 nw = make_uint2(0x3C003C00u, 0x3C003C00u);      // fp16 ones
    if (k < n_in) {
      if (F16) {
        const uint2 r = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(src) + k);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
        v = make_float4(a.x, a.y, c.x, c.y);
        if (x_copy && k >= copy_lo && k < copy_hi) *reinterpret_cast<float4*>(x_copy + k) = v;
      } else {
        v = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + k));
      }
      if (norm_w) nw = *reinterpret_cast<const uint2*>(norm_w + k);
    }
    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&nw.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&nw.y));
    quant_block_8x4(make_float4(v.x * a.x, v.y * a.y, v.z * c.x, v.w * c.y), q, b, dst);
  }
  return ss;
}

template <typename KV> struct KvT;
template <> struct KvT<__half> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ float dot(const __half* k, const float* q) {
    const uint4 r = *reinterpret_cast<const uint4*>(k);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&r.y));
    const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&r.z)), d = __half22float2(*reinterpret_cast<const __half2*>(&r.w));
    return a.x * q[0] + a.y * q[1] + b.x * q[2] + b.y * q[3] + c.x * q[4] + c.y * q[5] + d.x * q[6] + d.y * q[7];
  }
  static __device__ __forceinline__ float get(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ __half cast(float v) { return __float2half_rn(v); }
};
template <> struct KvT<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ float dot(const float* k, const float* q) {
    const float4 r = *reinterpret_cast<const float4*>(k);
    return r.x * q[0] + r.y * q[1] + r.z * q[2] + r.w * q[3];
  }
  static __device__ __forceinline__ float get(const float* p) { return *p; }
  static __device__ __forceinline__ float cast(float v) { return v; }
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// diagnostics: thread 0 of every CTA notes the time at each stage boundary (the host reads them to see where a step's time goes)
#define DS_STAMP() do { if (p.prof && threadIdx.x == 0 && n_stamp < p.prof_n) p.prof[(size_t)blockIdx.x * p.prof_n + n_stamp++] = global_ns(); } while (0)

__device__ __forceinline__ void argmax_combine2(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// Grid barrier: every CTA arrives once; returns false if the wait ran out or another CTA raised the abort word.
__device__ __forceinline__ bool grid_barrier(const DsParams& p, unsigned& target, volatile int* s_abort) {
  __syncthreads();
  if (threadIdx.x == 0) {
    target += gridDim.x;
    __threadfence();
    red_release_add(p.ctrl, 1u);
    bool ok = false;
    for (int i = 0; i < DS_GRID_SPIN; i++) {
      if ((int)(ld_acquire(p.ctrl) - target) >= 0) { ok = true; break; }
      if ((i & 63) == 63 && ld_acquire(p.ctrl + 2) != 0) break;
      if (i > 4096) __nanosleep(64);
    }
    if (!ok) { *s_abort = 1; atomicExch(&g_status, 1); atomicExch(p.ctrl + 2, 1u); }
  }
  __syncthreads();
  return *s_abort == 0;
}

// Cache rows [lo, lo + n_old) of one KV head -> shared memory, asynchronously (one commit group).
template <typename KV>
__device__ __forceinline__ void attn_fetch_rows(const DsParams& p, const b200q_decode_layer& L, int kvh, int lo, int n_old, KV* s_k, KV* s_v, int rstride) {
  constexpr int VEC = KvT<KV>::VEC;
  const KV* kc = reinterpret_cast<const KV*>(L.k_cache) + (size_t)kvh * p.max_ctx * p.hd;
  const KV* vc = reinterpret_cast<const KV*>(L.v_cache) + (size_t)kvh * p.max_ctx * p.hd;
  const int wpr = p.hd / VEC, words = n_old * wpr;
  for (int i = threadIdx.x; i < words; i += DS_THREADS) {
    const int r = i / wpr, cc = (i - r * wpr) * VEC;
    cp_async16(s_k + r * rstride + cc, kc + (size_t)(lo + r) * p.hd + cc);
    cp_async16(s_v + r * rstride + cc, vc + (size_t)(lo + r) * p.hd + cc);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// `v` was written by other CTAs of this grid in the stage before: read it past L1 (an earlier block may have left its old value there)
__device__ __forceinline__ float rope_at(const float* v, const float* rope, int d, int half_r, int rope_dim) {
  if (d < half_r) return __ldcg(v + d) * rope[d] - __ldcg(v + d + half_r) * rope[half_r + d];
  if (d < rope_dim) return __ldcg(v + d) * rope[d - half_r] + __ldcg(v + d - half_r) * rope[d];
  return __ldcg(v + d);
}

// One (KV head, slice) unit of attention for the new token at `pos`.  All 1024 threads take part.
template <typename KV>
__device__ void attention_unit(const DsParams& p, const b200q_decode_layer& L, int pos, int kvh, int slice, int n_slices, bool rows_in_flight,
                               unsigned char* asmem) {
  constexpr int VEC = KvT<KV>::VEC;
  const int hd = p.hd, n_rep = p.n_rep, half_r = p.rope_dim >> 1, rstride = hd + VEC, wph = p.wph, ppw = DS_CHUNK / wph;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  KV* s_k = reinterpret_cast<KV*>(asmem);
  KV* s_v = s_k + DS_CHUNK * rstride;
  float* s_q = reinterpret_cast<float*>(s_v + DS_CHUNK * rstride);      // [n_rep][hd]
  float* s_sc = s_q + n_rep * hd;                                       // [n_rep][64]
  float* s_stat = s_sc + n_rep * DS_CHUNK;                              // [n_rep][2]: max, denominator
  float* s_o = reinterpret_cast<float*>(asmem);                         // [n_rep][wph][hd], over the K rows once the scores are done
  __shared__ int s_last;
  const int lo = slice * DS_CHUNK, n = min(DS_CHUNK, pos + 1 - lo);
  if (!rows_in_flight) attn_fetch_rows<KV>(p, L, kvh, lo, max(0, min(DS_CHUNK, pos - lo)), s_k, s_v, rstride);
  const float* rope = p.rope + (size_t)pos * p.rope_dim;
  for (int i = tid; i < n_rep * hd; i += DS_THREADS) {
    const int r = i / hd, d = i - r * hd;
    s_q[i] = rope_at(p.qkv + (size_t)(kvh * n_rep + r) * hd, rope, d, half_r, p.rope_dim);      // written by this grid's QKV stage, read after the barrier
  }
  if (lo <= pos && pos < lo + DS_CHUNK) {      // this unit owns the new position: append it to the cache and to the slice
    KV* kc = reinterpret_cast<KV*>(L.k_cache) + (size_t)kvh * p.max_ctx * hd;
    KV* vc = reinterpret_cast<KV*>(L.v_cache) + (size_t)kvh * p.max_ctx * hd;
    const float* kq = p.qkv + p.q_dim + (size_t)kvh * hd;
    const float* vq = p.qkv + p.q_dim + p.kv_dim + (size_t)kvh * hd;
    for (int d = tid; d < hd; d += DS_THREADS) {
      const KV kk = KvT<KV>::cast(rope_at(kq, rope, d, half_r, p.rope_dim)), vv = KvT<KV>::cast(__ldcg(vq + d));
      kc[(size_t)pos * hd + d] = kk; vc[(size_t)pos * hd + d] = vv;
      s_k[(pos - lo) * rstride + d] = kk; s_v[(pos - lo) * rstride + d] = vv;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  const int r = warp / wph, sub = warp - r * wph;
  const bool active = r < n_rep;
  const float scale = 1.0f / sqrtf((float)hd);
  if (active) {      // scores: 4 lanes per position, a quarter of the head dims each
    const int part = lane & 3, dq = hd >> 2;
    const float* q = s_q + r * hd + part * dq;
    for (int i0 = sub * ppw; i0 < (sub + 1) * ppw; i0 += 8) {
      const int i = i0 + (lane >> 2);
      float s = 0.f;
      if (i < n) {
        const KV* kr = s_k + i * rstride + part * dq;
        for (int d = 0; d < dq; d += VEC) s += KvT<KV>::dot(kr + d, q + d);
      }
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      if (part == 0 && i < n) s_sc[r * DS_CHUNK + i] = s * scale;
    }
  }
  __syncthreads();
  float mx = -INFINITY, den = 0.f;
  float o[4] = {0.f, 0.f, 0.f, 0.f};
  const int dpl = hd >> 5;                     // head dims per lane (head_dim is a multiple of 32, at most 128)
  if (active) {
    const float* sc = s_sc + r * DS_CHUNK;
    for (int i = lane; i < n; i += 32) mx = fmaxf(mx, sc[i]);
    mx = warp_max(mx);
    for (int i = lane; i < n; i += 32) den += __expf(sc[i] - mx);
    den = warp_sum(den);
    const int i_end = min(n, (sub + 1) * ppw);
    for (int i = sub * ppw; i < i_end; i++) {
      const float pr = __expf(sc[i] - mx);
      const KV* vr = s_v + i * rstride + lane * dpl;
#pragma unroll
      for (int d = 0; d < 4; d++) if (d < dpl) o[d] = fmaf(pr, KvT<KV>::get(vr + d), o[d]);
    }
  }
  __syncthreads();                             // every warp is done with the K rows: their space now takes the partial outputs
  if (active) {
    float* so = s_o + (size_t)(r * wph + sub) * hd + lane * dpl;
#pragma unroll
    for (int d = 0; d < 4; d++) if (d < dpl) so[d] = o[d];
    if (sub == 0 && lane == 0) { s_stat[2 * r] = mx; s_stat[2 * r + 1] = den; }
  }
  __syncthreads();
  const int pstride = hd + 4;
  for (int i = tid; i < n_rep * hd; i += DS_THREADS) {
    const int rr = i / hd, d = i - rr * hd, head = kvh * n_rep + rr;
    float v = 0.f;
    for (int s = 0; s < wph; s++) v += s_o[(size_t)(rr * wph + s) * hd + d];
    if (n_slices == 1) p.attn[(size_t)head * hd + d] = v / s_stat[2 * rr + 1];
    else {
      float* pp = p.attn_part + ((size_t)head * p.n_split + slice) * pstride;
      pp[d] = v;
      if (d == 0) { pp[hd] = s_stat[2 * rr]; pp[hd + 1] = s_stat[2 * rr + 1]; }
    }
  }
  if (n_slices == 1) return;
  // the last unit of this KV head to get here merges the slices
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(&p.attn_cnt[kvh], 1u);
    s_last = (prev == (unsigned)n_slices - 1);
    if (s_last) p.attn_cnt[kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = tid; i < n_rep * hd; i += DS_THREADS) {
    const int rr = i / hd, d = i - rr * hd, head = kvh * n_rep + rr;
    const float* hp = p.attn_part + (size_t)head * p.n_split * pstride;
    float gm = -INFINITY;
    for (int s = 0; s < n_slices; s++) gm = fmaxf(gm, __ldcg(hp + (size_t)s * pstride + hd));
    float dn = 0.f, acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < n_slices; s++) {
      const float w = __expf(__ldcg(hp + (size_t)s * pstride + hd) - gm);
      dn = fmaf(w, __ldcg(hp + (size_t)s * pstride + hd + 1), dn);
      acc = fmaf(w, __ldcg(hp + (size_t)s * pstride + d), acc);
    }
    p.attn[(size_t)head * hd + d] = acc / dn;
  }
}

template <int QT, typename KV>
__global__ void __launch_bounds__(DS_THREADS, 1) decode_step_kernel(const __grid_constant__ DsParams p) {
  constexpr int TB = tile_bytes(QT);
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cta = blockIdx.x, n_ctas = gridDim.x;
  const int g = lane >> 2, t = lane & 3;
  unsigned char* ring = smem + (size_t)warp * p.depth * TB;
  unsigned char* record = smem + p.rec_off;
  unsigned char* asmem = smem + p.attn_off;
  float* wred = reinterpret_cast<float*>(smem + p.wred_off);             // [warp][DS_MAXT][16]
  unsigned char* misc = smem + p.misc_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(misc);                     // [warp][DS_MAX_DEPTH]
  float* ssq = reinterpret_cast<float*>(bars + DS_WARPS * DS_MAX_DEPTH);  // [warp]
  int* wt_first = reinterpret_cast<int*>(ssq + DS_WARPS);                 // [warp] first row tile of the warp's run
  int* wt_n = wt_first + DS_WARPS;                                        // [warp] row tiles it touches
  float* cv = reinterpret_cast<float*>(wt_n + DS_WARPS);                  // [warp] arg-max candidates
  int* ci = reinterpret_cast<int*>(cv + DS_WARPS);
  uint4* zero = reinterpret_cast<uint4*>(ci + DS_WARPS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(zero + 1);
  const uint32_t ring_u = smem_u32(ring), bars_u = smem_u32(bars + warp * DS_MAX_DEPTH);

  if (lane == 0) for (int s = 0; s < p.depth; s++) mbar_init(bars_u + 8 * s, 1);
  if (tid == 0) { *s_abort = 0; *zero = make_uint4(0, 0, 0, 0); }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncthreads();

  const int pos = __ldcg(p.pos);
  if (pos < 0 || pos >= p.max_ctx) {            // no cache row for this position (uniform over the grid): touch nothing
    if (tid == 0 && cta == 0) atomicExch(&g_status, 2);
    return;
  }
  unsigned bar_target = __ldcg(p.ctrl + 1);
  const unsigned seq_base = __ldcg(p.ctrl + 3);
  int tok = __ldcg(p.tokens + pos);
  tok = tok < 0 ? 0 : (tok >= p.embd_vocab ? p.embd_vocab - 1 : tok);
  const int n_ph = 4 * p.n_layers + (p.with_head ? 1 : 0);

  // ---- start the weight stream: `depth` atoms in flight per warp from here on
  WStream ws;
  ws.ph = -1; ws.a = ws.a_end = 0; ws.base = nullptr; ws.slot = 0; ws.issued = 0; ws.done = false;
  for (int s = 0; s < p.depth; s++) stream_issue<QT>(ws, p, n_ph, cta, n_ctas, warp, lane, ring_u, bars_u);
  int c_slot = 0, c_par = 0, consumed = 0;       // consumer side of the ring
  bool live = true;
  int n_stamp = 0;
  DS_STAMP();

  for (int ph = 0; ph < n_ph && live; ph++) {
    const Stage f = stage_of(p, ph);
    const b200q_decode_layer& L = p.layers[f.kind == K_HEAD ? 0 : (ph >> 2)];
    // ---- attention's cache rows of this CTA's first unit: fetched now, used after the next barrier
    const int n_slices = (pos + DS_CHUNK) / DS_CHUNK, n_units = p.n_kv * n_slices;
    constexpr int VEC = KvT<KV>::VEC;
    if (f.kind == K_QKV && cta < n_units) {
      const int kvh = cta / n_slices, slice = cta - kvh * n_slices, lo = slice * DS_CHUNK;
      KV* s_k = reinterpret_cast<KV*>(asmem);
      attn_fetch_rows<KV>(p, L, kvh, lo, max(0, min(DS_CHUNK, pos - lo)), s_k, s_k + DS_CHUNK * (p.hd + VEC), p.hd + VEC);
    }
    // ---- the stage's input vector -> quantised record in shared memory
    float ss = 0.f;
    const __half* norm_w = nullptr;
    if (f.kind == K_QKV) {
      norm_w = (const __half*)L.attn_norm;
      if (ph == 0) {      // the embedding row itself (token_embd(tokens).float(), tinygrad/llm/model.py:359); this CTA also writes its share of x
        int lo, hi; split_range(p.dim / 4, cta, n_ctas, lo, hi);
        ss = stage_record<true>(p.embd + (size_t)tok * p.dim, f.n_in, f.KG, norm_w, record, tid, p.x, 4 * lo, 4 * hi);
      } else ss = stage_record<false>(p.x, f.n_in, f.KG, norm_w, record, tid, nullptr, 0, 0);
    } else if (f.kind == K_O) ss = stage_record<false>(p.attn, f.n_in, f.KG, nullptr, record, tid, nullptr, 0, 0);
    else if (f.kind == K_GU) { norm_w = (const __half*)L.ffn_norm; ss = stage_record<false>(p.x, f.n_in, f.KG, norm_w, record, tid, nullptr, 0, 0); }
    else if (f.kind == K_DOWN) ss = stage_record<false>(p.act, f.n_in, f.KG, nullptr, record, tid, nullptr, 0, 0);
    else { norm_w = p.out_norm; ss = stage_record<false>(p.x, f.n_in, f.KG, norm_w, record, tid, nullptr, 0, 0); }
    if (norm_w) { ss = warp_sum(ss); if (lane == 0) ssq[warp] = ss; }
    // ---- this warp's run of atoms
    int a0, a1, w0, w1;
    split_range(f.A, cta, n_ctas, a0, a1);
    split_range(a1 - a0, warp, DS_WARPS, w0, w1);
    w0 += a0; w1 += a0;
    int rt = w0 / f.KG, j = w0 - rt * f.KG;
    const int rt_first = rt;
    if (lane == 0) { wt_first[warp] = rt_first; wt_n[warp] = w1 > w0 ? (w1 - 1) / f.KG - rt_first + 1 : 0; }
    __syncthreads();                              // record complete
    DS_STAMP();
    float rs = 1.f;
    if (norm_w) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < DS_WARPS; w++) tot += ssq[w];
      rs = rsqrtf(tot / (float)f.n_in + p.eps);
    }
    {
      const uint4* xq = reinterpret_cast<const uint4*>(record);
      const float4* xsc = reinterpret_cast<const float4*>(record + (size_t)f.KG * 256);
      const bool diag = (t == (g & 3));
      float acc0 = 0.f, acc1 = 0.f;
      bool pend = false;
      float* my_red = wred + warp * DS_MAXT * 16;
      for (int a = w0; a < w1; a++) {
        if (!mbar_wait(bars_u + 8 * c_slot, c_par)) { *s_abort = 1; atomicExch(p.ctrl + 2, 1u); break; }
        const uint4* q0 = diag ? xq + (j * 2 + 0) * 8 + g : zero;      // select the address, not the loaded value (no branch around the loads)
        const uint4* q1 = diag ? xq + (j * 2 + 1) * 8 + g : zero;
        const uint4 bq0 = *q0, bq1 = *q1;
        const float4 st = xsc[(j * 2 + (t >> 1)) * 2 + (t & 1)];
        tile_mac<QT>(ring + c_slot * TB, lane, bq0, bq1, st, acc0, acc1);
        pend = true;
        __syncwarp();
        stream_issue<QT>(ws, p, n_ph, cta, n_ctas, warp, lane, ring_u, bars_u);      // refills the slot just read
        consumed++;
        if (++c_slot == p.depth) { c_slot = 0; c_par ^= 1; }
        if (++j == f.KG) {                       // row tile complete for this warp: quad lanes hold the four column pairs
          acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1); acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
          acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
          if (t == 0) { my_red[(rt - rt_first) * 16 + g] = acc0; my_red[(rt - rt_first) * 16 + 8 + g] = acc1; }
          acc0 = acc1 = 0.f; pend = false; j = 0; rt++;
        }
      }
      if (pend) {
        acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1); acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
        acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
        if (t == 0) { my_red[(rt - rt_first) * 16 + g] = acc0; my_red[(rt - rt_first) * 16 + 8 + g] = acc1; }
      }
    }
    __syncthreads();
    DS_STAMP();
    if (*s_abort) { live = false; break; }
    // ---- finish the CTA's row tiles: thread (tile, row), 64 tiles per pass.  Tiles cut by a CTA boundary: the CTA holding the
    // tile's first atom finishes it, the others leave their partial sums in global memory behind a flag.
    {
      const unsigned seq = seq_base + (unsigned)ph + 1u;
      const int T0 = a0 / f.KG, NT = a1 > a0 ? (a1 - 1) / f.KG - T0 + 1 : 0, row = tid & 15;
      float best = -INFINITY; int best_i = 0x7fffffff;
      for (int base = 0; base < NT; base += DS_THREADS / 16) {
        const int lt = base + (tid >> 4), T = T0 + lt;
        const bool mine = lt < NT;
        float v = 0.f;
        if (mine) {
#pragma unroll 8
          for (int w = 0; w < DS_WARPS; w++) {
            const int k = T - wt_first[w];
            if (k >= 0 && k < wt_n[w]) v += wred[(w * DS_MAXT + k) * 16 + row];
          }
        }
        const int first_atom = T * f.KG, last_atom = first_atom + f.KG - 1;
        const bool owner = mine && first_atom >= a0, complete = owner && last_atom < a1;
        const int c_owner = mine && !owner ? (int)((((long long)first_atom + 1) * n_ctas - 1) / f.A) : cta;
        if (mine && !owner) {
          p.part[((size_t)T * p.maxc + (cta - c_owner - 1)) * 16 + row] = v;
          __threadfence();
        }
        __syncwarp();
        if (mine && !owner && row == 0) st_release(p.pflag + (size_t)T * p.maxc + (cta - c_owner - 1), seq);
        if (owner && !complete) {
          const int c_last = (int)((((long long)last_atom + 1) * n_ctas - 1) / f.A);
          for (int k = 0; k < c_last - cta; k++) {
            int o0, o1;
            split_range(f.A, cta + 1 + k, n_ctas, o0, o1);
            if (o1 == o0) continue;                       // a CTA without atoms in this stage leaves nothing
            const size_t slot = (size_t)T * p.maxc + k;
            bool ok = false;
            for (int i = 0; i < DS_GRID_SPIN; i++) {
              if (ld_acquire(p.pflag + slot) == seq) { ok = true; break; }
              if ((i & 63) == 63 && ld_acquire(p.ctrl + 2) != 0) break;
            }
            if (!ok) { *s_abort = 1; atomicExch(&g_status, 1); atomicExch(p.ctrl + 2, 1u); break; }
            v += __ldcg(p.part + slot * 16 + row);
          }
        }
        v *= rs;
        __syncwarp();
        if (f.kind == K_GU) {
          const float up = __shfl_down_sync(0xffffffffu, v, 8);        // rows 8..15 of a tile are the `up` rows
          const int o_row = T * 8 + row;
          if (owner && row < 8 && o_row < f.n_out) p.act[o_row] = (v / (1.f + __expf(-v))) * up;
        } else if (owner) {
          const int o_row = T * 16 + row;
          if (o_row < f.n_out) {
            if (f.kind == K_QKV) { if (L.qkv_bias) v += __half2float(((const __half*)L.qkv_bias)[o_row]); p.qkv[o_row] = v; }
            else if (f.kind == K_HEAD) { p.logits[o_row] = v; argmax_combine2(best, best_i, v, o_row); }
            else p.x[o_row] = v + __ldcg(p.x + o_row);                  // O and down: residual add in place
          }
        }
      }
      if (f.kind == K_HEAD) {      // this CTA's arg-max candidate (lowest index wins ties)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
          argmax_combine2(best, best_i, ov, oi);
        }
        if (lane == 0) { cv[warp] = best; ci[warp] = best_i; }
        __syncthreads();
        if (tid == 0) {
          for (int w = 1; w < DS_WARPS; w++) argmax_combine2(best, best_i, cv[w], ci[w]);
          p.cand_val[cta] = best; p.cand_idx[cta] = best_i;
        }
      }
    }
    __syncthreads();
    DS_STAMP();
    if (!grid_barrier(p, bar_target, s_abort)) { live = false; break; }
    DS_STAMP();
    // ---- attention between the QKV and the output projection
    if (f.kind == K_QKV) {
      bool first = true;
      for (int u = cta; u < n_units; u += n_ctas, first = false) {
        const int kvh = u / n_slices, slice = u - kvh * n_slices;
        attention_unit<KV>(p, L, pos, kvh, slice, n_slices, first, asmem);
        __syncthreads();
      }
      DS_STAMP();
      if (!grid_barrier(p, bar_target, s_abort)) { live = false; break; }
      DS_STAMP();
    }
  }

  if (live) {
    // ---- greedy sample (tinygrad/llm/model.py:364 at temperature 0) and the state for the next launch
    if (cta == 0) {
      if (p.with_head) {
        float best = -INFINITY; int best_i = 0x7fffffff;
        for (int i = tid; i < n_ctas; i += DS_THREADS) argmax_combine2(best, best_i, __ldcg(p.cand_val + i), __ldcg(p.cand_idx + i));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best, o); const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
          argmax_combine2(best, best_i, ov, oi);
        }
        __syncthreads();
        if (lane == 0) { cv[warp] = best; ci[warp] = best_i; }
        __syncthreads();
        if (tid == 0) {
          for (int w = 1; w < DS_WARPS; w++) argmax_combine2(best, best_i, cv[w], ci[w]);
          p.tokens[pos + 1] = best_i == 0x7fffffff ? 0 : best_i;      // the table has max_context + 1 entries
        }
      }
      if (tid == 0) {
        *p.pos = pos + 1;
        p.ctrl[1] = bar_target;                       // every CTA has passed the last barrier: the counter stands at this value
        p.ctrl[3] = seq_base + (unsigned)n_ph + 1u;
      }
    }
    return;
  }
  // ---- a wait ran out somewhere: nothing may still be landing in this CTA's shared memory when it exits
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  for (int k = consumed; k < ws.issued; k++) {   // the copies issued and not yet consumed sit in the slots from c_slot on
    mbar_wait(bars_u + 8 * c_slot, c_par);
    if (++c_slot == p.depth) { c_slot = 0; c_par ^= 1; }
  }
}

template <int QT, typename KV>
int launch_decode_step(const DsParams& p, int grid, size_t smem, cudaStream_t stream) {
  auto kern = decode_step_kernel<QT, KV>;
  static PerDeviceFlag attr_set;
  const int dev = b200q_current_device();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!attr_set.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DS_SMEM_BUDGET));
    attr_set.set(dev);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(DS_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident at once: they wait on one another
  attr[0].val.cooperative = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  B200Q_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  return B200Q_OK;
}

struct DsPlan { int grid, depth, maxc, r_max, n_split; size_t smem; int rec_off, attn_off, wred_off, misc_off; size_t ws_part, ws_flag, ws_attn, ws_cnt, ws_cand, ws_total; };

// Shape checks and the shared-memory / workspace plan.  Returns B200Q_OK or the reason the whole-step kernel cannot take this model.
int plan_decode_step(const b200q_decode_step_args* a, DsPlan& pl) {
  if (!a || !a->layers || !a->token_embd || !a->output_norm || !a->rope || !a->tokens || !a->pos || !a->x || !a->qkv || !a->attn || !a->act) return B200Q_ERR_BAD_ARG;
  if (a->with_head && (!a->output || !a->logits)) return B200Q_ERR_BAD_ARG;
  if (a->qtype != B200Q_Q4_0 && a->qtype != B200Q_Q8_0) return B200Q_ERR_UNSUPPORTED;
  if (a->kv_dtype != B200Q_F16 && a->kv_dtype != B200Q_F32) return B200Q_ERR_BAD_ARG;
  if (a->n_layers <= 0 || a->dim <= 0 || a->hidden_dim <= 0 || a->n_heads <= 0 || a->n_kv_heads <= 0 || a->vocab <= 0 || a->embd_vocab <= 0 || a->max_context <= 0) return B200Q_ERR_BAD_ARG;
  if (a->n_heads % a->n_kv_heads || a->n_heads / a->n_kv_heads > DS_MAX_REP) return B200Q_ERR_UNSUPPORTED;
  if (a->head_dim % 32 || a->head_dim > 128 || a->head_dim <= 0) return B200Q_ERR_UNSUPPORTED;
  if (a->rope_dim < 0 || a->rope_dim > a->head_dim || a->rope_dim % 2) return B200Q_ERR_BAD_SHAPE;
  if (a->dim % 32 || a->hidden_dim % 32) return B200Q_ERR_BAD_SHAPE;
  const int q_dim = a->n_heads * a->head_dim, kv_dim = a->n_kv_heads * a->head_dim;
  if (q_dim % 16 || kv_dim % 16) return B200Q_ERR_UNSUPPORTED;      // q | k | v are packed back to back in whole row tiles
  const int n_sm = b200q_sm_count();
  if (n_sm <= 0) return B200Q_ERR_CUDA;
  pl.grid = n_sm;
  const int tb = tile_bytes(a->qtype);
  // per stage: atoms per CTA decide how many row tiles a warp / a CTA touches and how many CTAs share a row tile
  const int n_out[5] = {q_dim + 2 * kv_dim, a->dim, a->hidden_dim, a->dim, a->vocab}, n_in[5] = {a->dim, q_dim, a->dim, a->hidden_dim, a->dim};
  pl.maxc = 1; pl.r_max = 1;
  int kg_max = 1;
  for (int k = 0; k < 5; k++) {
    const int KG = ceil_div(n_in[k], GROUP_ELEMS), R = k == K_GU ? ceil_div(n_out[k], 8) : ceil_div(n_out[k], TILE_ROWS);
    const long long A = (long long)R * KG;
    if (A > 0x3fffffff) return B200Q_ERR_TOO_LARGE;
    const int per_cta_max = (int)((A + pl.grid - 1) / pl.grid), per_cta_min = (int)(A / pl.grid);
    const int per_warp_max = ceil_div(per_cta_max, DS_WARPS);
    const int tiles_per_warp = per_warp_max > 0 ? (per_warp_max - 1 + KG - 1) / KG + 1 : 0;
    const int tiles_per_cta = per_cta_max > 0 ? (per_cta_max - 1 + KG - 1) / KG + 1 : 0;
    if (tiles_per_warp > DS_MAXT || tiles_per_cta > DS_MAX_TILES) return B200Q_ERR_UNSUPPORTED;
    (void)per_cta_min;
    long long span = ((long long)KG * pl.grid + A - 1) / A + 1;      // CTAs past the owner that one row tile's atoms can reach (empty ones included)
    if (span > pl.grid - 1) span = pl.grid - 1;
    if ((int)span > pl.maxc) pl.maxc = (int)span;
    if (R > pl.r_max) pl.r_max = R;
    if (KG > kg_max) kg_max = KG;
  }
  pl.n_split = ceil_div(a->max_context, DS_CHUNK);
  const int n_rep = a->n_heads / a->n_kv_heads, esz = a->kv_dtype == B200Q_F16 ? 2 : 4, vec = 16 / esz;
  const size_t rec = ((size_t)kg_max * XQ_GROUP_BYTES + 127) & ~(size_t)127;
  const size_t attn = (((size_t)2 * DS_CHUNK * (a->head_dim + vec) * esz + (size_t)n_rep * (a->head_dim + DS_CHUNK + 2) * sizeof(float)) + 127) & ~(size_t)127;
  const size_t wred = (size_t)DS_WARPS * DS_MAXT * 16 * sizeof(float);
  const size_t misc = (size_t)DS_WARPS * DS_MAX_DEPTH * 8 + 5 * DS_WARPS * 4 + 16 + 16;
  const size_t fixed = rec + attn + wred + misc, budget = DS_SMEM_BUDGET;
  if (fixed + (size_t)2 * DS_WARPS * tb > budget) return B200Q_ERR_TOO_LARGE;
  int depth = (int)((budget - fixed) / ((size_t)DS_WARPS * tb));
  pl.depth = depth > DS_MAX_DEPTH ? DS_MAX_DEPTH : depth;
  const size_t ring = ((size_t)DS_WARPS * pl.depth * tb + 127) & ~(size_t)127;
  pl.rec_off = (int)ring; pl.attn_off = (int)(ring + rec); pl.wred_off = (int)(ring + rec + attn); pl.misc_off = (int)(ring + rec + attn + wred);
  pl.smem = ring + fixed;
  pl.ws_part = 256;
  pl.ws_flag = pl.ws_part + (size_t)pl.r_max * pl.maxc * 16 * sizeof(float);
  pl.ws_attn = (pl.ws_flag + (size_t)pl.r_max * pl.maxc * sizeof(unsigned) + 255) & ~(size_t)255;
  pl.ws_cnt = pl.ws_attn + (size_t)a->n_heads * pl.n_split * (a->head_dim + 4) * sizeof(float);
  pl.ws_cand = (pl.ws_cnt + (size_t)a->n_kv_heads * sizeof(unsigned) + 255) & ~(size_t)255;
  pl.ws_total = pl.ws_cand + (size_t)pl.grid * 8;
  return B200Q_OK;
}

}  // namespace

int b200q_decode_step_status_take(int* status) {
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
  return B200Q_OK;
}

extern "C" size_t b200q_decode_step_workspace_bytes(const b200q_decode_step_args* a) {
  DsPlan pl;
  return plan_decode_step(a, pl) == B200Q_OK ? pl.ws_total : 0;
}

extern "C" int b200q_decode_step_supported(const b200q_decode_step_args* a) {
  DsPlan pl;
  return plan_decode_step(a, pl);
}

extern "C" int b200q_decode_step(const b200q_decode_step_args* a, void* stream) {
  DsPlan pl;
  const int rc = plan_decode_step(a, pl);
  if (rc != B200Q_OK) return rc;
  if (!a->workspace || a->workspace_bytes < pl.ws_total) return B200Q_ERR_BAD_ARG;
  if (((uintptr_t)a->workspace & 255) || ((uintptr_t)a->x | (uintptr_t)a->qkv | (uintptr_t)a->attn | (uintptr_t)a->act | (uintptr_t)a->token_embd) & 15) return B200Q_ERR_MISALIGNED;
  if ((uintptr_t)a->output & 15) return B200Q_ERR_MISALIGNED;
  DsParams p;
  p.layers = a->layers; p.n_layers = a->n_layers; p.dim = a->dim; p.hidden = a->hidden_dim; p.n_heads = a->n_heads; p.n_kv = a->n_kv_heads;
  p.hd = a->head_dim; p.rope_dim = a->rope_dim; p.max_ctx = a->max_context; p.vocab = a->vocab; p.embd_vocab = a->embd_vocab;
  p.q_dim = a->n_heads * a->head_dim; p.kv_dim = a->n_kv_heads * a->head_dim; p.qkv_rows = p.q_dim + 2 * p.kv_dim;
  p.n_rep = a->n_heads / a->n_kv_heads; p.n_split = pl.n_split; p.wph = p.n_rep <= 4 ? 8 : 4;
  p.eps = a->norm_eps; p.embd = (const __half*)a->token_embd; p.out_norm = (const __half*)a->output_norm; p.out_w = (const uint8_t*)a->output;
  p.rope = a->rope; p.tokens = a->tokens; p.pos = a->pos; p.x = a->x; p.qkv = a->qkv; p.attn = a->attn; p.act = a->act; p.logits = a->logits;
  unsigned char* ws = (unsigned char*)a->workspace;
  p.ctrl = (unsigned*)ws; p.part = (float*)(ws + pl.ws_part); p.pflag = (unsigned*)(ws + pl.ws_flag); p.maxc = pl.maxc;
  p.attn_part = (float*)(ws + pl.ws_attn); p.attn_cnt = (unsigned*)(ws + pl.ws_cnt);
  p.cand_val = (float*)(ws + pl.ws_cand); p.cand_idx = (int*)(ws + pl.ws_cand + (size_t)pl.grid * 4);
  p.with_head = a->with_head ? 1 : 0; p.depth = pl.depth;
  p.rec_off = pl.rec_off; p.attn_off = pl.attn_off; p.wred_off = pl.wred_off; p.misc_off = pl.misc_off;
  p.prof = (unsigned long long*)a->profile; p.prof_n = a->profile ? a->profile_stamps : 0;
  const bool f16 = a->kv_dtype == B200Q_F16;
  if (a->qtype == B200Q_Q4_0) return f16 ? launch_decode_step<B200Q_Q4_0, __half>(p, pl.grid, pl.smem, (cudaStream_t)stream)
                                         : launch_decode_step<B200Q_Q4_0, float>(p, pl.grid, pl.smem, (cudaStream_t)stream);
  return f16 ? launch_decode_step<B200Q_Q8_0, __half>(p, pl.grid, pl.smem, (cudaStream_t)stream)
             : launch_decode_step<B200Q_Q8_0, float>(p, pl.grid, pl.smem, (cudaStream_t)stream);
}
