// The non-GEMV kernels of one decode step: embedding lookup, one-token GQA attention
// with RoPE and KV-cache update, greedy arg-max.  Semantics follow
// tinygrad/llm/model.py:167-198 (attention, T == 1), :29-33 (RoPE), :358-364 (forward).
#include "common.cuh"
#include "actquant.cuh"
#include <math.h>

namespace {

// Sticky status of this file's kernels: 2 = a position outside [0, max_context) reached a kernel, which then skipped
// its work instead of reading or writing past the token table / KV cache.  b200q_status_read_clear reports it.
__device__ int g_decode_status = 0;

// Also leaves, for the first GEMV of the step, the row already multiplied by that GEMV's RMSNorm weight and
// quantised (actquant.cuh), with one partial sum of squares per block of 32.
__global__ void __launch_bounds__(256) embed_kernel(const __half* __restrict__ table, const int32_t* __restrict__ tokens,
                                                    const int32_t* __restrict__ pos, float* __restrict__ x, int dim, int vocab, int max_context,
                                                    void* xq_out, const __half* __restrict__ norm_w, float* ss_out) {
  pdl_launch_dependents();
  pdl_wait();
  int p = *pos;
  if (p < 0 || p > max_context) {      // the token table has max_context + 1 entries
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(&g_decode_status, 2);
    p = p < 0 ? 0 : max_context;       // keep the activations finite; the step's result is flagged invalid
  }
  int tok = tokens[p];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const __half* row = table + (size_t)tok * dim;
  if (!xq_out) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x) x[i] = __half2float(row[i]);
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, kgroups = (dim + GROUP_ELEMS - 1) / GROUP_ELEMS;
  const int wpb = blockDim.x >> 5;
  const XqDst dst(xq_out, kgroups);
  for (int b = blockIdx.x * wpb + warp; b < kgroups * 4; b += gridDim.x * wpb) {      // one warp per block of 32, lane = element
    const int k = b * 32 + lane;
    float v = 0.f;
    if (k < dim) { v = __half2float(row[k]); x[k] = v; }
    if (ss_out && b * 32 < dim) { const float s2 = warp_sum(v * v); if (lane == 0) ss_out[b] = s2; }
    quant_block_32x1((norm_w && k < dim) ? v * __half2float(norm_w[k]) : v, lane, b, dst);
  }
}

__global__ void advance_kernel(int32_t* pos, int max_context) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    const int p = *pos;
    if (p < 0 || p >= max_context) atomicExch(&g_decode_status, 2);
    else *pos = p + 1;
  }
}

// ---------------------------------------------------------------------------
// attention.  grid (n_kv_heads, n_split); split s owns the fixed position range
// [s*ATTN_CHUNK, (s+1)*ATTN_CHUNK); CTAs past the current context leave at once.
// One warp per query head of the KV group.  The CTA first copies its K and V rows to
// shared memory with every thread's loads in flight together (one global latency), then
//   scores: each lane takes whole positions (full head_dim dot against the roped query),
//   values: each lane owns 4 consecutive head dims and walks the positions.
// Scratch layout:
//   float partial[n_heads][n_split][head_dim + 4]   (o[head_dim], running max, denominator, 2 pad)
//   uint  counter[n_kv_heads]                       (arrival count, reset by the last CTA)
constexpr int MAX_HD = 128;
constexpr int MAX_REP = 8;
#ifndef B200Q_ATTN_CHUNK
#define B200Q_ATTN_CHUNK 64
#endif
constexpr int ATTN_CHUNK = B200Q_ATTN_CHUNK;    // positions per CTA

template <typename KV> struct KvIO;
template <> struct KvIO<__half> {
  static constexpr int VEC = 8;   // elements per 16-byte word
  static __device__ __forceinline__ float dot(const __half* k, const float* q) {
    uint4 r = *reinterpret_cast<const uint4*>(k);
    float2 a = __half22float2(*reinterpret_cast<__half2*>(&r.x)), b = __half22float2(*reinterpret_cast<__half2*>(&r.y));
    float2 c = __half22float2(*reinterpret_cast<__half2*>(&r.z)), d = __half22float2(*reinterpret_cast<__half2*>(&r.w));
    return a.x * q[0] + a.y * q[1] + b.x * q[2] + b.y * q[3] + c.x * q[4] + c.y * q[5] + d.x * q[6] + d.y * q[7];
  }
  static __device__ __forceinline__ float4 load4(const __half* p) {
    uint2 r = *reinterpret_cast<const uint2*>(p);
    float2 a = __half22float2(*reinterpret_cast<__half2*>(&r.x)), b = __half22float2(*reinterpret_cast<__half2*>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ __half cast(float v) { return __float2half_rn(v); }
};
template <> struct KvIO<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ float dot(const float* k, const float* q) {
    float4 r = *reinterpret_cast<const float4*>(k);
    return r.x * q[0] + r.y * q[1] + r.z * q[2] + r.w * q[3];
  }
  static __device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ float cast(float v) { return v; }
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}

#ifdef B200Q_GEMV_PROF
__device__ unsigned long long g_attn_prof[4096 * 8];
__device__ unsigned g_attn_prof_n;
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define ASTAMP(i) do { if (threadIdx.x == 0) g_attn_prof[prof_slot * 8 + (i)] = gtime(); } while (0)
#else
#define ASTAMP(i) do {} while (0)
#endif

// Sequence blockIdx.z of a batch in lock-step: element strides between consecutive sequences (all zero for one sequence)
struct SeqStride { size_t qkv, cache, out, scratch_bytes; int pos; };

template <typename KV>
__global__ void __launch_bounds__(MAX_REP * 32) attn_decode_kernel(const b200q_attn_args a_in, const SeqStride sq) {
  constexpr int VEC = KvIO<KV>::VEC;
  b200q_attn_args a = a_in;
  if (blockIdx.z) {
    const size_t z = blockIdx.z;
    a.qkv += z * sq.qkv; a.out += z * sq.out; a.pos += z * sq.pos;
    a.k_cache = reinterpret_cast<KV*>(a.k_cache) + z * sq.cache; a.v_cache = reinterpret_cast<KV*>(a.v_cache) + z * sq.cache;
    a.scratch = reinterpret_cast<unsigned char*>(a.scratch) + z * sq.scratch_bytes;
  }
  extern __shared__ __align__(16) unsigned char asmem[];
  const int hd = a.head_dim, n_rep = a.n_heads / a.n_kv_heads, half_r = a.rope_dim >> 1;
  const int rstride = hd + VEC;                           // padded row: lanes reading different rows hit different banks
  KV* s_k = reinterpret_cast<KV*>(asmem);                 // [ATTN_CHUNK][rstride]
  KV* s_v = s_k + ATTN_CHUNK * rstride;                   // [ATTN_CHUNK][rstride]
  float* s_q = reinterpret_cast<float*>(s_v + ATTN_CHUNK * rstride);   // [n_rep][hd] roped queries
  float* s_sc = s_q + n_rep * hd;                         // [n_rep][ATTN_CHUNK] scores, then probabilities
  float* s_part = s_sc + n_rep * ATTN_CHUNK;              // [n_rep][hd + 4] what a head's second warp hands to its first (rows stay 16-byte aligned)
  __shared__ int s_last;
  const int kvh = blockIdx.x, split = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#ifdef B200Q_GEMV_PROF
  __shared__ unsigned s_prof_slot;
  if (threadIdx.x == 0) {
    s_prof_slot = (unsigned)a.flags >> 16;           // experiment builds: the host puts the launch's slot into the upper half of flags
    if (blockIdx.x == 0 && blockIdx.y == 0) g_attn_prof[s_prof_slot * 8 + 0] = gtime();
  }
  __syncthreads();
  const unsigned prof_slot = s_prof_slot;
  const bool prof_cta = blockIdx.x == 0 && blockIdx.y == 0;
#endif
  pdl_launch_dependents();
  const int lo = split * ATTN_CHUNK;
  KV* kc = reinterpret_cast<KV*>(a.k_cache) + (size_t)kvh * a.max_context * hd;
  KV* vc = reinterpret_cast<KV*>(a.v_cache) + (size_t)kvh * a.max_context * hd;
  // All cached rows of the slice -> shared memory with asynchronous 16-byte copies: every copy of the CTA is in flight at once
  // (one global latency).  The rows were written by earlier steps, so the copies are issued BEFORE the wait for the previous
  // kernel (they overlap its tail); only the position counter they are sized by could, in principle, still be the previous
  // step's, so it is read again after the wait and the copies are redone in the (never observed) case that it moved.
  auto fetch_rows = [&](int pos_now) {
    const int wpr = hd / VEC, n_old = max(0, min(min(ATTN_CHUNK, a.max_context - lo), pos_now - lo)), words = n_old * wpr;
    for (int i = threadIdx.x; i < words; i += blockDim.x) {
      const int r = i / wpr, c = (i - r * wpr) * VEC;
      cp_async16(s_k + r * rstride + c, kc + (size_t)(lo + r) * hd + c);
      cp_async16(s_v + r * rstride + c, vc + (size_t)(lo + r) * hd + c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int pos_early = min(max(__ldcg(a.pos), 0), a.max_context - 1);
  fetch_rows(pos_early);
  pdl_wait();
#ifdef B200Q_GEMV_PROF
  if (prof_cta) ASTAMP(1);
#endif
  const int pos = __ldcg(a.pos);
  if (pos < 0 || pos >= a.max_context) {        // no cache row for this position: touch nothing (uniform over the grid)
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (threadIdx.x == 0) atomicExch(&g_decode_status, 2);
    return;
  }
  if (pos != pos_early) {                       // uniform over the CTA
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    fetch_rows(pos);
  }
#ifdef B200Q_GEMV_PROF
  if (prof_cta) ASTAMP(5);
#endif
  const int n_ctx = pos + 1;
  if (lo >= n_ctx) { asm volatile("cp.async.wait_group 0;" ::: "memory"); return; }
  const int n = min(ATTN_CHUNK, n_ctx - lo);
  const int n_active = (n_ctx + ATTN_CHUNK - 1) / ATTN_CHUNK;
  // RoPE, half-split layout: (x1 cos - x2 sin) || (x2 cos + x1 sin); dims past rope_dim pass through
  const float* rope = a.rope + (size_t)pos * a.rope_dim;
  for (int i = threadIdx.x; i < n_rep * hd; i += blockDim.x) {
    const int r = i / hd, d = i - r * hd;
    const float* q = a.qkv + (size_t)(kvh * n_rep + r) * hd;
    float v = q[d];
    if (d < half_r) v = q[d] * rope[d] - q[d + half_r] * rope[half_r + d];
    else if (d < a.rope_dim) v = q[d] * rope[d - half_r] + q[d - half_r] * rope[d];
    s_q[i] = v;
  }
  if (lo <= pos && pos < lo + ATTN_CHUNK) {   // this CTA owns the new position: append it to the cache and to its slice
    const float* kq = a.qkv + (size_t)a.n_heads * hd + (size_t)kvh * hd;
    const float* vq = a.qkv + (size_t)(a.n_heads + a.n_kv_heads) * hd + (size_t)kvh * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
      float v = kq[d];
      if (d < half_r) v = kq[d] * rope[d] - kq[d + half_r] * rope[half_r + d];
      else if (d < a.rope_dim) v = kq[d] * rope[d - half_r] + kq[d - half_r] * rope[d];
      const KV kk = KvIO<KV>::cast(v), vv = KvIO<KV>::cast(vq[d]);
      kc[(size_t)pos * hd + d] = kk; vc[(size_t)pos * hd + d] = vv;
      s_k[(pos - lo) * rstride + d] = kk; s_v[(pos - lo) * rstride + d] = vv;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
#ifdef B200Q_GEMV_PROF
  if (prof_cta) ASTAMP(6);
#endif

  const int d0 = lane * 4;
  const bool dl = d0 < hd;
  const float scale = 1.0f / sqrtf((float)hd);
  float* partial = reinterpret_cast<float*>(a.scratch);
  const int pstride = hd + 4;   // keeps every record 16-byte aligned
  // A head's positions are shared by `ws` warps (blockDim = ws * n_rep warps; ws = 2 when the block has room): warp w works on head
  // w % n_rep and on the positions 32 * (w / n_rep) + 32 * ws * j + lane.  Each has its own running max / denominator / output; the
  // head's first warp merges them (the same merge as across slices) and carries on alone.
  const int ws = (int)(blockDim.x >> 5) / n_rep, head = warp % n_rep, part = warp / n_rep;
  float mx = -INFINITY, den = 0.f;
  float4 o = make_float4(0, 0, 0, 0);
  {
    float* sc = s_sc + head * ATTN_CHUNK;
    const float* q = s_q + head * hd;
    float lmax = -INFINITY;
    for (int i = 32 * part + lane; i < n; i += 32 * ws) {
      const KV* kr = s_k + i * rstride;
      // four running sums: a lane's dot product is a dependent chain otherwise
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      int d = 0;
      for (; d + 4 * VEC <= hd; d += 4 * VEC) {
        s0 += KvIO<KV>::dot(kr + d, q + d); s1 += KvIO<KV>::dot(kr + d + VEC, q + d + VEC);
        s2 += KvIO<KV>::dot(kr + d + 2 * VEC, q + d + 2 * VEC); s3 += KvIO<KV>::dot(kr + d + 3 * VEC, q + d + 3 * VEC);
      }
      for (; d < hd; d += VEC) s0 += KvIO<KV>::dot(kr + d, q + d);
      float s = (s0 + s1) + (s2 + s3);
      s *= scale;
      sc[i] = s;
      lmax = fmaxf(lmax, s);
    }
    mx = warp_max(lmax);
    float lsum = 0.f;
    for (int i = 32 * part + lane; i < n; i += 32 * ws) { const float pr = __expf(sc[i] - mx); sc[i] = pr; lsum += pr; }
    den = warp_sum(lsum);
    __syncwarp();
    if (dl) {
      const KV* vr = s_v + d0;
      float4 o2 = make_float4(0, 0, 0, 0);      // two independent sums
      for (int b0 = 32 * part; b0 < n; b0 += 32 * ws) {      // this warp's runs of 32 positions
        const int e = min(n, b0 + 32);
        int i = b0;
#pragma unroll 4
        for (; i + 2 <= e; i += 2) {
          const float pr = sc[i], pr2 = sc[i + 1];
          const float4 v = KvIO<KV>::load4(vr + i * rstride), v2 = KvIO<KV>::load4(vr + (i + 1) * rstride);
          o.x = fmaf(pr, v.x, o.x); o.y = fmaf(pr, v.y, o.y); o.z = fmaf(pr, v.z, o.z); o.w = fmaf(pr, v.w, o.w);
          o2.x = fmaf(pr2, v2.x, o2.x); o2.y = fmaf(pr2, v2.y, o2.y); o2.z = fmaf(pr2, v2.z, o2.z); o2.w = fmaf(pr2, v2.w, o2.w);
        }
        if (i < e) {
          const float pr = sc[i];
          const float4 v = KvIO<KV>::load4(vr + i * rstride);
          o.x = fmaf(pr, v.x, o.x); o.y = fmaf(pr, v.y, o.y); o.z = fmaf(pr, v.z, o.z); o.w = fmaf(pr, v.w, o.w);
        }
      }
      o.x += o2.x; o.y += o2.y; o.z += o2.z; o.w += o2.w;
    }
  }
  if (ws > 1) {
    float* hp = s_part + head * (hd + 4);
    if (part == 1) {
      if (dl) *reinterpret_cast<float4*>(hp + d0) = o;
      if (lane == 0) { hp[hd] = mx; hp[hd + 1] = den; }
    }
    __syncthreads();
    if (part == 0) {
      const float m1 = hp[hd], l1 = hp[hd + 1];
      const float gm = fmaxf(mx, m1);                       // the first warp always holds position 0 of the slice: mx is finite
      const float c0 = __expf(mx - gm), c1 = l1 > 0.f ? __expf(m1 - gm) : 0.f;
      float4 o1 = make_float4(0, 0, 0, 0);
      if (dl) o1 = *reinterpret_cast<const float4*>(hp + d0);
      o.x = o.x * c0 + o1.x * c1; o.y = o.y * c0 + o1.y * c1; o.z = o.z * c0 + o1.z * c1; o.w = o.w * c0 + o1.w * c1;
      den = den * c0 + l1 * c1;
      mx = gm;
    }
  }
  if (part == 0) {
    if (n_active == 1) {   // short context: this CTA holds the whole softmax
      const float inv = 1.f / den;
      const float4 r = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
      if (dl) *reinterpret_cast<float4*>(a.out + (size_t)(kvh * n_rep + head) * hd + d0) = r;
      if (a.xq_out) quant_block_8x4(r, lane & 7, (kvh * n_rep + head) * 4 + (lane >> 3), XqDst(a.xq_out, a.n_heads));   // head_dim 128: one group per head
    } else {
      float* pp = partial + ((size_t)(kvh * n_rep + head) * a.n_split + split) * pstride;
      if (dl) *reinterpret_cast<float4*>(pp + d0) = o;
      if (lane == 0) { pp[hd] = mx; pp[hd + 1] = den; }
    }
  }
  if (n_active == 1) return;
#ifdef B200Q_GEMV_PROF
  if (prof_cta) ASTAMP(2);
  if (threadIdx.x == 0) atomicMax(&g_attn_prof[prof_slot * 8 + 7], gtime());      // this slot is re-used: max over CTAs of "partials done"
#endif
  // last CTA of this KV head merges the slices
  __threadfence();
  __syncthreads();
  unsigned* counter = reinterpret_cast<unsigned*>(partial + (size_t)a.n_heads * a.n_split * pstride);
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&counter[kvh], 1u);
    s_last = (prev == (unsigned)n_active - 1);
    if (s_last) counter[kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
#ifdef B200Q_GEMV_PROF
  if (kvh == 0) { if (threadIdx.x == 0) g_attn_prof[prof_slot * 8 + 3] = gtime(); }
#endif
  if (warp < n_rep) {
    const float* hp = partial + (size_t)(kvh * n_rep + warp) * a.n_split * pstride;
    // Batches of 16 slices: the statistics (one slice per lane) and every lane's 4 output dims of all 16 slices are
    // loaded before anything is used, so a batch costs one L2 round trip.  Running max / denominator across batches.
    float gm = -INFINITY, den = 0.f;
    float4 o = make_float4(0, 0, 0, 0);
    for (int s0 = 0; s0 < n_active; s0 += 16) {
      const int cnt = min(16, n_active - s0);
      float2 ml = make_float2(-INFINITY, 0.f);
      if (lane < cnt) ml = __ldcg(reinterpret_cast<const float2*>(hp + (size_t)(s0 + lane) * pstride + hd));
      float4 ov[16];
#pragma unroll
      for (int j = 0; j < 16; j++)
        ov[j] = (dl && j < cnt) ? __ldcg(reinterpret_cast<const float4*>(hp + (size_t)(s0 + j) * pstride + d0)) : make_float4(0, 0, 0, 0);
      const float nm = fmaxf(gm, warp_max(ml.x));
      const float corr = __expf(gm - nm);
      const float w = lane < cnt ? __expf(ml.x - nm) : 0.f;
      den = den * corr + warp_sum(w * ml.y);
      o.x *= corr; o.y *= corr; o.z *= corr; o.w *= corr;
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const float wj = __shfl_sync(0xffffffffu, w, j);      // every lane takes part in the shuffle
        o.x = fmaf(wj, ov[j].x, o.x); o.y = fmaf(wj, ov[j].y, o.y); o.z = fmaf(wj, ov[j].z, o.z); o.w = fmaf(wj, ov[j].w, o.w);
      }
      gm = nm;
    }
    const float inv = 1.f / den;
    const float4 r = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    if (dl) *reinterpret_cast<float4*>(a.out + (size_t)(kvh * n_rep + warp) * hd + d0) = r;
    if (a.xq_out) quant_block_8x4(r, lane & 7, (kvh * n_rep + warp) * 4 + (lane >> 3), XqDst(a.xq_out, a.n_heads));
  }
#ifdef B200Q_GEMV_PROF
  if (kvh == 0) { __syncthreads(); if (threadIdx.x == 0) g_attn_prof[prof_slot * 8 + 4] = gtime(); }
#endif
}

#ifdef B200Q_GEMV_PROF
}  // namespace
extern "C" int b200q_attn_prof_read(unsigned long long* out, int max_slots, unsigned* n) {
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_attn_prof, sizeof(unsigned long long) * 8 * (max_slots < 4096 ? max_slots : 4096)));
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(n, g_attn_prof_n, sizeof(unsigned)));
  return B200Q_OK;
}
extern "C" int b200q_attn_prof_reset(void) {
  static unsigned long long zeros[4096 * 8];
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_attn_prof, zeros, sizeof(zeros)));
  return B200Q_OK;
}
namespace {
#endif

// ---------------------------------------------------------------------------
// arg-max with the lowest index winning ties, then tokens[pos+1] = it and pos += 1.
// scratch: float val[ARGMAX_CTAS], int idx[ARGMAX_CTAS], uint counter.
constexpr int ARGMAX_CTAS = 128;
constexpr int ARGMAX_THREADS = 256;

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const float* __restrict__ logits, int n, int32_t* tokens, int32_t* pos,
                                                                int max_context, float* sval, int* sidx, unsigned* counter) {
  __shared__ float wv[ARGMAX_THREADS / 32];
  __shared__ int wi[ARGMAX_THREADS / 32];
  __shared__ int s_last;
  pdl_launch_dependents();
  pdl_wait();
  float v = -INFINITY; int idx = 0x7fffffff;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) argmax_combine(v, idx, logits[i], i);
  auto block_reduce = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, v, o); int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      argmax_combine(v, idx, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { wv[threadIdx.x >> 5] = v; wi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
      v = threadIdx.x < ARGMAX_THREADS / 32 ? wv[threadIdx.x] : -INFINITY;
      idx = threadIdx.x < ARGMAX_THREADS / 32 ? wi[threadIdx.x] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o); int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_combine(v, idx, ov, oi);
      }
    }
  };
  block_reduce();
  if (threadIdx.x == 0) {
    sval[blockIdx.x] = v; sidx[blockIdx.x] = idx;
    __threadfence();
    unsigned prev = atomicAdd(counter, 1u);
    s_last = (prev == gridDim.x - 1);
    if (s_last) *counter = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  v = -INFINITY; idx = 0x7fffffff;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) argmax_combine(v, idx, __ldcg(sval + i), __ldcg(sidx + i));
  __syncthreads();
  block_reduce();
  if (threadIdx.x == 0) {
    const int p = *pos;
    if (p < 0 || p >= max_context) atomicExch(&g_decode_status, 2);      // tokens[max_context] is the last entry
    else { tokens[p + 1] = idx == 0x7fffffff ? 0 : idx; *pos = p + 1; }
  }
}

}  // namespace

int b200q_decode_status_take(int* status) {
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_decode_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int)));
  return B200Q_OK;
}

extern "C" int b200q_embed(const void* table, const int32_t* tokens, const int32_t* pos, float* x, int dim, int vocab, int max_context, void* xq_out,
                           const void* xq_norm_weight, float* ss_out, int flags, void* stream) {
  if (!table || !tokens || !pos || !x || dim <= 0 || vocab <= 0 || max_context <= 0) return B200Q_ERR_BAD_ARG;
  if ((uintptr_t)xq_out & 15) return B200Q_ERR_MISALIGNED;
  if (xq_out && dim % 32) return B200Q_ERR_BAD_SHAPE;
  B200Q_CHECK_CUDA(launch_k(embed_kernel, dim3(ceil_div(dim, 256)), dim3(256), 0, (cudaStream_t)stream, (flags & B200Q_FLAG_PDL) != 0,
                            (const __half*)table, tokens, pos, x, dim, vocab, max_context, xq_out, (const __half*)xq_norm_weight, ss_out));
  return B200Q_OK;
}

extern "C" int b200q_advance(int32_t* pos, int max_context, int flags, void* stream) {
  if (!pos || max_context <= 0) return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(launch_k(advance_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (flags & B200Q_FLAG_PDL) != 0, pos, max_context));
  return B200Q_OK;
}

extern "C" int b200q_attn_min_split(int max_context) { return max_context <= 0 ? 0 : ceil_div(max_context, ATTN_CHUNK); }

extern "C" size_t b200q_attn_scratch_bytes(int n_heads, int n_kv_heads, int head_dim, int n_split) {
  if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_split <= 0) return 0;
  return ((size_t)n_heads * n_split * (head_dim + 4)) * sizeof(float) + (size_t)n_kv_heads * sizeof(unsigned);
}

// Argument checks shared by both attention entry points (`scratch` is checked by the caller that needs it).
static int attn_validate(const b200q_attn_args* a) {
  if (!a || !a->qkv || !a->k_cache || !a->v_cache || !a->rope || !a->pos || !a->out) return B200Q_ERR_BAD_ARG;
  if (a->n_heads <= 0 || a->n_kv_heads <= 0 || a->n_heads % a->n_kv_heads || a->n_split <= 0 || a->max_context <= 0) return B200Q_ERR_BAD_ARG;
  if (a->head_dim <= 0 || a->head_dim > MAX_HD || a->head_dim % 8 || a->n_heads / a->n_kv_heads > MAX_REP) return B200Q_ERR_BAD_SHAPE;
  if (a->rope_dim < 0 || a->rope_dim > a->head_dim || a->rope_dim % 2) return B200Q_ERR_BAD_SHAPE;
  if (a->kv_dtype != B200Q_F16 && a->kv_dtype != B200Q_F32) return B200Q_ERR_BAD_ARG;
  if (a->xq_out && (a->head_dim != 128 || ((uintptr_t)a->xq_out & 15))) return B200Q_ERR_BAD_SHAPE;   // one 128-wide group per head
  if (((uintptr_t)a->k_cache | (uintptr_t)a->v_cache | (uintptr_t)a->qkv | (uintptr_t)a->out) & 15) return B200Q_ERR_MISALIGNED;
  if ((int64_t)a->n_split * ATTN_CHUNK < a->max_context) return B200Q_ERR_BAD_SHAPE;   // the slices must cover the whole cache
  return B200Q_OK;
}

extern "C" size_t b200q_attn_seq_scratch_stride(int n_heads, int n_kv_heads, int head_dim, int n_split) {
  return (b200q_attn_scratch_bytes(n_heads, n_kv_heads, head_dim, n_split) + 255) & ~(size_t)255;
}

static int attn_decode_launch(const b200q_attn_args* a, int n_seqs, void* stream) {
  const int rc = attn_validate(a);
  if (rc != B200Q_OK) return rc;
  if (!a->scratch) return B200Q_ERR_BAD_ARG;
  if ((uintptr_t)a->scratch & 15) return B200Q_ERR_MISALIGNED;
  int n_rep = a->n_heads / a->n_kv_heads;
  const int ws = 2 * n_rep <= MAX_REP ? 2 : 1;              // warps per head
  dim3 grid(a->n_kv_heads, a->n_split, n_seqs), block(ws * n_rep * 32);
  SeqStride sq = {};
  if (n_seqs > 1) {
    sq.qkv = (size_t)(a->n_heads + 2 * a->n_kv_heads) * a->head_dim; sq.cache = (size_t)a->n_kv_heads * a->max_context * a->head_dim;
    sq.out = (size_t)a->n_heads * a->head_dim; sq.pos = 1;
    sq.scratch_bytes = b200q_attn_seq_scratch_stride(a->n_heads, a->n_kv_heads, a->head_dim, a->n_split);
  }
  bool pdl = (a->flags & B200Q_FLAG_PDL) != 0;
  const int esz = a->kv_dtype == B200Q_F16 ? 2 : 4, vec = 16 / esz;
  size_t smem = (size_t)2 * ATTN_CHUNK * (a->head_dim + vec) * esz + (size_t)n_rep * (a->head_dim + ATTN_CHUNK + a->head_dim + 4) * sizeof(float);
  static PerDeviceFlag attr_set;
  const int dev = b200q_current_device();
  if (dev < 0) return B200Q_ERR_CUDA;
  if (!attr_set.test(dev)) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(attn_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(attn_decode_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    attr_set.set(dev);
  }
#ifdef B200Q_GEMV_PROF
  static int prof_counter = 0;
  b200q_attn_args ap = *a;
  ap.flags = (ap.flags & 0xFFFF) | ((prof_counter++ & 4095) << 16);
  a = &ap;
#endif
  if (a->kv_dtype == B200Q_F16) B200Q_CHECK_CUDA(launch_k(attn_decode_kernel<__half>, grid, block, smem, (cudaStream_t)stream, pdl, *a, sq));
  else B200Q_CHECK_CUDA(launch_k(attn_decode_kernel<float>, grid, block, smem, (cudaStream_t)stream, pdl, *a, sq));
  return B200Q_OK;
}

extern "C" int b200q_attn_decode(const b200q_attn_args* a, void* stream) { return attn_decode_launch(a, 1, stream); }

extern "C" int b200q_attn_decode_seqs(const b200q_attn_args* a, int n_seqs, void* stream) {
  if (n_seqs <= 0 || (a && a->xq_out)) return B200Q_ERR_BAD_ARG;
  return attn_decode_launch(a, n_seqs, stream);
}

extern "C" size_t b200q_argmax_scratch_bytes(void) { return ARGMAX_CTAS * (sizeof(float) + sizeof(int)) + sizeof(unsigned); }

extern "C" int b200q_argmax_advance(const float* logits, int n, int32_t* tokens, int32_t* pos, int max_context, void* scratch, int flags, void* stream) {
  if (!logits || !tokens || !pos || !scratch || n <= 0 || max_context <= 0) return B200Q_ERR_BAD_ARG;
  float* sval = (float*)scratch; int* sidx = (int*)(sval + ARGMAX_CTAS); unsigned* counter = (unsigned*)(sidx + ARGMAX_CTAS);
  int grid = ceil_div(n, ARGMAX_THREADS); if (grid > ARGMAX_CTAS) grid = ARGMAX_CTAS;
  B200Q_CHECK_CUDA(launch_k(argmax_kernel, dim3(grid), dim3(ARGMAX_THREADS), 0, (cudaStream_t)stream, (flags & B200Q_FLAG_PDL) != 0,
                            logits, n, tokens, pos, max_context, sval, sidx, counter));
  return B200Q_OK;
}

// ---------------------------------------------------------------------------
// Attention for callers that may not allocate device memory.
//
// Some hosts of this library hand out device memory themselves and forbid anything else from doing so: a serving loop
// that froze its memory pool after warm-up, an engine whose planner owns one arena and replays captured work, or code
// running while a stream is being captured (the CUDA allocator calls are illegal there).  Such a caller cannot provide
// the scratch buffer b200q_attn_decode needs unless it planned for it.  This variant brings its own: a fixed array that
// is part of the library image, so every GPU that loads the library holds these bytes until the process exits.
constexpr size_t ATTN_STATIC_SCRATCH_BYTES = (size_t)2 << 20;     // 2 MiB: e.g. 64 heads x 62 slices (3968 positions) of head_dim 128
static __device__ __align__(256) unsigned char g_attn_static_scratch[ATTN_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = B200Q_MAX_DEVICES;
static void* g_attn_static_ptr[MAX_DEVICES];   // device address of the array on each device, filled on first use

extern "C" size_t b200q_attn_decode_static_capacity(void) { return ATTN_STATIC_SCRATCH_BYTES; }

extern "C" int b200q_attn_decode_static(const b200q_attn_args* a, void* stream) {
  if (!a) return B200Q_ERR_BAD_ARG;
  const size_t need = b200q_attn_scratch_bytes(a->n_heads, a->n_kv_heads, a->head_dim, a->n_split);
  if (need == 0) return B200Q_ERR_BAD_ARG;
  if (need > ATTN_STATIC_SCRATCH_BYTES) return B200Q_ERR_TOO_LARGE;
  const int rc = attn_validate(a);      // before anything is put on the stream
  if (rc != B200Q_OK) return rc;   // heads x slices x (head_dim + 4) floats must fit the built-in array
  int dev = -1;
  B200Q_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return B200Q_ERR_TOO_LARGE;
  if (!g_attn_static_ptr[dev]) {
    // In host code the array's name is only a handle; the kernel needs the address the array has on THIS device.
    void* p = nullptr;
    B200Q_CHECK_CUDA(cudaGetSymbolAddress(&p, g_attn_static_scratch));
    g_attn_static_ptr[dev] = p;
  }
  // The arrival counters sit behind the partial results, at an offset that depends on the geometry, and the array keeps
  // whatever the last call left there: zero them (stream-ordered, no allocation) before the kernel counts arrivals.
  unsigned char* base = static_cast<unsigned char*>(g_attn_static_ptr[dev]);
  const size_t counters_at = need - (size_t)a->n_kv_heads * sizeof(unsigned);
  B200Q_CHECK_CUDA(cudaMemsetAsync(base + counters_at, 0, (size_t)a->n_kv_heads * sizeof(unsigned), (cudaStream_t)stream));
  b200q_attn_args b = *a;
  b.scratch = base;
  b.flags &= ~B200Q_FLAG_PDL;   // the memset in front is not a kernel: launch the kernel fully ordered behind it
  return b200q_attn_decode(&b, stream);
}
