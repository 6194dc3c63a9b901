// MXFP8 (E4M3 values + one E8M0 scale per 32 along K) mixture-of-experts path:
// activation quantiser, top-k routing tables, row dispatch / combine, SwiGLU + requantise.
// The grouped expert GEMM is in mxfp8_gemm.cu.
//
// Semantics follow extra/gemm/cdna_asm_gemm.py:149-173 (quantize_mxfp8, _mx_block_scale),
// tinygrad/dtype.py:237-260 (E4M3 round-to-nearest-even, saturating), extra/gemm/moe_routing.py:89-131
// (route / dispatch / combine, groups padded to 256 rows) and tinygrad/llm/model.py:35-41,110-130
// (softmax-over-all-experts gating with compare-count top-k, the OLMoE default).
#include "common.cuh"
#include "mxq.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <math.h>

namespace {

constexpr int BLOCK_ROW = 256;   // extra/gemm/moe_routing.py:4

__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  bf16x8_to_f32(*reinterpret_cast<const uint4*>(p), v);
}
__device__ __forceinline__ float amax8_quad(const float (&v)[8]) {      // |max| over the 32 values held by 4 neighbouring lanes
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(v[i]));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  return fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
}

// One warp per 256 consecutive values of a row: 4 lanes share a block of 32, a lane holds 8 values (16-byte loads, 8-byte stores).
// Rows of x go to rows dest[r] of the outputs (dest == nullptr: identity); `fan` consecutive dest entries per input row.
template <typename T>
__global__ void quantize_mxfp8_kernel(const T* __restrict__ x, int64_t rows, int k, const int32_t* __restrict__ dest, int fan,
                                      uint8_t* __restrict__ q, uint8_t* __restrict__ e8) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int kb = k >> 5, chunks = (kb + 7) >> 3;
  if (warp >= rows * chunks) return;
  const int64_t r = warp / chunks;
  const int b = (int)(warp - r * chunks) * 8 + (lane >> 2), col = b * 32 + (lane & 3) * 8;
  const bool valid = b < kb;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (valid) load8<T>(x + r * k + col, v);
  const uint8_t e = mx_scale_exponent(amax8_quad(v));
  const uint2 pk = mx_quant8(v, e);
  if (!valid) return;
  for (int f = 0; f < fan; f++) {
    const int64_t o = dest ? (int64_t)dest[r * fan + f] : r;
    *reinterpret_cast<uint2*>(q + o * k + col) = pk;
    if ((lane & 3) == 0) e8[o * kb + b] = e;
  }
}

// SwiGLU between the two expert GEMMs: h = [gate | up] (bf16, [m, 2f]) -> act = silu(gate) * up computed in fp32,
// rounded to bf16 as a tensor would be stored, then quantised like any activation.  Same work split as the quantiser.
__global__ void swiglu_quant_kernel(const __nv_bfloat16* __restrict__ h, int64_t rows, const int32_t* __restrict__ rows_used, int f,
                                    uint8_t* __restrict__ q, uint8_t* __restrict__ e8) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int kb = f >> 5, chunks = (kb + 7) >> 3;
  if (rows_used) rows = min(rows, (int64_t)*rows_used);
  if (warp >= rows * chunks) return;
  const int64_t r = warp / chunks;
  const int b = (int)(warp - r * chunks) * 8 + (lane >> 2), col = b * 32 + (lane & 3) * 8;
  const bool valid = b < kb;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (valid) {
    float g[8], u[8];
    load8<__nv_bfloat16>(h + r * 2 * f + col, g);
    load8<__nv_bfloat16>(h + r * 2 * f + f + col, u);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __bfloat162float(__float2bfloat16_rn((g[i] / (1.f + expf(-g[i]))) * u[i]));
  }
  const uint8_t e = mx_scale_exponent(amax8_quad(v));
  const uint2 pk = mx_quant8(v, e);
  if (!valid) return;
  *reinterpret_cast<uint2*>(q + r * f + col) = pk;
  if ((lane & 3) == 0) e8[r * kb + b] = e;
}

// ---------------------------------------------------------------------------
// routing, step 1: one warp per token.  mode 0 (extra/gemm/moe_routing.py:115-116): top-k of the raw logits in
// descending order, weights = softmax over the k.  mode 1 (tinygrad/llm/model.py:118,123-124 with the OLMoE defaults):
// scores = softmax over all experts, top-k listed in ascending order of score, weights = the scores, not renormalised.
// Ties: the lower expert index ranks higher (model.py:35-41).
constexpr int MAX_E_PER_LANE = 8;   // up to 256 experts

__global__ void route_topk_kernel(const float* __restrict__ logits, int n_tokens, int n_experts, int k, int mode, int32_t* __restrict__ topi,
                                  float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (tok >= n_tokens) return;
  float v[MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; i++) {
    const int e = i * 32 + lane;
    v[i] = e < n_experts ? logits[(size_t)tok * n_experts + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float denom = 0.f;
  if (mode == 1) {
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) denom += (i * 32 + lane < n_experts) ? expf(v[i] - mx) : 0.f;
    denom = warp_sum(denom);
  }
  float top1 = 0.f, ksum = 0.f;
  for (int j = 0; j < k; j++) {
    float bv = -INFINITY; int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) { const int e = i * 32 + lane; if (v[i] > bv) { bv = v[i]; bi = e; } }   // lowest index wins inside a lane
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) if (i * 32 + lane == bi) v[i] = -INFINITY;    // taken
    if (j == 0) top1 = bv;
    const int slot = mode == 1 ? k - 1 - j : j;
    float w;
    if (mode == 1) w = expf(bv - mx) / denom;
    else { w = expf(bv - top1); ksum += w; }
    if (lane == 0) { topi[(size_t)tok * k + slot] = bi; weights[(size_t)tok * k + slot] = w; }
  }
  if (mode == 0) {
    __syncwarp();
    if (lane < k) weights[(size_t)tok * k + lane] /= ksum;
  }
}


// The gating of tinygrad's own MoE block (tinygrad/llm/model.py:110-128), one warp per token:
//   scores = logits (SOFTMAX_WEIGHT) | softmax(logits) | sigmoid(logits) | sqrt(softplus(logits));
//   sel    = the k best of scores (+ sel_bias), listed in ascending order, the lower expert index ranking higher on ties
//            (`pairwise_topk`, model.py:35-41);
//   probs  = scores[sel]; SOFTMAX_WEIGHT: softmax over the k; normalize: / sum; times `scale`.
// The reference's own shortcut is applied by the caller: SOFTMAX with normalize and no bias is run as SOFTMAX_WEIGHT (model.py:116-117).
enum { GATE_SOFTMAX = 1, GATE_SIGMOID = 2, GATE_SOFTMAX_WEIGHT = 3, GATE_SQRT_SOFTPLUS = 4 };     // ExpertGating, model.py:9-13

__global__ void route_gating_kernel(const float* __restrict__ logits, const float* __restrict__ sel_bias, int n_tokens, int n_experts, int k, int gating,
                                    int normalize, float scale, int32_t* __restrict__ topi, float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (tok >= n_tokens) return;
  float sc[MAX_E_PER_LANE], key[MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; i++) {
    const int e = i * 32 + lane;
    sc[i] = e < n_experts ? logits[(size_t)tok * n_experts + e] : -INFINITY;
    mx = fmaxf(mx, sc[i]);
  }
  if (gating == GATE_SOFTMAX) {
    mx = warp_max(mx);
    float denom = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) { if (i * 32 + lane < n_experts) { sc[i] = expf(sc[i] - mx); denom += sc[i]; } }
    denom = warp_sum(denom);
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) if (i * 32 + lane < n_experts) sc[i] /= denom;
  } else if (gating == GATE_SIGMOID) {
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) if (i * 32 + lane < n_experts) sc[i] = 1.f / (1.f + expf(-sc[i]));
  } else if (gating == GATE_SQRT_SOFTPLUS) {
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) if (i * 32 + lane < n_experts) sc[i] = sqrtf(sc[i] > 20.f ? sc[i] : log1pf(expf(sc[i])));
  }
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; i++) {
    const int e = i * 32 + lane;
    key[i] = e < n_experts ? (sel_bias ? sc[i] + sel_bias[e] : sc[i]) : -INFINITY;
  }
  float pv = 0.f;                        // lane j < k keeps the probability of slot j
  for (int j = 0; j < k; j++) {
    float bv = -INFINITY, bs = 0.f; int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) { const int e = i * 32 + lane; if (key[i] > bv) { bv = key[i]; bs = sc[i]; bi = e; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bs = os; bi = oi; }
    }
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; i++) if (i * 32 + lane == bi) key[i] = -INFINITY;    // taken
    const int slot = k - 1 - j;          // ascending order of rank
    if (lane == slot) pv = bs;
    if (lane == 0) topi[(size_t)tok * k + slot] = bi;
  }
  const bool mine = lane < k;
  if (gating == GATE_SOFTMAX_WEIGHT) {
    const float m2 = warp_max(mine ? pv : -INFINITY);
    const float ev = mine ? expf(pv - m2) : 0.f;
    pv = ev / warp_sum(ev);
  }
  if (normalize) pv = pv / warp_sum(mine ? pv : 0.f);
  if (mine) weights[(size_t)tok * k + lane] = pv * scale;
}

// routing, steps 2-4: stable counting sort of the T*k (token, slot) pairs by expert.
// dest_row[i] = off[e_i] + (number of pairs before i with the same expert); off = cumulative group sizes padded to 256.
constexpr int ROUTE_CHUNK = 1024;

__global__ void __launch_bounds__(ROUTE_CHUNK) route_count_kernel(const int32_t* __restrict__ topi, int n, int n_experts, int32_t* __restrict__ counts) {
  extern __shared__ int s_cnt[];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * ROUTE_CHUNK + threadIdx.x;
  if (i < n) atomicAdd(&s_cnt[topi[i]], 1);      // integer counts: the order of the adds does not matter
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[(size_t)blockIdx.x * n_experts + e] = s_cnt[e];
}

// one thread per expert: exclusive scan of its chunk counts (in place), then thread 0 builds the padded offsets
__global__ void route_scan_kernel(int32_t* __restrict__ counts, int n_chunks, int n_experts, int32_t* __restrict__ off, int pad,
                                  int32_t* __restrict__ counts_out) {
  extern __shared__ int s_tot[];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < n_chunks; c++) { const int v = counts[(size_t)c * n_experts + e]; counts[(size_t)c * n_experts + e] = run; run += v; }
    s_tot[e] = run;
    if (counts_out) counts_out[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    off[0] = 0;
    for (int e = 0; e < n_experts; e++) { run += (s_tot[e] + pad - 1) / pad * pad; off[e + 1] = run; }
  }
}

// rows of `row_bytes` bytes moved by an index table: scatter dst[idx[i]] = src[i] or gather dst[i] = src[idx[i]]; idx < 0 skips
template <typename V>
__global__ void permute_rows_kernel(const V* __restrict__ src, const int32_t* __restrict__ idx, int64_t n_rows, int row_vecs, V* __restrict__ dst,
                                    int gather) {
  const int64_t r = blockIdx.x;
  const int j = idx[r];
  if (j < 0) return;
  const V* s = src + (gather ? (int64_t)j : r) * row_vecs;
  V* d = dst + (gather ? r : (int64_t)j) * row_vecs;
  for (int i = threadIdx.x; i < row_vecs; i += blockDim.x) d[i] = s[i];
}

__global__ void __launch_bounds__(ROUTE_CHUNK) route_place_kernel(const int32_t* __restrict__ topi, int n, int n_experts,
                                                                  const int32_t* __restrict__ counts, const int32_t* __restrict__ off,
                                                                  int32_t* __restrict__ dest_row) {
  extern __shared__ int s_wcnt[];                 // [32 warps][n_experts] pairs of each expert seen by each warp
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j = threadIdx.x; j < 32 * n_experts; j += blockDim.x) s_wcnt[j] = 0;
  __syncthreads();
  const int i = blockIdx.x * ROUTE_CHUNK + threadIdx.x;
  const int e = i < n ? topi[i] : -1;
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const int before_in_warp = __popc(same & ((1u << lane) - 1));
  if (e >= 0 && before_in_warp == 0) s_wcnt[warp * n_experts + e] = __popc(same);
  __syncthreads();
  if (e >= 0) {
    int before = counts[(size_t)blockIdx.x * n_experts + e] + before_in_warp;
    for (int w = 0; w < warp; w++) before += s_wcnt[w * n_experts + e];
    dest_row[i] = off[e] + before;
  }
}

// combine (extra/gemm/moe_routing.py:128-131): out[t] = sum_j weights[t, j] * y[dest_row[t*k + j]], fp32 sum in slot order, bf16 out
__global__ void combine_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ dest_row, const float* __restrict__ weights,
                               int n_tokens, int k, int d, __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < k; j++) acc += weights[(size_t)t * k + j] * __bfloat162float(y[(size_t)dest_row[(size_t)t * k + j] * d + c]);
    out[(size_t)t * d + c] = __float2bfloat16_rn(acc);
  }
}
// d % 8 == 0: a thread sums 8 neighbouring columns over the k rows (16-byte loads), same order of additions
__global__ void combine8_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ dest_row, const float* __restrict__ weights,
                                int n_tokens, int k, int d, __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; j++) {
      const float w = weights[(size_t)t * k + j];
      float v[8];
      load8<__nv_bfloat16>(y + (size_t)dest_row[(size_t)t * k + j] * d + c, v);
#pragma unroll
      for (int i = 0; i < 8; i++) acc[i] += w * v[i];
    }
    uint4 pk;
    __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int i = 0; i < 4; i++) hp[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)t * d + c) = pk;
  }
}

}  // namespace

extern "C" int b200q_quantize_mxfp8(const void* x, int x_dtype, int64_t rows, int k, const int32_t* dest_row, int fan, void* q, void* e8, void* stream) {
  if (rows < 0 || k <= 0 || (rows && (!x || !q || !e8))) return B200Q_ERR_BAD_ARG;
  if (x_dtype != B200Q_F32 && x_dtype != B200Q_BF16) return B200Q_ERR_BAD_ARG;
  if (k % 32) return B200Q_ERR_BAD_SHAPE;
  if (dest_row ? fan <= 0 : fan != 1) return B200Q_ERR_BAD_ARG;
  if (rows == 0) return B200Q_OK;
  if (((uintptr_t)x | (uintptr_t)q) & 15) return B200Q_ERR_MISALIGNED;
  const int64_t warps = rows * ((k / 32 + 7) / 8);
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (x_dtype == B200Q_F32) quantize_mxfp8_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)x, rows, k, dest_row, fan, (uint8_t*)q, (uint8_t*)e8);
  else quantize_mxfp8_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, rows, k, dest_row, fan, (uint8_t*)q, (uint8_t*)e8);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_swiglu_quantize_mxfp8(const void* h_bf16, int64_t rows, const int32_t* rows_used, int f, void* q, void* e8, void* stream) {
  if (rows < 0 || f <= 0 || (rows && (!h_bf16 || !q || !e8))) return B200Q_ERR_BAD_ARG;
  if (f % 32) return B200Q_ERR_BAD_SHAPE;
  if (((uintptr_t)h_bf16 | (uintptr_t)q) & 15) return B200Q_ERR_MISALIGNED;
  if (rows == 0) return B200Q_OK;
  const int64_t warps = rows * ((f / 32 + 7) / 8);
  swiglu_quant_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)h_bf16, rows, rows_used, f, (uint8_t*)q,
                                                                                       (uint8_t*)e8);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" size_t b200q_moe_route_scratch_bytes(int n_tokens, int n_experts, int k) {
  if (n_tokens <= 0 || n_experts <= 0 || k <= 0) return 0;
  return (size_t)ceil_div(n_tokens * k, ROUTE_CHUNK) * n_experts * sizeof(int32_t);
}

extern "C" int b200q_moe_rows_max(int n_tokens, int n_experts, int k) {   // m_max_for, extra/gemm/moe_routing.py:89-90
  return (ceil_div(n_tokens * k, BLOCK_ROW) + n_experts) * BLOCK_ROW;
}

extern "C" int b200q_moe_route(const float* logits, int n_tokens, int n_experts, int k, int mode, int32_t* topi, float* weights, int32_t* dest_row,
                               int32_t* off, void* scratch, void* stream) {
  return b200q_moe_route_pad(logits, n_tokens, n_experts, k, mode, BLOCK_ROW, topi, weights, dest_row, off, nullptr, scratch, stream);
}

extern "C" int b200q_permute_rows(const void* src, const int32_t* idx, int64_t n_rows, int row_bytes, void* dst, int gather, void* stream) {
  if (n_rows < 0 || row_bytes <= 0 || (n_rows && (!src || !idx || !dst))) return B200Q_ERR_BAD_ARG;
  if (row_bytes % 4) return B200Q_ERR_BAD_SHAPE;
  if (n_rows == 0) return B200Q_OK;
  if (row_bytes % 16 == 0 && !(((uintptr_t)src | (uintptr_t)dst) & 15))
    permute_rows_kernel<uint4><<<(unsigned)n_rows, 128, 0, (cudaStream_t)stream>>>((const uint4*)src, idx, n_rows, row_bytes / 16, (uint4*)dst, gather);
  else
    permute_rows_kernel<uint32_t><<<(unsigned)n_rows, 128, 0, (cudaStream_t)stream>>>((const uint32_t*)src, idx, n_rows, row_bytes / 4, (uint32_t*)dst, gather);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_moe_route_pad(const float* logits, int n_tokens, int n_experts, int k, int mode, int pad, int32_t* topi, float* weights,
                                   int32_t* dest_row, int32_t* off, int32_t* counts, void* scratch, void* stream) {
  if (!logits || !topi || !weights || !dest_row || !off || !scratch || pad <= 0) return B200Q_ERR_BAD_ARG;
  if (n_tokens <= 0 || n_experts <= 0 || k <= 0 || k > n_experts || (mode != 0 && mode != 1)) return B200Q_ERR_BAD_ARG;
  if (n_experts > 32 * MAX_E_PER_LANE || k > 32) return B200Q_ERR_BAD_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int n = n_tokens * k, n_chunks = ceil_div(n, ROUTE_CHUNK);
  route_topk_kernel<<<ceil_div(n_tokens, 8), 256, 0, st>>>(logits, n_tokens, n_experts, k, mode, topi, weights);
  route_count_kernel<<<n_chunks, ROUTE_CHUNK, n_experts * sizeof(int), st>>>(topi, n, n_experts, (int32_t*)scratch);
  route_scan_kernel<<<1, 256, n_experts * sizeof(int), st>>>((int32_t*)scratch, n_chunks, n_experts, off, pad, counts);
  route_place_kernel<<<n_chunks, ROUTE_CHUNK, 32 * n_experts * sizeof(int), st>>>(topi, n, n_experts, (const int32_t*)scratch, off, dest_row);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_moe_route_tables(const int32_t* topi, int n_tokens, int n_experts, int k, int pad, int32_t* dest_row, int32_t* off, int32_t* counts,
                                      void* scratch, void* stream) {
  if (!topi || !dest_row || !off || !scratch || pad <= 0 || n_tokens <= 0 || n_experts <= 0 || k <= 0) return B200Q_ERR_BAD_ARG;
  if (n_experts > 32 * MAX_E_PER_LANE) return B200Q_ERR_BAD_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int n = n_tokens * k, n_chunks = ceil_div(n, ROUTE_CHUNK);
  route_count_kernel<<<n_chunks, ROUTE_CHUNK, n_experts * sizeof(int), st>>>(topi, n, n_experts, (int32_t*)scratch);
  route_scan_kernel<<<1, 256, n_experts * sizeof(int), st>>>((int32_t*)scratch, n_chunks, n_experts, off, pad, counts);
  route_place_kernel<<<n_chunks, ROUTE_CHUNK, 32 * n_experts * sizeof(int), st>>>(topi, n, n_experts, (const int32_t*)scratch, off, dest_row);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_moe_route_gating(const float* logits, const float* sel_bias, int n_tokens, int n_experts, int k, int gating, int normalize, float scale,
                                      int pad, int32_t* topi, float* weights, int32_t* dest_row, int32_t* off, int32_t* counts, void* scratch, void* stream) {
  if (!logits || !topi || !weights || !dest_row || !off || !scratch || pad <= 0) return B200Q_ERR_BAD_ARG;
  if (n_tokens <= 0 || n_experts <= 0 || k <= 0 || k > n_experts || gating < GATE_SOFTMAX || gating > GATE_SQRT_SOFTPLUS) return B200Q_ERR_BAD_ARG;
  if (n_experts > 32 * MAX_E_PER_LANE || k > 32) return B200Q_ERR_BAD_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int n = n_tokens * k, n_chunks = ceil_div(n, ROUTE_CHUNK);
  route_gating_kernel<<<ceil_div(n_tokens, 8), 256, 0, st>>>(logits, sel_bias, n_tokens, n_experts, k, gating, normalize, scale, topi, weights);
  route_count_kernel<<<n_chunks, ROUTE_CHUNK, n_experts * sizeof(int), st>>>(topi, n, n_experts, (int32_t*)scratch);
  route_scan_kernel<<<1, 256, n_experts * sizeof(int), st>>>((int32_t*)scratch, n_chunks, n_experts, off, pad, counts);
  route_place_kernel<<<n_chunks, ROUTE_CHUNK, 32 * n_experts * sizeof(int), st>>>(topi, n, n_experts, (const int32_t*)scratch, off, dest_row);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_moe_combine(const void* y_bf16, const int32_t* dest_row, const float* weights, int n_tokens, int k, int d, void* out_bf16,
                                 void* stream) {
  if (!y_bf16 || !dest_row || !weights || !out_bf16 || n_tokens <= 0 || k <= 0 || d <= 0) return B200Q_ERR_BAD_ARG;
  if (d % 8 == 0 && !(((uintptr_t)y_bf16 | (uintptr_t)out_bf16) & 15))
    combine8_kernel<<<n_tokens, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y_bf16, dest_row, weights, n_tokens, k, d, (__nv_bfloat16*)out_bf16);
  else
    combine_kernel<<<n_tokens, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y_bf16, dest_row, weights, n_tokens, k, d, (__nv_bfloat16*)out_bf16);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
