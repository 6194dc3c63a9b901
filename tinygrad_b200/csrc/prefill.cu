// Prompt processing (T tokens at once) around the tensor-core GEMMs: the row-wise pieces of Transformer.forward
// (tinygrad/llm/model.py:358-364) and TransformerBlock._attention (model.py:167-198) for T > 1:
//   embed_rows    token_embd[tokens[t]] -> fp32 residual rows                              (model.py:359)
//   rmsnorm_rows  fp32 rows -> RMSNorm * weight, rounded to fp16 (the GEMM operand dtype)   (nn/__init__.py:300-304)
//   rope_kv_rows  rotate q and k of every row (half-split RoPE, model.py:29-33), append k / v to the cache (model.py:200-207)
//   attn_prefill  causal attention of the T new queries over the cache (scaled_dot_product_attention with the causal mask,
//                 model.py:189-195), flash style: mma.sync m16n8k16 fp16 with fp32 accumulation and an online softmax.
// Attention FLOPs are a few percent of a prompt's GEMM FLOPs at these context lengths, so this kernel uses the warp-level
// MMA; the projections around it run on tcgen05 (tc_gemm.cu).
#include "common.cuh"
#include <cuda_bf16.h>

namespace {

__global__ void embed_rows_kernel(const __half* __restrict__ table, const int32_t* __restrict__ tokens, int token_stride, const int32_t* __restrict__ pos_dev,
                                  int n_rows, int dim, int vocab, float* __restrict__ x) {
  const int t = blockIdx.x;
  int tok = tokens[(size_t)t * token_stride + (pos_dev ? *pos_dev : 0)];
  tok = min(max(tok, 0), vocab - 1);
  const __half2* src = reinterpret_cast<const __half2*>(table + (size_t)tok * dim);
  float2* dst = reinterpret_cast<float2*>(x + (size_t)t * dim);
  for (int i = threadIdx.x; i < dim / 2; i += blockDim.x) dst[i] = __half22float2(src[i]);
}

template <typename O> __device__ __forceinline__ O out_cast(float v);
template <> __device__ __forceinline__ __half out_cast<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float out_cast<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 out_cast<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// x[i] += y[i] (bf16): the residual add behind a bf16 expert output (model.py:360 `h + self._feed_forward(...)`)
__global__ void add_rows_bf16_kernel(float* __restrict__ x, const __nv_bfloat16* __restrict__ y, size_t n) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i + 1 < n) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(y + i));
    float2 a = *reinterpret_cast<float2*>(x + i);
    a.x += v.x; a.y += v.y;
    *reinterpret_cast<float2*>(x + i) = a;
  } else if (i < n) x[i] += __bfloat162float(y[i]);
}

template <typename O>
__global__ void rmsnorm_rows_kernel(const float* __restrict__ x, const __half* __restrict__ w, float eps, int dim, O* __restrict__ out) {
  __shared__ float red[32];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* xr = x + (size_t)t * dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float v = xr[i]; ss += v * v; }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < nw; i++) tot += red[i];
  const float sc = 1.0f / sqrtf(tot / (float)dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[(size_t)t * dim + i] = out_cast<O>(xr[i] * sc * __half2float(w[i]));
}

template <typename KV> __device__ __forceinline__ KV kv_cast(float v);
template <> __device__ __forceinline__ __half kv_cast<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float kv_cast<float>(float v) { return v; }

// qkv [T][(n_heads + 2 n_kv) * hd] fp32 -> q_out [T][n_heads * hd] fp32 (rotated), cache rows start_pos + t
template <typename KV>
__global__ void rope_kv_rows_kernel(const float* __restrict__ qkv, const float* __restrict__ rope, int start_pos, int n_heads, int n_kv, int hd,
                                    int rope_dim, int max_context, KV* __restrict__ k_cache, KV* __restrict__ v_cache, float* __restrict__ q_out, int batch,
                                    const int32_t* __restrict__ pos_dev) {
  if (pos_dev) start_pos = min(max(*pos_dev, 0), max_context - 1);      // position kept on the device (graph replay)
  // batch = 0: row t is the token at position start_pos + t of one sequence; batch = 1: row t is sequence t's token at start_pos
  const int t = blockIdx.x, pos = start_pos + (batch ? 0 : t), half_r = rope_dim >> 1;
  if (batch) { k_cache += (size_t)t * n_kv * max_context * hd; v_cache += (size_t)t * n_kv * max_context * hd; }
  const int row = (n_heads + 2 * n_kv) * hd;
  const float* src = qkv + (size_t)t * row;
  const float* rp = rope + (size_t)pos * rope_dim;
  // gridDim.y CTAs share a row (few rows, as in batched decode: one element per thread instead of a long loop per CTA)
  const int tid = blockIdx.y * blockDim.x + threadIdx.x, nthr = gridDim.y * blockDim.x;
  for (int i = tid; i < (n_heads + n_kv) * hd; i += nthr) {
    const int h = i / hd, d = i - h * hd;
    const float* v = src + (size_t)h * hd;
    float o = v[d];
    if (d < half_r) o = v[d] * rp[d] - v[d + half_r] * rp[half_r + d];
    else if (d < rope_dim) o = v[d] * rp[d - half_r] + v[d - half_r] * rp[d];
    if (h < n_heads) q_out[(size_t)t * n_heads * hd + i] = o;
    else k_cache[((size_t)(h - n_heads) * max_context + pos) * hd + d] = kv_cast<KV>(o);
  }
  const float* vs = src + (size_t)(n_heads + n_kv) * hd;
  for (int i = tid; i < n_kv * hd; i += nthr) {
    const int h = i / hd, d = i - h * hd;
    v_cache[((size_t)h * max_context + pos) * hd + d] = kv_cast<KV>(vs[i]);
  }
}

// ---------------------------------------------------------------------------
// causal attention of T queries (positions start_pos .. start_pos+T-1) over cache rows 0 .. start_pos+T-1.
// grid (n_heads, ceil(T / 64)); 4 warps, 16 query rows each; key chunks of 64 staged in shared memory as fp16.
constexpr int PQ = 64, PK = 64, PF_THREADS = 128;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD, typename KV, typename O>
__global__ void __launch_bounds__(PF_THREADS) attn_prefill_kernel(const float* __restrict__ q, const KV* __restrict__ k_cache, const KV* __restrict__ v_cache,
                                                                  int start_pos, int n_rows, int n_heads, int n_kv, int max_context,
                                                                  O* __restrict__ out, int batch, const int32_t* __restrict__ pos_dev) {
  if (pos_dev) start_pos = min(max(*pos_dev, 0), max_context - 1);
  constexpr int STRIDE = HD + 8;                         // halves per shared row: 32-bit fragment loads hit distinct banks
  extern __shared__ __align__(16) unsigned char psm[];
  __half* s_q = reinterpret_cast<__half*>(psm);          // [2][PQ][STRIDE]: fp16 high and low halves of the fp32 queries
  __half* s_k = s_q + 2 * PQ * STRIDE;                   // [PK][STRIDE]
  __half* s_v = s_k + PK * STRIDE;                       // [PK][STRIDE]
  // batch = 1 (one new token per sequence, all at start_pos): the CTA serves row blockIdx.y alone, on that sequence's cache
  const int head = blockIdx.x, q0 = batch ? blockIdx.y : blockIdx.y * PQ, kvh = head / (n_heads / n_kv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int rows_end = batch ? q0 + 1 : n_rows;                       // rows of this tile are q0 .. min(q0 + PQ, rows_end) - 1
  const int pos0 = start_pos + (batch ? 0 : q0);                     // position of the tile's first row
  const size_t seq_off = batch ? (size_t)q0 * n_kv * max_context * HD : 0;
  const KV* kc = k_cache + seq_off + (size_t)kvh * max_context * HD;
  const KV* vc = v_cache + seq_off + (size_t)kvh * max_context * HD;
  // queries of this tile (rows past n_rows read as zero)
  const int q_rows = batch ? 16 : PQ;                    // batch: only warp 0's 16 rows are read (one of them live)
  for (int i = tid; i < q_rows * (HD / 8); i += PF_THREADS) {
    const int r = i / (HD / 8), c = (i - r * (HD / 8)) * 8;
    uint4 hi4 = make_uint4(0, 0, 0, 0), lo4 = make_uint4(0, 0, 0, 0);
    if (q0 + r < rows_end) {
      const float* src = q + ((size_t)(q0 + r) * n_heads + head) * HD + c;
      const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
      const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      uint32_t hw[4], lw[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const __half2 h2 = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
        const float2 back = __half22float2(h2);
        hw[j] = *reinterpret_cast<const uint32_t*>(&h2);
        lw[j] = pack_h2(f[2 * j] - back.x, f[2 * j + 1] - back.y);
      }
      hi4 = make_uint4(hw[0], hw[1], hw[2], hw[3]); lo4 = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
    *reinterpret_cast<uint4*>(s_q + r * STRIDE + c) = hi4;
    *reinterpret_cast<uint4*>(s_q + (PQ + r) * STRIDE + c) = lo4;
  }
  __syncthreads();
  // q = hi + lo (both fp16): the scores keep the fp32 query's precision, as the one-token kernel's fp32 dot products do
  uint32_t qa[HD / 16][4], ql[HD / 16][4];
  {
    const __half* qr = s_q + ((batch ? 0 : warp * 16) + g) * STRIDE + tq * 2;
    const __half* qs = qr + PQ * STRIDE;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      qa[kk][0] = *reinterpret_cast<const uint32_t*>(qr + kk * 16);
      qa[kk][1] = *reinterpret_cast<const uint32_t*>(qr + 8 * STRIDE + kk * 16);
      qa[kk][2] = *reinterpret_cast<const uint32_t*>(qr + kk * 16 + 8);
      qa[kk][3] = *reinterpret_cast<const uint32_t*>(qr + 8 * STRIDE + kk * 16 + 8);
      ql[kk][0] = *reinterpret_cast<const uint32_t*>(qs + kk * 16);
      ql[kk][1] = *reinterpret_cast<const uint32_t*>(qs + 8 * STRIDE + kk * 16);
      ql[kk][2] = *reinterpret_cast<const uint32_t*>(qs + kk * 16 + 8);
      ql[kk][3] = *reinterpret_cast<const uint32_t*>(qs + 8 * STRIDE + kk * 16 + 8);
    }
  }
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int qpos0 = pos0 + warp * 16 + g, qpos1 = qpos0 + 8;                // positions of this lane's two rows
  const int n_keys = pos0 + min(rows_end - q0, PQ);                          // keys any row of the tile may see
  const float scale = 1.0f / sqrtf((float)HD);

  for (int k0 = 0; k0 < n_keys; k0 += PK) {
    __syncthreads();                                     // the previous chunk has been consumed
    for (int i = tid; i < PK * (HD / 8); i += PF_THREADS) {
      const int r = i / (HD / 8), c = (i - r * (HD / 8)) * 8;
      uint4 kk4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
      if (k0 + r < n_keys) {
        if constexpr (sizeof(KV) == 2) {
          kk4 = *reinterpret_cast<const uint4*>(kc + (size_t)(k0 + r) * HD + c);
          vv4 = *reinterpret_cast<const uint4*>(vc + (size_t)(k0 + r) * HD + c);
        } else {
          const float4 a = *reinterpret_cast<const float4*>(kc + (size_t)(k0 + r) * HD + c), b = *reinterpret_cast<const float4*>(kc + (size_t)(k0 + r) * HD + c + 4);
          const float4 e = *reinterpret_cast<const float4*>(vc + (size_t)(k0 + r) * HD + c), f = *reinterpret_cast<const float4*>(vc + (size_t)(k0 + r) * HD + c + 4);
          kk4 = make_uint4(pack_h2(a.x, a.y), pack_h2(a.z, a.w), pack_h2(b.x, b.y), pack_h2(b.z, b.w));
          vv4 = make_uint4(pack_h2(e.x, e.y), pack_h2(e.z, e.w), pack_h2(f.x, f.y), pack_h2(f.z, f.w));
        }
      }
      *reinterpret_cast<uint4*>(s_k + r * STRIDE + c) = kk4;
      *reinterpret_cast<uint4*>(s_v + r * STRIDE + c) = vv4;
    }
    __syncthreads();
    if (k0 > pos0 + warp * 16 + 15) continue;  // every key of the chunk is after this warp's last query
    if (batch && warp > 0) continue;           // one query row per CTA: warps 1..3 only help to stage the keys and values
    // S = Q K^T for 16 rows x 64 keys
    float s[PK / 8][4];
#pragma unroll
    for (int j = 0; j < PK / 8; j++) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const __half* kr = s_k + (j * 8 + g) * STRIDE + tq * 2;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr + kk * 16), b1 = *reinterpret_cast<const uint32_t*>(kr + kk * 16 + 8);
        mma16816(s[j], qa[kk], b0, b1);
        mma16816(s[j], ql[kk], b0, b1);
      }
    }
    // scale, causal mask, online softmax (rows g and g + 8; a row's 64 scores live in the 4 lanes of a quad)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < PK / 8; j++) {
      const int key = k0 + j * 8 + tq * 2;
      s[j][0] = key <= qpos0 ? s[j][0] * scale : -INFINITY;
      s[j][1] = key + 1 <= qpos0 ? s[j][1] * scale : -INFINITY;
      s[j][2] = key <= qpos1 ? s[j][2] * scale : -INFINITY;
      s[j][3] = key + 1 <= qpos1 ? s[j][3] * scale : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    // a row whose keys so far are all masked keeps max = -inf: guard the exponent so that it stays 0, not NaN
    const float c0 = mn0 == -INFINITY ? 0.f : __expf(m0 - mn0), c1 = mn1 == -INFINITY ? 0.f : __expf(m1 - mn1);
    const float b0 = mn0 == -INFINITY ? 0.f : mn0, b1 = mn1 == -INFINITY ? 0.f : mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < PK / 8; j++) {
      s[j][0] = __expf(s[j][0] - b0); s[j][1] = __expf(s[j][1] - b0);
      s[j][2] = __expf(s[j][2] - b1); s[j][3] = __expf(s[j][3] - b1);
      sum0 += s[j][0] + s[j][1]; sum1 += s[j][2] + s[j][3];
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * c0 + sum0; l1 = l1 * c1 + sum1; m0 = mn0; m1 = mn1;
#pragma unroll
    for (int j = 0; j < HD / 8; j++) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    // O += P V: P from the score fragments (fp16), V through transposing ldmatrix
#pragma unroll
    for (int kk = 0; kk < PK / 16; kk++) {
      // probabilities as fp16 hi + lo as well (two MMAs per tile): their rounding would otherwise be the largest error left
      uint32_t pa[4], pl[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float a = s[2 * kk + (e >> 1)][(e & 1) * 2], b = s[2 * kk + (e >> 1)][(e & 1) * 2 + 1];
        const __half2 h2 = __floats2half2_rn(a, b);
        const float2 back = __half22float2(h2);
        pa[e] = *reinterpret_cast<const uint32_t*>(&h2);
        pl[e] = pack_h2(a - back.x, b - back.y);
      }
#pragma unroll
      for (int n0 = 0; n0 < HD; n0 += 16) {
        // four 8x8 blocks: keys kk*16 + {0..7, 8..15} x dims n0 + {0..7, 8..15}; lane l supplies the row address of block l / 8
        const __half* vp = s_v + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * STRIDE + n0 + (lane >> 4) * 8;
        uint32_t r0, r1, r2, r3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"((uint32_t)__cvta_generic_to_shared(vp)));
        mma16816(o[n0 / 8], pa, r0, r1);
        mma16816(o[n0 / 8], pl, r0, r1);
        mma16816(o[n0 / 8 + 1], pa, r2, r3);
        mma16816(o[n0 / 8 + 1], pl, r2, r3);
      }
    }
  }
  const float i0 = 1.f / l0, i1 = 1.f / l1;
  const int r0 = q0 + warp * 16 + g, r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < HD / 8; j++) {
    const int d = j * 8 + tq * 2;
    if (r0 < rows_end) { O* dst = out + ((size_t)r0 * n_heads + head) * HD + d; dst[0] = out_cast<O>(o[j][0] * i0); dst[1] = out_cast<O>(o[j][1] * i0); }
    if (r1 < rows_end) { O* dst = out + ((size_t)r1 * n_heads + head) * HD + d; dst[0] = out_cast<O>(o[j][2] * i1); dst[1] = out_cast<O>(o[j][3] * i1); }
  }
}

template <int HD, typename KV, typename O>
cudaError_t launch_prefill_attn2(const void* q, const void* kc, const void* vc, int start_pos, int n_rows, int n_heads, int n_kv, int max_context, void* out,
                                 int batch, const int32_t* pos_dev, cudaStream_t st) {
  const size_t smem = (size_t)(2 * PQ + 2 * PK) * (HD + 8) * sizeof(__half);
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD, KV, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  attn_prefill_kernel<HD, KV, O><<<dim3(n_heads, batch ? n_rows : ceil_div(n_rows, PQ)), PF_THREADS, smem, st>>>(
      (const float*)q, (const KV*)kc, (const KV*)vc, start_pos, n_rows, n_heads, n_kv, max_context, (O*)out, batch, pos_dev);
  return cudaGetLastError();
}
template <int HD, typename KV>
cudaError_t launch_prefill_attn(const void* q, const void* kc, const void* vc, int start_pos, int n_rows, int n_heads, int n_kv, int max_context, void* out,
                                bool out_f16, int batch, const int32_t* pos_dev, cudaStream_t st) {
  return out_f16 ? launch_prefill_attn2<HD, KV, __half>(q, kc, vc, start_pos, n_rows, n_heads, n_kv, max_context, out, batch, pos_dev, st)
                 : launch_prefill_attn2<HD, KV, float>(q, kc, vc, start_pos, n_rows, n_heads, n_kv, max_context, out, batch, pos_dev, st);
}

}  // namespace

extern "C" int b200q_embed_rows(const void* table_f16, const int32_t* tokens, int token_stride, const int32_t* pos_dev, int n_rows, int dim, int vocab,
                                float* x, void* stream) {
  if (!table_f16 || !tokens || !x || n_rows <= 0 || dim <= 0 || vocab <= 0 || token_stride < 0) return B200Q_ERR_BAD_ARG;
  if (dim % 2) return B200Q_ERR_BAD_SHAPE;
  embed_rows_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>((const __half*)table_f16, tokens, token_stride, pos_dev, n_rows, dim, vocab, x);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_rmsnorm_rows(const float* x, const void* weight_f16, float eps, int n_rows, int dim, void* out, int out_dtype, void* stream) {
  if (!x || !weight_f16 || !out || n_rows <= 0 || dim <= 0) return B200Q_ERR_BAD_ARG;
  if (out_dtype != B200Q_F16 && out_dtype != B200Q_F32 && out_dtype != B200Q_BF16) return B200Q_ERR_BAD_ARG;
  if (out_dtype == B200Q_BF16) rmsnorm_rows_kernel<__nv_bfloat16><<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, (const __half*)weight_f16, eps, dim,
                                                                                                           (__nv_bfloat16*)out);
  else if (out_dtype == B200Q_F16) rmsnorm_rows_kernel<__half><<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, (const __half*)weight_f16, eps, dim, (__half*)out);
  else rmsnorm_rows_kernel<float><<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, (const __half*)weight_f16, eps, dim, (float*)out);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

// x[r][c] += y[r][c] * (gate ? sigmoid(gate[r]) : 1): the shared expert's output joining the residual stream (tinygrad/llm/model.py:131-134)
__global__ void add_rows_gated_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gate, int n_rows, int dim) {
  const int r = blockIdx.x;
  const float g = gate ? 1.f / (1.f + expf(-gate[r])) : 1.f;
  for (int c = threadIdx.x; c < dim; c += blockDim.x) x[(size_t)r * dim + c] += y[(size_t)r * dim + c] * g;
}

extern "C" int b200q_add_rows_gated(float* x, const float* y, const float* gate_logit, int n_rows, int dim, void* stream) {
  if (!x || !y || n_rows < 0 || dim <= 0) return B200Q_ERR_BAD_ARG;
  if (n_rows == 0) return B200Q_OK;
  add_rows_gated_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, y, gate_logit, n_rows, dim);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_add_rows_bf16(float* x, const void* y_bf16, int64_t n, void* stream) {
  if (!x || !y_bf16 || n < 0) return B200Q_ERR_BAD_ARG;
  if (((uintptr_t)x & 7) || ((uintptr_t)y_bf16 & 3)) return B200Q_ERR_MISALIGNED;
  if (n == 0) return B200Q_OK;
  add_rows_bf16_kernel<<<(unsigned)((n / 2 + 256) / 256), 256, 0, (cudaStream_t)stream>>>(x, (const __nv_bfloat16*)y_bf16, (size_t)n);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

static int attn_rows(const float* qkv, void* k_cache, void* v_cache, int kv_dtype, const float* rope, int start_pos, int n_rows, int n_heads,
                     int n_kv_heads, int head_dim, int rope_dim, int max_context, void* q_scratch, void* out, int out_dtype, int batch,
                     const int32_t* pos_dev, void* stream) {
  if (!qkv || !k_cache || !v_cache || !rope || !q_scratch || !out || (out_dtype != B200Q_F16 && out_dtype != B200Q_F32)) return B200Q_ERR_BAD_ARG;
  const bool of16 = out_dtype == B200Q_F16;
  if (n_rows <= 0 || start_pos < 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return B200Q_ERR_BAD_ARG;
  if (kv_dtype != B200Q_F16 && kv_dtype != B200Q_F32) return B200Q_ERR_BAD_ARG;
  if (start_pos + (batch ? 1 : n_rows) > max_context) return B200Q_ERR_TOO_LARGE;
  if (rope_dim < 0 || rope_dim > head_dim || rope_dim % 2) return B200Q_ERR_BAD_SHAPE;
  if (head_dim != 16 && head_dim != 32 && head_dim != 64 && head_dim != 128) return B200Q_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  const bool h = kv_dtype == B200Q_F16;
  const int row_ctas = n_rows >= 64 ? 1 : ceil_div((n_heads + n_kv_heads) * head_dim, 256);
  const dim3 rgrid(n_rows, row_ctas);
  if (h) rope_kv_rows_kernel<__half><<<rgrid, 256, 0, st>>>(qkv, rope, start_pos, n_heads, n_kv_heads, head_dim, rope_dim, max_context, (__half*)k_cache,
                                                           (__half*)v_cache, (float*)q_scratch, batch, pos_dev);
  else rope_kv_rows_kernel<float><<<rgrid, 256, 0, st>>>(qkv, rope, start_pos, n_heads, n_kv_heads, head_dim, rope_dim, max_context, (float*)k_cache,
                                                        (float*)v_cache, (float*)q_scratch, batch, pos_dev);
  B200Q_CHECK_CUDA(cudaGetLastError());
  cudaError_t e;
#define PF_CASE(HD)                                                                                                                     \
  case HD: e = h ? launch_prefill_attn<HD, __half>(q_scratch, k_cache, v_cache, start_pos, n_rows, n_heads, n_kv_heads, max_context, out, of16, batch, pos_dev, st)  \
                 : launch_prefill_attn<HD, float>(q_scratch, k_cache, v_cache, start_pos, n_rows, n_heads, n_kv_heads, max_context, out, of16, batch, pos_dev, st); break;
  switch (head_dim) { PF_CASE(16) PF_CASE(32) PF_CASE(64) default: PF_CASE(128) }
#undef PF_CASE
  B200Q_CHECK_CUDA(e);
  return B200Q_OK;
}

extern "C" int b200q_attn_prefill(const float* qkv, void* k_cache, void* v_cache, int kv_dtype, const float* rope, int start_pos, int n_rows,
                                  int n_heads, int n_kv_heads, int head_dim, int rope_dim, int max_context, void* q_scratch, void* out,
                                  int out_dtype, void* stream) {
  return attn_rows(qkv, k_cache, v_cache, kv_dtype, rope, start_pos, n_rows, n_heads, n_kv_heads, head_dim, rope_dim, max_context, q_scratch, out, out_dtype, 0,
                   nullptr, stream);
}

extern "C" int b200q_attn_decode_batch(const float* qkv, void* k_cache, void* v_cache, int kv_dtype, const float* rope, int pos, const int32_t* pos_dev,
                                       int n_seqs, int n_heads, int n_kv_heads, int head_dim, int rope_dim, int max_context, void* q_scratch, void* out,
                                       int out_dtype, void* stream) {
  return attn_rows(qkv, k_cache, v_cache, kv_dtype, rope, pos_dev ? 0 : pos, n_seqs, n_heads, n_kv_heads, head_dim, rope_dim, max_context, q_scratch, out,
                   out_dtype, 1, pos_dev, stream);
}
