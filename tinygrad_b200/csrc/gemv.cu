// Weight-dequant-fused GEMV for GGUF Q4_0 / Q8_0 weights (decode: one activation row).
//
// Replaces the kernels tinygrad generates for `Linear.__call__` on a lazily
// dequantised GGUF weight (tinygrad/nn/__init__.py:177 over tinygrad/llm/gguf.py:46,56).
//
// Data flow per CTA: the activation row is staged once into shared memory as fp16
// hi + lo halves (x = hi + lo to ~22 bits, so the product keeps fp32-grade accuracy);
// each warp then streams whole weight tiles (16 rows x 4 quant blocks) with 128-bit
// coalesced loads, unpacks nibbles/bytes to exact fp16 integers in registers and
// feeds them to mma.m16n8k16: the 8 accumulator columns are the 4 blocks of the tile
// times {hi, lo}, i.e. B is block-diagonal, so every block's integer dot product
// lands in its own column and is scaled by that block's fp16 scale afterwards.
// The k-reduction happens inside the MMA and across the 4 lanes of a quad (warp
// shuffles), then across warps through shared memory, in a fixed order
// (bit-reproducible).  The kernel is HBM-bound: the MMA only removes the
// per-element FMA from the issue slots.
#include "common.cuh"

namespace {

struct GemvParams {
  const uint8_t* w;
  const void* x;
  const __half* norm_w;
  const __half* bias;
  const float* residual;
  void* y;
  int n_out, n_in, kgroups, n_row_tiles;
  int x_f16, y_f16, epilogue;
  float eps;
};

constexpr int NWARPS = 8;
constexpr int NTHREADS = NWARPS * 32;

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {   // (a & b) | c
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
  uint32_t d; asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel)); return d;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Where element e (0..31) of a quant block sits among the 16 B-fragment registers
// a lane holds for that block: register q (0..15) and half slot (0 = low 16 bits).
template <int QT> __device__ __forceinline__ void b_slot(int e, int& q, int& hs);
template <> __device__ __forceinline__ void b_slot<B200Q_Q4_0>(int e, int& q, int& hs) {
  // byte i of the 16 quant bytes holds element i (low nibble) and i+16 (high nibble); word i/4 feeds
  // one MMA with its low nibbles and the next with its high nibbles: regs {e0,e2}, {e1,e3}
  int hl = e >> 4, i = (e & 15) >> 2, r = e & 3;
  q = (2 * i + hl) * 2 + (r & 1); hs = r >> 1;
}
template <> __device__ __forceinline__ void b_slot<B200Q_Q8_0>(int e, int& q, int& hs) { q = e >> 1; hs = e & 1; }

template <int QT> struct Frag;
template <> struct Frag<B200Q_Q4_0> { uint4 lo, hi; uint2 sc; };            // rows g / g+8
template <> struct Frag<B200Q_Q8_0> { uint4 lo0, lo1, hi0, hi1; uint2 sc; };

template <int QT> __device__ __forceinline__ void load_frag(Frag<QT>& f, const uint8_t* tile, int lane);
template <> __device__ __forceinline__ void load_frag<B200Q_Q4_0>(Frag<B200Q_Q4_0>& f, const uint8_t* tile, int lane) {
  const uint4* tp = reinterpret_cast<const uint4*>(tile);
  f.lo = ldg_stream(tp + lane); f.hi = ldg_stream(tp + 32 + lane);
  f.sc = ldg_stream(reinterpret_cast<const uint2*>(tile + 1024) + (2 * (lane >> 2) + (lane & 1)));
}
template <> __device__ __forceinline__ void load_frag<B200Q_Q8_0>(Frag<B200Q_Q8_0>& f, const uint8_t* tile, int lane) {
  const uint4* tp = reinterpret_cast<const uint4*>(tile);
  f.lo0 = ldg_stream(tp + lane); f.lo1 = ldg_stream(tp + 32 + lane);
  f.hi0 = ldg_stream(tp + 64 + lane); f.hi1 = ldg_stream(tp + 96 + lane);
  f.sc = ldg_stream(reinterpret_cast<const uint2*>(tile + 2048) + (2 * (lane >> 2) + (lane & 1)));
}

// One Q4_0 word pair (rows g and g+8): low-nibble MMA then high-nibble MMA.
__device__ __forceinline__ void q4_word(float (&c)[4], uint32_t w0, uint32_t w1, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  const uint32_t MAGIC = 0x64006400u;        // half2(1024, 1024): nibble lands in the mantissa
  const uint32_t SUB_LO = 0x64086408u;       // half2(1032): (1024 + n) - 1032 = n - 8
  const uint32_t MUL_HI = 0x2C002C00u;       // half2(1/16)
  const uint32_t ADD_HI = 0xD480D480u;       // half2(-72): (1024 + 16 n) / 16 - 72 = n - 8
  uint32_t v0 = w0 >> 8, v1 = w1 >> 8;
  uint32_t a0 = h2_sub(lop3_and_or(w0, 0x000F000Fu, MAGIC), SUB_LO), a1 = h2_sub(lop3_and_or(w1, 0x000F000Fu, MAGIC), SUB_LO);
  uint32_t a2 = h2_sub(lop3_and_or(v0, 0x000F000Fu, MAGIC), SUB_LO), a3 = h2_sub(lop3_and_or(v1, 0x000F000Fu, MAGIC), SUB_LO);
  mma16816(c, a0, a1, a2, a3, b0, b1);
  a0 = h2_fma(lop3_and_or(w0, 0x00F000F0u, MAGIC), MUL_HI, ADD_HI); a1 = h2_fma(lop3_and_or(w1, 0x00F000F0u, MAGIC), MUL_HI, ADD_HI);
  a2 = h2_fma(lop3_and_or(v0, 0x00F000F0u, MAGIC), MUL_HI, ADD_HI); a3 = h2_fma(lop3_and_or(v1, 0x00F000F0u, MAGIC), MUL_HI, ADD_HI);
  mma16816(c, a0, a1, a2, a3, b2, b3);
}
// One Q8_0 word pair: 4 sign-flipped bytes per row -> exact fp16 integers.
__device__ __forceinline__ void q8_word(float (&c)[4], uint32_t w0, uint32_t w1, uint32_t b0, uint32_t b1) {
  const uint32_t HI = 0x64646464u, SUB = 0x64806480u;   // 0x64bb = 1024 + bb; minus 1152 = int8 value
  uint32_t a0 = h2_sub(prmt(w0, HI, 0x4140u), SUB), a1 = h2_sub(prmt(w1, HI, 0x4140u), SUB);
  uint32_t a2 = h2_sub(prmt(w0, HI, 0x4342u), SUB), a3 = h2_sub(prmt(w1, HI, 0x4342u), SUB);
  mma16816(c, a0, a1, a2, a3, b0, b1);
}

template <int QT> __device__ __forceinline__ void compute_frag(const Frag<QT>& f, const uint4 (&bf)[4], float& acc0, float& acc1);
template <> __device__ __forceinline__ void compute_frag<B200Q_Q4_0>(const Frag<B200Q_Q4_0>& f, const uint4 (&bf)[4], float& acc0, float& acc1) {
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  q4_word(c, f.lo.x, f.hi.x, bf[0].x, bf[0].y, bf[0].z, bf[0].w);
  q4_word(c, f.lo.y, f.hi.y, bf[1].x, bf[1].y, bf[1].z, bf[1].w);
  q4_word(c, f.lo.z, f.hi.z, bf[2].x, bf[2].y, bf[2].z, bf[2].w);
  q4_word(c, f.lo.w, f.hi.w, bf[3].x, bf[3].y, bf[3].z, bf[3].w);
  float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&f.sc.x)), d1 = __half22float2(*reinterpret_cast<const __half2*>(&f.sc.y));
  acc0 = fmaf(c[0], d0.x, fmaf(c[1], d0.y, acc0));
  acc1 = fmaf(c[2], d1.x, fmaf(c[3], d1.y, acc1));
}
template <> __device__ __forceinline__ void compute_frag<B200Q_Q8_0>(const Frag<B200Q_Q8_0>& f, const uint4 (&bf)[4], float& acc0, float& acc1) {
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  q8_word(c, f.lo0.x, f.hi0.x, bf[0].x, bf[0].y); q8_word(c, f.lo0.y, f.hi0.y, bf[0].z, bf[0].w);
  q8_word(c, f.lo0.z, f.hi0.z, bf[1].x, bf[1].y); q8_word(c, f.lo0.w, f.hi0.w, bf[1].z, bf[1].w);
  q8_word(c, f.lo1.x, f.hi1.x, bf[2].x, bf[2].y); q8_word(c, f.lo1.y, f.hi1.y, bf[2].z, bf[2].w);
  q8_word(c, f.lo1.z, f.hi1.z, bf[3].x, bf[3].y); q8_word(c, f.lo1.w, f.hi1.w, bf[3].z, bf[3].w);
  float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&f.sc.x)), d1 = __half22float2(*reinterpret_cast<const __half2*>(&f.sc.y));
  acc0 = fmaf(c[0], d0.x, fmaf(c[1], d0.y, acc0));
  acc1 = fmaf(c[2], d1.x, fmaf(c[3], d1.y, acc1));
}

template <int QT, int U>
__global__ void __launch_bounds__(NTHREADS) qgemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint4* xs = reinterpret_cast<uint4*>(smem);                                   // [kgroups][4][8] B-fragment words
  float* red = reinterpret_cast<float*>(smem + (size_t)p.kgroups * 512);        // [NWARPS][16]
  float* fin = red + NWARPS * 16;                                               // [16]
  float* s_ss = fin + 16;                                                       // [NWARPS] + [1]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int m = blockIdx.y;
  constexpr int TB = tile_bytes(QT);

  pdl_launch_dependents();

  // weights do not depend on the previous kernel: start streaming the first chunk before waiting for it
  int rt = blockIdx.x;
  Frag<QT> fr[U];
#pragma unroll
  for (int u = 0; u < U; u++) {
    int j = warp + u * NWARPS;
    if (rt < p.n_row_tiles && j < p.kgroups) load_frag<QT>(fr[u], p.w + ((size_t)rt * p.kgroups + j) * TB, lane);
  }
  pdl_wait();

  // ---- stage the activation row: x (* norm weight) -> fp16 hi/lo B fragments
  {
    const int kpad = p.kgroups * GROUP_ELEMS;
    __half* xh = reinterpret_cast<__half*>(xs);
    float ss = 0.f;
    for (int k = tid; k < kpad; k += NTHREADS) {
      float v = 0.f;
      if (k < p.n_in) {
        v = p.x_f16 ? __half2float(reinterpret_cast<const __half*>(p.x)[(size_t)m * p.n_in + k])
                    : reinterpret_cast<const float*>(p.x)[(size_t)m * p.n_in + k];
        ss = fmaf(v, v, ss);
        if (p.norm_w) v *= __half2float(p.norm_w[k]);
      }
      __half hi = __float2half_rn(v), lo = __float2half_rn(v - __half2float(hi));
      int b = k >> 5, e = k & 31, j = b >> 2, tb = b & 3, q, hs;
      b_slot<QT>(e, q, hs);
      int base = ((j * 4 + (q >> 2)) * 8) * 8 + (q & 3) * 2 + hs;   // half index of lane-slot 0
      xh[base + tb * 8] = hi;
      xh[base + (tb + 4) * 8] = lo;
    }
    if (p.norm_w) {
      ss = warp_sum(ss);
      if (lane == 0) s_ss[warp] = ss;
    }
  }
  __syncthreads();
  float rs = 1.f;
  if (p.norm_w) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; w++) tot += s_ss[w];
    rs = rsqrtf(tot / (float)p.n_in + p.eps);
  }
  const bool b_active = (t == (g & 3));

  bool first = true;
  for (; rt < p.n_row_tiles; rt += gridDim.x) {
    float acc0 = 0.f, acc1 = 0.f;
    for (int jb = warp; jb < p.kgroups; jb += NWARPS * U) {
      if (!first) {
#pragma unroll
        for (int u = 0; u < U; u++) {
          int j = jb + u * NWARPS;
          if (j < p.kgroups) load_frag<QT>(fr[u], p.w + ((size_t)rt * p.kgroups + j) * TB, lane);
        }
      }
      first = false;
#pragma unroll
      for (int u = 0; u < U; u++) {
        int j = jb + u * NWARPS;
        if (j < p.kgroups) {
          uint4 bf[4];
#pragma unroll
          for (int c = 0; c < 4; c++) bf[c] = b_active ? xs[(j * 4 + c) * 8 + g] : make_uint4(0, 0, 0, 0);
          compute_frag<QT>(fr[u], bf, acc0, acc1);
        }
      }
    }
    first = false;
    // quad lanes hold the columns {blocks 0,1 hi}, {2,3 hi}, {0,1 lo}, {2,3 lo}: add them
    acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1); acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
    acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1); acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
    if (t == 0) { red[warp * 16 + g] = acc0; red[warp * 16 + 8 + g] = acc1; }
    __syncthreads();
    if (tid < 16) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < NWARPS; w++) v += red[w * 16 + tid];
      v *= rs;
      if (p.epilogue == B200Q_EPI_LINEAR) {
        int row = rt * 16 + tid;
        if (row < p.n_out) {
          if (p.bias) v += __half2float(p.bias[row]);
          if (p.residual) v += p.residual[(size_t)m * p.n_out + row];
          if (p.y_f16) reinterpret_cast<__half*>(p.y)[(size_t)m * p.n_out + row] = __float2half_rn(v);
          else reinterpret_cast<float*>(p.y)[(size_t)m * p.n_out + row] = v;
        }
      } else {
        fin[tid] = v;
      }
    }
    if (p.epilogue == B200Q_EPI_SILU_MUL) {
      __syncthreads();
      if (tid < 8) {
        int row = rt * 8 + tid;
        if (row < p.n_out) {
          float gt = fin[tid], up = fin[tid + 8];
          float v = (gt / (1.f + __expf(-gt))) * up;
          if (p.y_f16) reinterpret_cast<__half*>(p.y)[(size_t)m * p.n_out + row] = __float2half_rn(v);
          else reinterpret_cast<float*>(p.y)[(size_t)m * p.n_out + row] = v;
        }
      }
    }
    __syncthreads();
  }
}

template <int QT, int U>
int launch_gemv(const b200q_gemv_args* a, const GemvParams& p, cudaStream_t stream) {
  size_t smem = (size_t)p.kgroups * 512 + (NWARPS * 16 + 16 + NWARPS + 1) * sizeof(float);
  if (smem > 220 * 1024) return B200Q_ERR_TOO_LARGE;
  auto kern = qgemv_kernel<QT, U>;
  static int sm_count = 0;
  static size_t smem_set = 0;
  if (sm_count == 0) {
    int dev; B200Q_CHECK_CUDA(cudaGetDevice(&dev));
    B200Q_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  if (smem > 48 * 1024 && smem > smem_set) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    smem_set = 220 * 1024;
  }
  int occ = 0;
  B200Q_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, NTHREADS, smem));
  if (occ < 1) occ = 1;
  int max_ctas = a->max_ctas > 0 ? a->max_ctas : occ * sm_count;
  int grid_x = p.n_row_tiles < max_ctas ? p.n_row_tiles : max_ctas;
  B200Q_CHECK_CUDA(launch_k(kern, dim3(grid_x, a->m), dim3(NTHREADS), smem, stream, (a->flags & B200Q_FLAG_PDL) != 0, p));
  return B200Q_OK;
}

}  // namespace

extern "C" int b200q_gemv(const b200q_gemv_args* a, void* stream) {
  if (!a || !a->w_packed || !a->x || !a->y) return B200Q_ERR_BAD_ARG;
  if (a->qtype == B200Q_Q6_K) return B200Q_ERR_UNSUPPORTED;
  if (a->qtype != B200Q_Q4_0 && a->qtype != B200Q_Q8_0) return B200Q_ERR_BAD_ARG;
  if (a->n_out <= 0 || a->n_in <= 0 || a->m <= 0 || a->m > 65535) return B200Q_ERR_BAD_ARG;
  if (a->n_in % 32) return B200Q_ERR_BAD_SHAPE;
  if ((a->x_dtype != B200Q_F32 && a->x_dtype != B200Q_F16) || (a->y_dtype != B200Q_F32 && a->y_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (a->epilogue != B200Q_EPI_LINEAR && a->epilogue != B200Q_EPI_SILU_MUL) return B200Q_ERR_BAD_ARG;
  if (a->epilogue == B200Q_EPI_SILU_MUL && (a->bias || a->residual)) return B200Q_ERR_UNSUPPORTED;
  if ((uintptr_t)a->w_packed & 15) return B200Q_ERR_MISALIGNED;
  if (((uintptr_t)a->x & (a->x_dtype == B200Q_F32 ? 3 : 1)) || ((uintptr_t)a->y & (a->y_dtype == B200Q_F32 ? 3 : 1))) return B200Q_ERR_MISALIGNED;
  GemvParams p;
  p.w = (const uint8_t*)a->w_packed; p.x = a->x; p.norm_w = (const __half*)a->norm_weight; p.bias = (const __half*)a->bias;
  p.residual = (const float*)a->residual; p.y = a->y;
  p.n_out = a->n_out; p.n_in = a->n_in; p.kgroups = ceil_div(a->n_in, GROUP_ELEMS);
  p.n_row_tiles = a->epilogue == B200Q_EPI_SILU_MUL ? ceil_div(a->n_out, 8) : ceil_div(a->n_out, TILE_ROWS);
  p.x_f16 = a->x_dtype == B200Q_F16; p.y_f16 = a->y_dtype == B200Q_F16; p.epilogue = a->epilogue; p.eps = a->norm_eps;
  if (a->qtype == B200Q_Q4_0) return launch_gemv<B200Q_Q4_0, 4>(a, p, (cudaStream_t)stream);
  return launch_gemv<B200Q_Q8_0, 2>(a, p, (cudaStream_t)stream);
}
