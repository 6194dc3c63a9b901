// GGUF block formats: bit-exact dequantisation and the one-time lossless re-tiling
// into the layout the GEMV kernels stream (layout described in include/b200q.h).
// Semantics follow tinygrad/llm/gguf.py:38-72 (q_to_uint8, Q4_0 :46, Q4_1 :47-49, Q5_0 / Q5_1 :50-55, Q8_0 :56, Q4_K / Q5_K :57-67, Q6_K :68-72).
#include "common.cuh"

// ---------------------------------------------------------------------------
// raw GGUF blocks -> values.  One thread per element; fp32 results are single
// IEEE multiplies in the reference's order, so they are bit-identical to it.
template <typename OutT>
__device__ __forceinline__ void store_val(OutT* out, int64_t i, float v);
template <> __device__ __forceinline__ void store_val<float>(float* out, int64_t i, float v) { out[i] = v; }
template <> __device__ __forceinline__ void store_val<__half>(__half* out, int64_t i, float v) { out[i] = __float2half_rn(v); }

__device__ __forceinline__ float load_f16(const uint8_t* p) {
  return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

template <typename OutT>
__global__ void dequant_raw_kernel(int qtype, const uint8_t* __restrict__ raw, OutT* __restrict__ out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v;
  if (qtype == B200Q_Q4_0) {
    // element e of a block: low nibble of byte e (e < 16) or high nibble of byte e-16
    const uint8_t* b = raw + (i >> 5) * 18; int e = (int)(i & 31);
    int nib = (b[2 + (e & 15)] >> ((e >> 4) * 4)) & 0xF;
    v = __fmul_rn((float)(nib - 8), load_f16(b));
  } else if (qtype == B200Q_Q8_0) {
    const uint8_t* b = raw + (i >> 5) * 34; int e = (int)(i & 31);
    v = __fmul_rn(load_f16(b), (float)(int8_t)b[2 + e]);
  } else if (qtype == B200Q_Q4_1) {     // gguf.py:47-49: nibble * d + m; block = d, m, 16 quant bytes
    const uint8_t* b = raw + (i >> 5) * 20; int e = (int)(i & 31);
    int nib = (b[4 + (e & 15)] >> ((e >> 4) * 4)) & 0xF;
    v = __fadd_rn(__fmul_rn((float)nib, load_f16(b)), load_f16(b + 2));
  } else if (qtype == B200Q_Q5_0 || qtype == B200Q_Q5_1) {      // gguf.py:50-55: (nibble + 16 * high bit) * d + (m | -16 d)
    const int off = qtype == B200Q_Q5_0 ? 2 : 4;
    const uint8_t* b = raw + (i >> 5) * (qtype == B200Q_Q5_0 ? 22 : 24); int e = (int)(i & 31);
    const uint32_t qh = b[off] | (b[off + 1] << 8) | (b[off + 2] << 16) | ((uint32_t)b[off + 3] << 24);
    int q = ((b[off + 4 + (e & 15)] >> ((e >> 4) * 4)) & 0xF) + 16 * (int)((qh >> e) & 1);
    const float d = load_f16(b);
    v = __fadd_rn(__fmul_rn((float)q, d), qtype == B200Q_Q5_1 ? load_f16(b + 2) : __fmul_rn(-16.f, d));
  } else if (qtype == B200Q_Q4_K || qtype == B200Q_Q5_K) {      // gguf.py:57-67: (d * sc) * q - dmin * mn; 8 groups of 32 with 6-bit scales / mins
    const uint8_t* b = raw + (i >> 8) * (qtype == B200Q_Q4_K ? 144 : 176); int e = (int)(i & 255);
    const int grp = e >> 5, j = e & 31;
    const uint8_t* s = b + 4;
    int sc, mn;
    if (grp < 4) { sc = s[grp] & 63; mn = s[4 + grp] & 63; }
    else { sc = (s[4 + grp] & 0xF) | ((s[grp - 4] >> 6) << 4); mn = (s[4 + grp] >> 4) | ((s[grp] >> 6) << 4); }
    const uint8_t* qs = b + (qtype == B200Q_Q5_K ? 48 : 16);
    int q = (qs[(grp >> 1) * 32 + j] >> ((grp & 1) * 4)) & 0xF;
    if (qtype == B200Q_Q5_K) q += 16 * ((b[16 + j] >> grp) & 1);
    v = __fsub_rn(__fmul_rn(__fmul_rn(load_f16(b), (float)sc), (float)q), __fmul_rn(load_f16(b + 2), (float)mn));
  } else {  // Q6_K: 256 elements in 210 bytes: ql[128] qh[64] scales[16] d
    const uint8_t* b = raw + (i >> 8) * 210; int e = (int)(i & 255);
    int hh = e >> 7, m = e & 127;
    int xl = (b[hh * 64 + (m & 63)] >> ((m >> 6) * 4)) & 0xF;
    int xh = (b[128 + hh * 32 + (m & 31)] >> ((m >> 5) * 2)) & 3;
    int q = (int)(int8_t)(xl | (xh << 4)) - 32;
    float sc = (float)(int8_t)b[192 + (e >> 4)];
    v = __fmul_rn(__fmul_rn(load_f16(b + 208), (float)q), sc);   // (d * q) * scales, in that order
  }
  store_val<OutT>(out, i, v);
}

// ---------------------------------------------------------------------------
// re-tiling.  One thread per (tile, half, lane) = one (row, block) pair.
__global__ void repack_kernel(int qtype, const uint8_t* __restrict__ raw0, const uint8_t* __restrict__ raw1, uint8_t* __restrict__ packed,
                              int n_out, int nblk, int n_row_tiles, int kgroups) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)n_row_tiles * kgroups * 64;
  if (idx >= total) return;
  int l = (int)(idx & 31), h = (int)((idx >> 5) & 1);
  int64_t tile = idx >> 6;
  int j = (int)(tile % kgroups), rt = (int)(tile / kgroups);
  int g = l >> 2, t = l & 3;
  int blk = j * 4 + t;
  const uint8_t* src = nullptr;
  int row;
  if (raw1 == nullptr) { row = rt * 16 + h * 8 + g; if (row < n_out && blk < nblk) src = raw0; }
  else { row = rt * 8 + g; if (row < n_out && blk < nblk) src = h ? raw1 : raw0; }
  const int bbytes = qtype == B200Q_Q4_0 ? 18 : 34;
  const int tbytes = tile_bytes(qtype);
  uint8_t* tp = packed + tile * tbytes;
  unsigned short scale = 0;   // fp16 zero: a padded block contributes nothing
  if (qtype == B200Q_Q4_0) {
    uint32_t w[4] = {0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};   // nibble 8 == value 0
    if (src) {
      const uint8_t* b = src + ((int64_t)row * nblk + blk) * bbytes;
      scale = (unsigned short)(b[0] | (b[1] << 8));
      for (int i = 0; i < 4; i++) w[i] = b[2 + 4 * i] | (b[3 + 4 * i] << 8) | (b[4 + 4 * i] << 16) | ((uint32_t)b[5 + 4 * i] << 24);
    }
    reinterpret_cast<uint4*>(tp)[h * 32 + l] = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    uint32_t w[8];
    for (int i = 0; i < 8; i++) w[i] = 0u;
    if (src) {
      const uint8_t* b = src + ((int64_t)row * nblk + blk) * bbytes;
      scale = (unsigned short)(b[0] | (b[1] << 8));
      for (int i = 0; i < 8; i++)
        w[i] = b[2 + 4 * i] | (b[3 + 4 * i] << 8) | (b[4 + 4 * i] << 16) | ((uint32_t)b[5 + 4 * i] << 24);
    }
    reinterpret_cast<uint4*>(tp)[(2 * h) * 32 + l] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(tp)[(2 * h + 1) * 32 + l] = make_uint4(w[4], w[5], w[6], w[7]);
  }
  unsigned short* sp = reinterpret_cast<unsigned short*>(tp + (tbytes - 128));
  sp[(2 * g + (t >> 1)) * 4 + h * 2 + (t & 1)] = scale;
}

// Q6_K re-tiling (tile layout: tile_mac_q6k, qgemv_core.cuh).  One thread per (tile, half, lane) = one (row, 32-element block).
// Element e of a super-block: low nibble ql[(e >> 7) * 64 + (e & 63)] >> 4 * ((e >> 6) & 1), high bits qh[(e >> 7) * 32 + (e & 31)] >>
// 2 * ((e >> 5) & 3), scale scales[e >> 4] (tinygrad/llm/gguf.py:68-72).
__device__ __forceinline__ int q6k_quant(const uint8_t* b, int e) {
  const int hh = e >> 7, m = e & 127;
  const int xl = (b[hh * 64 + (m & 63)] >> ((m >> 6) * 4)) & 0xF, xh = (b[128 + hh * 32 + (m & 31)] >> ((m >> 5) * 2)) & 3;
  return xl | (xh << 4);
}
__global__ void repack_q6k_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ packed, int n_out, int nsb, int n_row_tiles, int kgroups) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)n_row_tiles * kgroups * 64;
  if (idx >= total) return;
  const int l = (int)(idx & 31), h = (int)((idx >> 5) & 1);
  const int64_t tile = idx >> 6;
  const int j = (int)(tile % kgroups), rt = (int)(tile / kgroups);
  const int g = l >> 2, t = l & 3, row = rt * 16 + h * 8 + g, sb = j >> 1, e0 = (j & 1) * 128 + t * 32;
  uint8_t* tp = packed + tile * 1696;
  uint32_t lw[4] = {0u, 0u, 0u, 0u}, hw[2] = {0u, 0u};
  int sc0 = 0, sc1 = 0;
  unsigned short d = 0;          // a padded row contributes nothing
  if (row < n_out && sb < nsb) {
    const uint8_t* b = raw + ((int64_t)row * nsb + sb) * 210;
    for (int i = 0; i < 16; i++) {
      const int qa = q6k_quant(b, e0 + i), qb = q6k_quant(b, e0 + 16 + i);
      lw[i >> 2] |= (uint32_t)((qa & 15) | ((qb & 15) << 4)) << ((i & 3) * 8);
      hw[0] |= (uint32_t)(qa >> 4) << ((i & 3) * 8 + (i >> 2) * 2);
      hw[1] |= (uint32_t)(qb >> 4) << ((i & 3) * 8 + (i >> 2) * 2);
    }
    sc0 = b[192 + (e0 >> 4)]; sc1 = b[192 + (e0 >> 4) + 1];
    d = (unsigned short)(b[208] | (b[209] << 8));
  }
  reinterpret_cast<uint4*>(tp)[h * 32 + l] = make_uint4(lw[0], lw[1], lw[2], lw[3]);
  reinterpret_cast<uint2*>(tp + 1024)[h * 32 + l] = make_uint2(hw[0], hw[1]);
  tp[1536 + (h * 8 + g) * 8 + t * 2] = (uint8_t)sc0;
  tp[1536 + (h * 8 + g) * 8 + t * 2 + 1] = (uint8_t)sc1;
  if (t == 0) reinterpret_cast<unsigned short*>(tp + 1664)[h * 8 + g] = d;
}

template <typename OutT>
__global__ void dequant_packed_q6k_kernel(const uint8_t* __restrict__ packed, OutT* __restrict__ out, int rows, int n_in, int n_row_tiles, int kgroups) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)n_row_tiles * kgroups * 64;
  if (idx >= total) return;
  const int l = (int)(idx & 31), h = (int)((idx >> 5) & 1);
  const int64_t tile = idx >> 6;
  const int j = (int)(tile % kgroups), rt = (int)(tile / kgroups);
  const int g = l >> 2, t = l & 3, row = rt * 16 + h * 8 + g, blk = j * 4 + t;
  if (row >= rows || blk * 32 >= n_in) return;
  const uint8_t* tp = packed + tile * 1696;
  const uint4 lq = reinterpret_cast<const uint4*>(tp)[h * 32 + l];
  const uint2 hq = reinterpret_cast<const uint2*>(tp + 1024)[h * 32 + l];
  const uint32_t lw[4] = {lq.x, lq.y, lq.z, lq.w}, hw[2] = {hq.x, hq.y};
  const float d = __half2float(__ushort_as_half(reinterpret_cast<const unsigned short*>(tp + 1664)[h * 8 + g]));
  OutT* o = out + (int64_t)row * n_in + blk * 32;
  for (int e = 0; e < 32; e++) {
    const int i = e & 15, hf = e >> 4;
    const int lo = (lw[i >> 2] >> ((i & 3) * 8 + hf * 4)) & 0xF, hi = (hw[hf] >> ((i & 3) * 8 + (i >> 2) * 2)) & 3;
    const float sc = (float)(int8_t)tp[1536 + (h * 8 + g) * 8 + t * 2 + hf];
    store_val<OutT>(o, e, __fmul_rn(__fmul_rn(d, (float)((lo | (hi << 4)) - 32)), sc));      // (d * q) * scales, in that order
  }
}

// packed -> row-major values, rows in packed order.  One thread per (row, block).
template <typename OutT>
__global__ void dequant_packed_kernel(int qtype, const uint8_t* __restrict__ packed, OutT* __restrict__ out, int rows, int n_in,
                                      int n_row_tiles, int kgroups) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)n_row_tiles * kgroups * 64;
  if (idx >= total) return;
  int l = (int)(idx & 31), h = (int)((idx >> 5) & 1);
  int64_t tile = idx >> 6;
  int j = (int)(tile % kgroups), rt = (int)(tile / kgroups);
  int g = l >> 2, t = l & 3;
  int row = rt * 16 + h * 8 + g, blk = j * 4 + t;
  if (row >= rows || blk * 32 >= n_in) return;
  const int tbytes = tile_bytes(qtype);
  const uint8_t* tp = packed + tile * tbytes;
  const unsigned short* sp = reinterpret_cast<const unsigned short*>(tp + (tbytes - 128));
  float d = __half2float(__ushort_as_half(sp[(2 * g + (t >> 1)) * 4 + h * 2 + (t & 1)]));
  OutT* o = out + (int64_t)row * n_in + blk * 32;
  if (qtype == B200Q_Q4_0) {
    uint4 q = reinterpret_cast<const uint4*>(tp)[h * 32 + l];
    uint32_t w[4] = {q.x, q.y, q.z, q.w};
    for (int e = 0; e < 32; e++) {
      int byte = e & 15, nib = (w[byte >> 2] >> ((byte & 3) * 8 + (e >> 4) * 4)) & 0xF;
      store_val<OutT>(o, e, __fmul_rn((float)(nib - 8), d));
    }
  } else {
    for (int half = 0; half < 2; half++) {
      uint4 q = reinterpret_cast<const uint4*>(tp)[(2 * h + half) * 32 + l];
      uint32_t w[4] = {q.x, q.y, q.z, q.w};
      for (int e = 0; e < 16; e++) {
        int v = (int)(int8_t)((w[e >> 2] >> ((e & 3) * 8)) & 0xFF);
        store_val<OutT>(o, half * 16 + e, __fmul_rn(d, (float)v));
      }
    }
  }
}

// ---------------------------------------------------------------------------
static bool known_qtype(int q) {
  return q == B200Q_Q4_0 || q == B200Q_Q4_1 || q == B200Q_Q5_0 || q == B200Q_Q5_1 || q == B200Q_Q8_0 || q == B200Q_Q4_K || q == B200Q_Q5_K || q == B200Q_Q6_K;
}
static int block_elems(int q) { return (q == B200Q_Q4_K || q == B200Q_Q5_K || q == B200Q_Q6_K) ? 256 : 32; }

extern "C" int b200q_dequant_raw(int qtype, const void* raw, void* out, int64_t n_elems, int out_dtype, void* stream) {
  if (!known_qtype(qtype) || (out_dtype != B200Q_F32 && out_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (n_elems < 0 || (n_elems && (!raw || !out))) return B200Q_ERR_BAD_ARG;
  if (n_elems % block_elems(qtype)) return B200Q_ERR_BAD_SHAPE;
  if (n_elems == 0) return B200Q_OK;
  unsigned blocks = (unsigned)((n_elems + 255) / 256);
  if (out_dtype == B200Q_F32) dequant_raw_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>(qtype, (const uint8_t*)raw, (float*)out, n_elems);
  else dequant_raw_kernel<__half><<<blocks, 256, 0, (cudaStream_t)stream>>>(qtype, (const uint8_t*)raw, (__half*)out, n_elems);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" size_t b200q_packed_bytes(int qtype, int n_out, int n_in) {
  if ((qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0 && qtype != B200Q_Q6_K) || n_out <= 0 || n_in <= 0) return 0;
  if (qtype == B200Q_Q6_K && n_in % 256) return 0;
  return (size_t)ceil_div(n_out, TILE_ROWS) * ceil_div(n_in, GROUP_ELEMS) * tile_bytes(qtype);
}

extern "C" int b200q_repack(int qtype, const void* raw0, const void* raw1, void* packed, int n_out, int n_in, void* stream) {
  if (qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0 && qtype != B200Q_Q6_K) return B200Q_ERR_BAD_ARG;
  if (!raw0 || !packed || n_out <= 0 || n_in <= 0) return B200Q_ERR_BAD_ARG;
  if (n_in % (qtype == B200Q_Q6_K ? 256 : 32)) return B200Q_ERR_BAD_SHAPE;
  if ((uintptr_t)packed & 15) return B200Q_ERR_MISALIGNED;
  if (qtype == B200Q_Q6_K) {
    if (raw1) return B200Q_ERR_UNSUPPORTED;       // no interleaved gate / up tiles for this format
    const int nrt = ceil_div(n_out, TILE_ROWS), kg = n_in / GROUP_ELEMS;
    const int64_t tot = (int64_t)nrt * kg * 64;
    repack_q6k_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)raw0, (uint8_t*)packed, n_out, n_in / 256, nrt, kg);
    B200Q_CHECK_CUDA(cudaGetLastError());
    return B200Q_OK;
  }
  int rows = raw1 ? 2 * ceil_div(n_out, 8) * 8 : n_out;       // interleaved: tiles of 8+8 rows
  int n_row_tiles = raw1 ? ceil_div(n_out, 8) : ceil_div(n_out, TILE_ROWS), kgroups = ceil_div(n_in, GROUP_ELEMS);
  (void)rows;
  int64_t total = (int64_t)n_row_tiles * kgroups * 64;
  repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(qtype, (const uint8_t*)raw0, (const uint8_t*)raw1,
                                                                                  (uint8_t*)packed, n_out, n_in / 32, n_row_tiles, kgroups);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_dequant_packed(int qtype, const void* packed, void* out, int n_out, int n_in, int out_dtype, void* stream) {
  if (qtype != B200Q_Q4_0 && qtype != B200Q_Q8_0 && qtype != B200Q_Q6_K) return B200Q_ERR_BAD_ARG;
  if (!packed || !out || n_out <= 0 || n_in <= 0 || (out_dtype != B200Q_F32 && out_dtype != B200Q_F16)) return B200Q_ERR_BAD_ARG;
  if (n_in % (qtype == B200Q_Q6_K ? 256 : 32)) return B200Q_ERR_BAD_SHAPE;
  if ((uintptr_t)packed & 15) return B200Q_ERR_MISALIGNED;
  int n_row_tiles = ceil_div(n_out, TILE_ROWS), kgroups = ceil_div(n_in, GROUP_ELEMS);
  int64_t total = (int64_t)n_row_tiles * kgroups * 64;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (qtype == B200Q_Q6_K) {
    if (out_dtype == B200Q_F32) dequant_packed_q6k_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, (float*)out, n_out, n_in, n_row_tiles, kgroups);
    else dequant_packed_q6k_kernel<__half><<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)packed, (__half*)out, n_out, n_in, n_row_tiles, kgroups);
    B200Q_CHECK_CUDA(cudaGetLastError());
    return B200Q_OK;
  }
  if (out_dtype == B200Q_F32)
    dequant_packed_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>(qtype, (const uint8_t*)packed, (float*)out, n_out, n_in, n_row_tiles, kgroups);
  else
    dequant_packed_kernel<__half><<<blocks, 256, 0, (cudaStream_t)stream>>>(qtype, (const uint8_t*)packed, (__half*)out, n_out, n_in, n_row_tiles, kgroups);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
