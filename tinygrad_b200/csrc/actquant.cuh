// Quantised activation record: what a GEMV CTA keeps in shared memory for one activation row,
// and what an upstream kernel may hand over ready-made so the GEMV only has to copy it.
//
// For a row of K values (K padded up to whole groups of 128 = 4 blocks of 32), kgroups = ceil(K / 128):
//   uint4  xq [kgroups][2][8]    B operands of the int8 MMAs: per group, per 16-byte half c, the slot of "lane" g:
//                                g < 4: hi digits of block g, g >= 4: lo digits of block g-4.  A block's 8 words sit in
//                                MMA order: word r = 2*j + h holds elements 4j..4j+3 (h = 0) or 16+4j..16+4j+3 (h = 1).
//   float4 xsc[kgroups][2][2]    per (digit, block pair): {scale_A, offset_A, scale_B, offset_B};
//                                hi digit: scale = 128 * s, offset = 8 * s * sum(q)  (removes Q4_0's -8);  lo digit: scale = s, offset = 0
// where block value x_i ~ s * q_i, q_i = 128 * hi_i + lo_i a 15-bit integer (|q_i| <= 16256), lo in [-64, 63].
// The record is kgroups * 320 bytes, xq first.
#pragma once
#include "common.cuh"

constexpr int XQ_GROUP_BYTES = 320;
constexpr float XQ_RANGE = 16256.f;    // 127 * 128

__host__ __device__ inline size_t xq_record_bytes(int k) { return (size_t)((k + GROUP_ELEMS - 1) / GROUP_ELEMS) * XQ_GROUP_BYTES; }

struct XqDst {
  uint32_t* xw;   // the xq words
  float* sw;      // the xsc floats
  __device__ __forceinline__ XqDst(void* record, int kgroups) : xw(reinterpret_cast<uint32_t*>(record)),
    sw(reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(record) + (size_t)kgroups * 256)) {}
};

__device__ __forceinline__ void xq_store_scales(const XqDst& d, int b, float s, int qsum) {
  const int j = b >> 2, tb = b & 3, pr = tb >> 1, sl = (tb & 1) * 2;
  d.sw[((j * 2 + 0) * 2 + pr) * 4 + sl] = 128.f * s;
  d.sw[((j * 2 + 0) * 2 + pr) * 4 + sl + 1] = 8.f * s * (float)qsum;
  d.sw[((j * 2 + 1) * 2 + pr) * 4 + sl] = s;
  d.sw[((j * 2 + 1) * 2 + pr) * 4 + sl + 1] = 0.f;
}
__device__ __forceinline__ void xq_store_words(const XqDst& d, int b, int q, uint32_t hiw, uint32_t low) {
  // q = which 4 elements of the block (4q..4q+3); their word position in MMA order
  const int r = (q & 3) * 2 + (q >> 2), j = b >> 2, tb = b & 3;
  d.xw[((j * 2 + (r >> 2)) * 8 + tb) * 4 + (r & 3)] = hiw;
  d.xw[((j * 2 + (r >> 2)) * 8 + tb + 4) * 4 + (r & 3)] = low;
}

// Block b of 32 values held by 8 consecutive lanes, 4 values each (q = lane & 7 gives elements 4q..4q+3).
// sub16 (optional): [block][2] floats, 32 * s * (sum of q over elements 0..15 / 16..31): what removes Q6_K's offset of 32 per 16-element
// sub-block (a sub-block has its own weight scale, so the block sum is not enough).
__device__ __forceinline__ void quant_block_8x4(float4 v, int q, int b, const XqDst& d, float* sub16 = nullptr) {
  float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  const bool live = amax > 0.f && amax < INFINITY;
  const float inv = live ? XQ_RANGE / amax : 0.f, s = live ? amax / XQ_RANGE : 0.f;
  const int i0 = __float2int_rn(v.x * inv), i1 = __float2int_rn(v.y * inv), i2 = __float2int_rn(v.z * inv), i3 = __float2int_rn(v.w * inv);
  int qsum = i0 + i1 + i2 + i3;
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
  if (sub16 && (q & 3) == 0) sub16[b * 2 + (q >> 2)] = 32.f * s * (float)qsum;
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 4);
  const int h0 = (i0 + 64) >> 7, h1 = (i1 + 64) >> 7, h2 = (i2 + 64) >> 7, h3 = (i3 + 64) >> 7;
  const uint32_t hiw = (h0 & 0xFF) | ((h1 & 0xFF) << 8) | ((h2 & 0xFF) << 16) | ((uint32_t)(h3 & 0xFF) << 24);
  const uint32_t low = ((i0 - (h0 << 7)) & 0xFF) | (((i1 - (h1 << 7)) & 0xFF) << 8) | (((i2 - (h2 << 7)) & 0xFF) << 16) |
                       ((uint32_t)((i3 - (h3 << 7)) & 0xFF) << 24);
  xq_store_words(d, b, q, hiw, low);
  if (q == 0) xq_store_scales(d, b, s, qsum);
}

// Block b of 32 values held by one warp, one value per lane (lane = element).
__device__ __forceinline__ void quant_block_32x1(float v, int lane, int b, const XqDst& d) {
  const float amax = warp_max(fabsf(v));
  const bool live = amax > 0.f && amax < INFINITY;
  const float inv = live ? XQ_RANGE / amax : 0.f, s = live ? amax / XQ_RANGE : 0.f;
  const int i = __float2int_rn(v * inv);
  int qsum = i;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
  const int h = (i + 64) >> 7;
  const uint32_t hb = h & 0xFF, lb = (i - (h << 7)) & 0xFF;
  const uint32_t hiw = hb | (__shfl_down_sync(0xffffffffu, hb, 1) << 8) | (__shfl_down_sync(0xffffffffu, hb, 2) << 16) | (__shfl_down_sync(0xffffffffu, hb, 3) << 24);
  const uint32_t low = lb | (__shfl_down_sync(0xffffffffu, lb, 1) << 8) | (__shfl_down_sync(0xffffffffu, lb, 2) << 16) | (__shfl_down_sync(0xffffffffu, lb, 3) << 24);
  if ((lane & 3) == 0) xq_store_words(d, b, lane >> 2, hiw, low);
  if (lane == 0) xq_store_scales(d, b, s, qsum);
}
