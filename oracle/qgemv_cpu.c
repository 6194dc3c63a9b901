/* CPU restatement of the GGUF block dequantisers and of the fused dequant-GEMV (TEST INFRASTRUCTURE / timed CPU baseline only).
 *
 * Follows the arithmetic of the kernels tinygrad generates for `Linear.__call__` on a lazily
 * dequantised GGUF weight with fp32 activations (tinygrad/nn/__init__.py:177 over
 * tinygrad/llm/gguf.py:46 for Q4_0 and :56 for Q8_0): per element an fp32 product of the
 * activation with the exact dequantised value, accumulated in fp32 along the row
 * (tinygrad/mixin/op.py:367-392).  Rows are independent, so they are spread over OpenMP threads.
 * Raw GGUF block layout, no repacking: Q4_0 = fp16 d + 16 bytes (byte j: element j low nibble,
 * element j+16 high nibble); Q8_0 = fp16 d + 32 int8.
 */
#include <stdint.h>
#include <string.h>
#include <math.h>

static inline float f16_to_f32(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF, u;
  if (e == 0) {
    if (m == 0) u = s;
    else { int sh = 0; while (!(m & 0x400)) { m <<= 1; sh++; } m &= 0x3FF; u = s | ((uint32_t)(113 - sh) << 23) | (m << 13); }
  } else if (e == 31) u = s | 0x7F800000u | (m << 13);
  else u = s | ((e + 112) << 23) | (m << 13);
  float f; memcpy(&f, &u, 4); return f;
}

/* Bytes / elements per block (tinygrad/llm/gguf.py:20-21). */
static int blk_bytes(int qtype) {
  switch (qtype) { case 2: return 18; case 3: return 20; case 6: return 22; case 7: return 24; case 8: return 34;
                   case 12: return 144; case 13: return 176; case 14: return 210; default: return 0; }
}
static int blk_elems(int qtype) { return (qtype == 12 || qtype == 13 || qtype == 14) ? 256 : 32; }

/* One block -> its fp32 values, operation by operation as tinygrad/llm/gguf.py:46-72 writes them (same products, same
 * order, so the fp32 result is the reference's bit for bit). */
static void dequant_block(int qtype, const uint8_t* b, float* o) {
  uint16_t h; 
  if (qtype == 2) {                                  /* gguf.py:46  (int8(nibble) - 8) * d */
    memcpy(&h, b, 2); const float d = f16_to_f32(h);
    for (int j = 0; j < 16; j++) { o[j] = (float)((int)(b[2 + j] & 0xF) - 8) * d; o[j + 16] = (float)((int)(b[2 + j] >> 4) - 8) * d; }
  } else if (qtype == 3) {                           /* gguf.py:47-49  nibble * d + m */
    memcpy(&h, b, 2); const float d = f16_to_f32(h); memcpy(&h, b + 2, 2); const float m = f16_to_f32(h);
    for (int j = 0; j < 16; j++) { o[j] = (float)(b[4 + j] & 0xF) * d + m; o[j + 16] = (float)(b[4 + j] >> 4) * d + m; }
  } else if (qtype == 6 || qtype == 7) {             /* gguf.py:50-55  (nibble + 16 * high bit) * d + (m | -16 d) */
    memcpy(&h, b, 2); const float d = f16_to_f32(h);
    const int qh_off = qtype == 6 ? 2 : 4;
    float add;
    if (qtype == 7) { memcpy(&h, b + 2, 2); add = f16_to_f32(h); } else add = -16.f * d;
    uint32_t qh; memcpy(&qh, b + qh_off, 4);
    const uint8_t* qs = b + qh_off + 4;
    for (int j = 0; j < 16; j++) {
      o[j] = (float)((qs[j] & 0xF) + 16 * ((qh >> j) & 1)) * d + add;
      o[j + 16] = (float)((qs[j] >> 4) + 16 * ((qh >> (j + 16)) & 1)) * d + add;
    }
  } else if (qtype == 8) {                           /* gguf.py:56  d * int8 */
    memcpy(&h, b, 2); const float d = f16_to_f32(h);
    for (int j = 0; j < 32; j++) o[j] = d * (float)(int8_t)b[2 + j];
  } else if (qtype == 12 || qtype == 13) {           /* gguf.py:57-67  (d * sc) * q - dmin * mn */
    memcpy(&h, b, 2); const float d = f16_to_f32(h); memcpy(&h, b + 2, 2); const float dmin = f16_to_f32(h);
    const uint8_t* s = b + 4;
    int sc[8], mn[8];
    for (int i = 0; i < 4; i++) {
      sc[i] = s[i] & 63; sc[4 + i] = (s[8 + i] & 0xF) | ((s[i] >> 6) << 4);
      mn[i] = s[4 + i] & 63; mn[4 + i] = (s[8 + i] >> 4) | ((s[4 + i] >> 6) << 4);
    }
    const uint8_t* qs = b + (qtype == 13 ? 48 : 16);
    const uint8_t* qhp = b + 16;                     /* Q5_K: 32 bytes, bit g of byte j = fifth bit of element j of group g */
    for (int c = 0; c < 4; c++)
      for (int half = 0; half < 2; half++) {
        const int g = 2 * c + half;
        const float ds = d * (float)sc[g], dm = dmin * (float)mn[g];
        for (int j = 0; j < 32; j++) {
          int q = half ? (qs[c * 32 + j] >> 4) : (qs[c * 32 + j] & 0xF);
          if (qtype == 13) q += 16 * ((qhp[j] >> g) & 1);
          o[g * 32 + j] = ds * (float)q - dm;
        }
      }
  } else if (qtype == 14) {                          /* gguf.py:68-72  (d * q) * scale */
    memcpy(&h, b + 208, 2); const float d = f16_to_f32(h);
    const int8_t* sc = (const int8_t*)(b + 192);
    for (int half = 0; half < 2; half++)
      for (int j = 0; j < 128; j++) {
        const int e = half * 128 + j;                /* element index inside the block */
        const uint8_t lb = b[half * 64 + (j & 63)];
        const int lo = (j < 64) ? (lb & 0xF) : (lb >> 4);
        const int hi = (b[128 + half * 32 + (j & 31)] >> (2 * (j >> 5))) & 3;
        const int q = (int)(int8_t)(uint8_t)(lo | (hi << 4)) - 32;
        o[e] = (d * (float)q) * (float)sc[e >> 4];
      }
  }
}

/* n_elems values of raw GGUF blocks -> fp32 (`ggml_data_to_tensor`, tinygrad/llm/gguf.py:23-72).  Returns 0, or -1 for a type
 * that is not restated here. */
int dequant_cpu(int qtype, const uint8_t* raw, float* out, int64_t n_elems) {
  const int bb = blk_bytes(qtype), be = blk_elems(qtype);
  if (!bb) return -1;
  const int64_t nblk = n_elems / be;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < nblk; i++) dequant_block(qtype, raw + i * bb, out + i * be);
  return 0;
}

/* y[n_out] = W x, W given as raw GGUF blocks of type qtype.  Per element the product the reference's fused kernel forms for
 * fp32 activations -- Q4_0: (x * q) * d, Q8_0: (x * d) * q, Q6_K: ((x * d) * q) * scale, other types: x * dequantised value --
 * added into one fp32 accumulator in element order (tinygrad/mixin/op.py:367-392; the generated kernel's accumulation order
 * differs by its unrolling, which fp32 tolerances absorb). */
void qgemv_cpu(int qtype, const uint8_t* raw, const float* x, float* y, int n_out, int n_in) {
  const int bb = blk_bytes(qtype), be = blk_elems(qtype), nblk = n_in / (be ? be : 32);
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n_out; r++) {
    const uint8_t* row = raw + (size_t)r * nblk * bb;
    float acc = 0.f;
    for (int b = 0; b < nblk; b++) {
      const uint8_t* blk = row + (size_t)b * bb;
      const float* xb = x + b * be;
      uint16_t dh;
      if (qtype == 2) {
        memcpy(&dh, blk, 2); const float d = f16_to_f32(dh);
        for (int j = 0; j < 16; j++) acc += (xb[j] * (float)((int)(blk[2 + j] & 0xF) - 8)) * d;
        for (int j = 0; j < 16; j++) acc += (xb[j + 16] * (float)((int)(blk[2 + j] >> 4) - 8)) * d;
      } else if (qtype == 8) {
        memcpy(&dh, blk, 2); const float d = f16_to_f32(dh);
        for (int j = 0; j < 32; j++) acc += (xb[j] * d) * (float)(int8_t)blk[2 + j];
      } else {
        float w[256];
        dequant_block(qtype, blk, w);
        for (int j = 0; j < be; j++) acc += xb[j] * w[j];
      }
    }
    y[r] = acc;
  }
}

/* x * rsqrt(mean(x^2) + eps) * w  (tinygrad/nn/__init__.py:300-304), w fp16 */
void rmsnorm_cpu(const float* x, const uint16_t* w, float* out, int n, float eps) {
  float ss = 0.f;
  for (int i = 0; i < n; i++) ss += x[i] * x[i];
  const float rs = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = 0; i < n; i++) out[i] = x[i] * rs * f16_to_f32(w[i]);
}
