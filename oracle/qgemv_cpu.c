/* CPU restatement of the fused dequant-GEMV (TEST INFRASTRUCTURE / timed CPU baseline only).
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

/* y[n_out] = W x, W given as raw GGUF blocks of type qtype (2 = Q4_0, 8 = Q8_0). */
void qgemv_cpu(int qtype, const uint8_t* raw, const float* x, float* y, int n_out, int n_in) {
  const int nblk = n_in / 32, bbytes = qtype == 2 ? 18 : 34;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < n_out; r++) {
    const uint8_t* row = raw + (size_t)r * nblk * bbytes;
    float acc = 0.f;
    for (int b = 0; b < nblk; b++) {
      const uint8_t* blk = row + (size_t)b * bbytes;
      uint16_t dh; memcpy(&dh, blk, 2);
      const float d = f16_to_f32(dh);
      const float* xb = x + b * 32;
      float s = 0.f;
      if (qtype == 2) {
        for (int j = 0; j < 16; j++) {
          s += xb[j] * (float)((int)(blk[2 + j] & 0xF) - 8);
          s += xb[j + 16] * (float)((int)(blk[2 + j] >> 4) - 8);
        }
      } else {
        for (int j = 0; j < 32; j++) s += xb[j] * (float)(int8_t)blk[2 + j];
      }
      acc += s * d;
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
