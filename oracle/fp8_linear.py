"""CPU restatement of the per-tensor FP8 linear (TEST INFRASTRUCTURE: only tests / smoke / the bench's CPU legs may import this).

Follows extra/fp8/fp8_linear.py: `quantize_to_fp8` (:4-16) and `FP8Linear.__call__` (:48-63); the contraction is the one `custom_matmul`
states (:18-30): products of the two FP8 tensors in float, summed over the input features.  E4M3 rounding: oracle/mxfp8.py (pinned on the
reference's own conversion).  Pinned on tests/golden/fp8linear.npz, which the reference produced."""
import numpy as np
from oracle import mxfp8 as mx


def quantize_to_fp8(x: np.ndarray):
  """-> (E4M3 codes uint8, factor fp32 = 1 / scale) with scale = 448 / (max|x| + 1e-8), fp32 arithmetic as the reference's tensor ops.
  The factor is (max|x| + 1e-8) * fp32(1 / 448): what the reference's simplifier makes of (448 / d).reciprocal() (bit-exact on the golden)."""
  x = np.asarray(x, dtype=np.float32)
  d = (np.abs(x).max().astype(np.float32) + np.float32(1e-8)).astype(np.float32)
  scale = np.float32(448.0) / d
  xs = np.clip((x * scale).astype(np.float32), np.float32(-448.0), np.float32(448.0))
  return mx.float_to_e4m3(xs), (d * np.float32(1.0 / 448.0)).astype(np.float32)


def fp8_linear(x: np.ndarray, w: np.ndarray, bias=None) -> np.ndarray:
  """x [..., in], w [out, in] fp32 -> y [..., out]: both operands quantised per tensor, product in fp32, rescaled, + bias."""
  xq, xf = quantize_to_fp8(x)
  wq, wf = quantize_to_fp8(w)
  t = mx.e4m3_table()
  acc = t[xq].astype(np.float32) @ t[wq].astype(np.float32).T
  y = (acc * wf).astype(np.float32) * xf
  return (y + np.asarray(bias, dtype=np.float32) if bias is not None else y).astype(np.float32)
