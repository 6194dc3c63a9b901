"""numpy restatement of the MXFP8 quantiser, its dequantiser, the MoE routing
tables and the grouped expert GEMM (test infrastructure).

Follows extra/gemm/cdna_asm_gemm.py:149-173 (``quantize_mxfp8``,
``_mx_block_scale``), tinygrad/dtype.py:237-274 (E4M3 round-to-nearest-even,
saturating), extra/gemm/moe_routing.py:89-131 (``route`` / ``dispatch`` /
``combine``) and the device-independent reference computation of
test/backend/test_asm_gemm.py:289-292,306 (dequantised operands matmul).
The reference holds no test for the grouped GEMM + routing composition:
that composition is parity-unpinned beyond these pieces.
"""
import numpy as np

BLOCK_ROW = 256      # extra/gemm/moe_routing.py:4


def e4m3_table() -> np.ndarray:
  """All 256 E4M3 codes as fp32 (tinygrad/dtype.py:262-274); 0x7F/0xFF are NaN."""
  t = np.zeros(256, dtype=np.float32)
  for c in range(256):
    s, e, m = c >> 7, (c >> 3) & 0xF, c & 7
    if e == 0xF and m == 7: v = np.nan
    elif e == 0: v = (m / 8.0) * 2.0 ** -6
    else: v = (1 + m / 8.0) * 2.0 ** (e - 7)
    t[c] = -v if s else v
  return t


def float_to_e4m3(x: np.ndarray) -> np.ndarray:
  """fp32 -> E4M3 code, round-to-nearest-even, saturating to +-448 (0x7E);
  non-finite -> 0x7F / 0xFF (tinygrad/dtype.py:237-260)."""
  x = np.asarray(x, dtype=np.float32)
  a = np.abs(x.astype(np.float64))
  sign = (np.signbit(x).astype(np.uint8) << 7)
  code = np.zeros(x.shape, dtype=np.int64)
  norm = a >= 2.0 ** -6
  with np.errstate(divide="ignore", invalid="ignore"):
    e = np.floor(np.log2(np.where(norm, a, 1.0))).astype(np.int64)
  e = np.clip(e, -6, 8)
  # correct log2 rounding at powers of two
  e = np.where(a < 2.0 ** e.astype(np.float64), e - 1, e)
  e = np.where(a >= 2.0 ** (e + 1).astype(np.float64), e + 1, e)
  mant = a / 2.0 ** e.astype(np.float64) * 8.0            # in [8, 16)
  m = np.rint(mant).astype(np.int64)                      # numpy rint is half-to-even
  cn = ((e + 7) << 3) + (m - 8)                           # a mantissa carry rolls into the exponent
  sub = np.rint(a * 2.0 ** 9).astype(np.int64)            # subnormal step 2^-9
  code = np.where(norm, cn, sub)
  code = np.where(a > 464.0, 0x7E, np.minimum(code, 0x7E))   # 464 = midpoint above 448: saturate
  code = np.where(np.isfinite(x), code, 0x7F)
  return (code.astype(np.uint8) | sign).astype(np.uint8)


def quantize_mxfp8(x: np.ndarray):
  """extra/gemm/cdna_asm_gemm.py:149-159: per 32 along the last axis,
  e8 = clamp(floor(log2(max(amax,1e-38))) + 127, 0, 254);
  q = e4m3(clamp(x * 2^(127-e8), +-448)).  Returns (q codes uint8, e8 uint8)."""
  *batch, K = x.shape
  xf = x.astype(np.float32).reshape(*batch, K // 32, 32)
  amax = np.abs(xf).max(-1)
  e8 = np.clip(np.floor(np.log2(np.maximum(amax, np.float32(1e-38)))) + 127, 0, 254).astype(np.uint8)
  qscale = np.exp2(127.0 - e8.astype(np.float32)).astype(np.float32)
  xs = np.clip(xf * qscale[..., None], -448.0, 448.0).astype(np.float32)
  return float_to_e4m3(xs).reshape(*batch, K), e8


def dequantize_mxfp8(q: np.ndarray, e8: np.ndarray) -> np.ndarray:
  """cdna_asm_gemm.py:165-173: value * 2^(e8-127), scale shared by 32."""
  *batch, K = q.shape
  v = e4m3_table()[q].reshape(*batch, K // 32, 32)
  return (v * np.exp2(e8.astype(np.float32) - 127.0)[..., None]).reshape(*batch, K).astype(np.float32)


def mxfp8_matmul(a_q, a_e8, b_q, b_e8) -> np.ndarray:
  """test/backend/test_asm_gemm.py:289-292,306: dequant(a) @ dequant(b)^T, fp32."""
  return dequantize_mxfp8(a_q, a_e8) @ dequantize_mxfp8(b_q, b_e8).T


def route(logits: np.ndarray, k: int, n_experts: int):
  """extra/gemm/moe_routing.py:109-122 for one device group.
  Returns (weights (T,k), topi (T,k), dest_row (T*k,), off (E+1,), m_l)."""
  T, E = logits.shape
  order = np.argsort(-logits, axis=-1, kind="stable")[:, :k]       # topk: descending, lowest index first on ties
  topv = np.take_along_axis(logits, order, -1)
  w = np.exp(topv - topv.max(-1, keepdims=True)); w = (w / w.sum(-1, keepdims=True)).astype(np.float32)
  flat = order.reshape(-1)
  onehot = np.zeros((T * k, E), dtype=np.int64); onehot[np.arange(T * k), flat] = 1
  pad = ((onehot.sum(0) + BLOCK_ROW - 1) // BLOCK_ROW) * BLOCK_ROW
  off = np.concatenate([[0], np.cumsum(pad)])
  dest = ((np.cumsum(onehot, 0) + off[:E][None, :]) * onehot).sum(-1) - 1
  m_l = (-(-T * k // BLOCK_ROW) + n_experts) * BLOCK_ROW           # moe_routing.py:89-90
  return w, order.astype(np.int32), dest.astype(np.int32), off.astype(np.int32), m_l


def dispatch(x: np.ndarray, dest_row: np.ndarray, m_l: int, k: int) -> np.ndarray:
  """moe_routing.py:84-87,124-126: zero-filled scatter of token rows."""
  out = np.zeros((m_l, x.shape[-1]), dtype=x.dtype)
  out[dest_row] = np.repeat(x, k, axis=0)
  return out


def combine(y: np.ndarray, dest_row: np.ndarray, weights: np.ndarray) -> np.ndarray:
  """moe_routing.py:128-131: gather k rows per token, weight, sum over k."""
  T, k = weights.shape
  sel = y[dest_row].reshape(T, k, -1).astype(np.float32)
  return (sel * weights[..., None]).sum(1)


def grouped_mx_gemm(a_q, a_e8, w_q, w_e8, off) -> np.ndarray:
  """extra/gemm/moe_gemm.py:112-134 semantics: rows of A grouped by expert
  (group e = rows off[e]:off[e+1]); C = A_deq @ W_deq[e]^T in fp32, then bf16
  as the kernel stores it (extra/thunder/amd/grouped_mxfp8_gemm.cpp:32-158)."""
  a = dequantize_mxfp8(a_q, a_e8)
  out = np.zeros((a.shape[0], w_q.shape[1]), dtype=np.float32)
  for e in range(w_q.shape[0]):
    lo, hi = int(off[e]), int(off[e + 1])
    if hi > lo: out[lo:hi] = a[lo:hi] @ dequantize_mxfp8(w_q[e], w_e8[e]).T
  return out


def to_bf16(x: np.ndarray) -> np.ndarray:
  """tinygrad/dtype.py:222-226: round-to-nearest-even to bf16, returned as fp32."""
  u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
  r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
  return np.where(np.isfinite(x), r.view(np.float32), x).astype(np.float32)
