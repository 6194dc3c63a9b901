"""numpy restatement of the GGUF block dequantisers (test infrastructure).

Follows tinygrad/llm/gguf.py:23-72 (``ggml_data_to_tensor``) operation by
operation, including the evaluation order of the fp32 multiplies, so the fp32
result is bit-identical to the reference's.
"""
import numpy as np

# tinygrad/llm/gguf.py:20-21 -- {ggml_type: (elements per block, bytes per block)}
GGML_QUANT = {2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}
Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K = 2, 3, 6, 7, 8, 12, 13, 14


def q_to_uint8(t: np.ndarray, b: int) -> np.ndarray:
  """tinygrad/llm/gguf.py:38-41 -- split every byte into 8//b fields of b bits;
  the output lists field 0 of all bytes, then field 1 of all bytes, ..."""
  shifts = np.array([2 ** (i * b) for i in range(8 // b)], dtype=np.uint8)
  mask = 0xFF >> (8 - b)
  f = (t[..., None] // shifts) & mask               # (..., nbytes, fields)
  f = np.swapaxes(f, -1, -2)                        # (..., fields, nbytes)
  return f.reshape(*f.shape[:-2], -1).astype(np.uint8)


def _blocks(raw: np.ndarray, n: int, ggml_type: int) -> np.ndarray:
  nel, nby = GGML_QUANT[ggml_type]
  raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
  return raw[:(n // nel) * nby].reshape(-1, nby)    # gguf.py:45


def dequantize(raw: np.ndarray, n: int, ggml_type: int) -> np.ndarray:
  """Raw GGUF bytes -> fp32 values, shape (n,).  tinygrad/llm/gguf.py:43-72."""
  blocks = _blocks(raw, n, ggml_type)
  if ggml_type == Q4_0:   # gguf.py:46: (int8(nibble) - 8) * float32(fp16 d)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    q = q_to_uint8(blocks[:, 2:], 4).view(np.int8) - np.int8(8)
    return (q.astype(np.float32) * d).reshape(-1)
  if ggml_type == Q8_0:   # gguf.py:56: float32(fp16 d) * int8 q
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    return (d * blocks[:, 2:].copy().view(np.int8).astype(np.float32)).reshape(-1)
  if ggml_type == Q4_1:   # gguf.py:47-49: nibble * d + m
    d, m = (blocks[:, s:s + 2].copy().view(np.float16).astype(np.float32) for s in (0, 2))
    return (q_to_uint8(blocks[:, 4:], 4).view(np.int8).astype(np.float32) * d + m).reshape(-1)
  if ggml_type in (Q5_0, Q5_1):   # gguf.py:50-55: (nibble + 16 * high bit) * d + (m | -16 d)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    qh_off = 2 if ggml_type == Q5_0 else 4
    qh = q_to_uint8(blocks[:, qh_off:qh_off + 4], 1).reshape(-1, 8, 4).swapaxes(-1, -2).reshape(-1, 32).view(np.int8)
    q = q_to_uint8(blocks[:, qh_off + 4:], 4).view(np.int8) + qh * np.int8(16)
    add = blocks[:, 2:4].copy().view(np.float16).astype(np.float32) if ggml_type == Q5_1 else np.float32(-16) * d
    return (q.astype(np.float32) * d + add).reshape(-1)
  if ggml_type in (Q4_K, Q5_K):   # gguf.py:57-67: (d * sc) * q - dmin * mn over 8 groups of 32
    d, dmin = (blocks[:, i:i + 2].copy().view(np.float16).astype(np.float32)[:, :, None] for i in (0, 2))
    s = blocks[:, 4:16]
    sc = np.concatenate([s[:, 0:4] & 63, (s[:, 8:12] & 0xF) | ((s[:, 0:4] >> 6) << 4)], axis=-1)
    mn = np.concatenate([s[:, 4:8] & 63, (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)], axis=-1)
    qs_off = 48 if ggml_type == Q5_K else 16
    qs = blocks[:, qs_off:qs_off + 128].reshape(-1, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(-1, 8, 32)
    if ggml_type == Q5_K: q = q + q_to_uint8(blocks[:, 16:48], 1).reshape(-1, 8, 32) * np.uint8(16)
    return ((d * sc[:, :, None].astype(np.float32)) * q.astype(np.float32) - dmin * mn[:, :, None].astype(np.float32)).reshape(-1)
  if ggml_type == Q6_K:   # gguf.py:68-72: (d * q) * scales, in that order
    xl = q_to_uint8(blocks[:, :128].reshape(-1, 2, 64), 4)
    xh = q_to_uint8(blocks[:, 128:192].reshape(-1, 2, 32), 2) << 4
    scales = np.repeat(blocks[:, 192:208].copy().view(np.int8)[:, :, None], 16, axis=2).reshape(-1, 256)
    d = blocks[:, -2:].copy().view(np.float16).astype(np.float32)
    q = ((xl | xh).view(np.int8) - np.int8(32)).reshape(-1, 256)
    return ((d * q.astype(np.float32)) * scales.astype(np.float32)).reshape(-1)
  raise ValueError(f"GGML type {ggml_type} is not restated here")


def dequantize_f16(raw: np.ndarray, n: int, ggml_type: int) -> np.ndarray:
  """The materialised weight: fp32 dequant rounded to fp16 (RNE).
  tinygrad/llm/model.py:376 (``v.cast('float16')``)."""
  return dequantize(raw, n, ggml_type).astype(np.float16)


def weight_matrix(raw: np.ndarray, n_out: int, n_in: int, ggml_type: int) -> np.ndarray:
  """GGUF stores dims innermost-first; a Linear weight is (out, in) row-major
  with blocks running along ``in`` (tinygrad/llm/gguf.py:148)."""
  return dequantize(raw, n_out * n_in, ggml_type).reshape(n_out, n_in)
