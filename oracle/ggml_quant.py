"""numpy restatement of the GGUF block dequantisers (test infrastructure).

Follows tinygrad/llm/gguf.py:23-72 (``ggml_data_to_tensor``) operation by
operation, including the evaluation order of the fp32 multiplies, so the fp32
result is bit-identical to the reference's.
"""
import numpy as np

# tinygrad/llm/gguf.py:20-21 -- {ggml_type: (elements per block, bytes per block)}
GGML_QUANT = {2: (32, 18), 8: (32, 34), 14: (256, 210)}
Q4_0, Q8_0, Q6_K = 2, 8, 14


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
