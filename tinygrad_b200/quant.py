"""GGUF-quantised weights on the device: dequantisation, packing, and the fused linear.

Host-side mirror of the reference's interface for this path: `dequantize` is
`ggml_data_to_tensor` (tinygrad/llm/gguf.py:23-72), `QuantLinear.__call__(x)` is
`nn.Linear.__call__(x)` on a GGUF weight (tinygrad/nn/__init__.py:177) -- same
argument meaning, same output dtype rule (the activation's dtype), errors raised
as exceptions.  All compute happens in libb200q.so.
"""
import ctypes
import numpy as np
from . import _lib
from ._lib import check, Q4_0, Q8_0, Q6_K, F32, F16, EPI_LINEAR, EPI_SILU_MUL, FLAG_PDL
from .runtime import DeviceBuffer, ptr_of, stream_ptr

# (elements, bytes) per block of the formats the dequantiser covers (tinygrad/llm/gguf.py:20-21); Q4_0 and Q8_0 also have fused kernels
GGML_QUANT = {Q4_0: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), Q8_0: (32, 34), 12: (256, 144), 13: (256, 176), Q6_K: (256, 210)}
_DT = {np.dtype(np.float32): F32, np.dtype(np.float16): F16}


def _as_device(a):
  return a if isinstance(a, DeviceBuffer) or a is None else DeviceBuffer.from_numpy(np.ascontiguousarray(a))


def dequantize(raw, n: int, ggml_type: int, dtype=np.float32, stream=None) -> DeviceBuffer:
  """Raw GGUF block bytes -> n values (fp32 bit-exact with the reference; fp16 = its RNE cast)."""
  if ggml_type not in GGML_QUANT: raise ValueError(f"GGML type '{ggml_type}' is not supported!")   # gguf.py:119
  raw = _as_device(raw)
  out = DeviceBuffer.empty((n,), dtype)
  check(_lib.load().b200q_dequant_raw(ggml_type, raw.ptr, out.ptr, n, _DT[np.dtype(dtype)], stream_ptr(stream)))
  return out


class PackedWeight:
  """A [n_out, n_in] quantised matrix re-tiled for the GEMV kernels (lossless)."""
  def __init__(self, qtype: int, n_out: int, n_in: int, buf: DeviceBuffer, interleaved: bool):
    self.qtype, self.n_out, self.n_in, self.buf, self.interleaved = qtype, n_out, n_in, buf, interleaved

  @property
  def rows(self) -> int: return 2 * self.n_out if self.interleaved else self.n_out

  @property
  def algorithmic_bytes(self) -> int:
    nel, nby = GGML_QUANT[self.qtype]
    return self.rows * self.n_in // nel * nby

  def dequantize(self, dtype=np.float32) -> DeviceBuffer:
    """Back to row-major values, rows in packed order (checks that packing lost nothing)."""
    rows = -(-self.rows // 16) * 16 if self.interleaved else self.n_out
    out = DeviceBuffer.empty((rows, self.n_in), dtype)
    check(_lib.load().b200q_dequant_packed(self.qtype, self.buf.ptr, out.ptr, rows, self.n_in, _DT[np.dtype(dtype)], None))
    return out


def packed_bytes(qtype: int, rows: int, n_in: int) -> int:
  n = _lib.load().b200q_packed_bytes(qtype, rows, n_in)
  if n == 0: raise ValueError(f"cannot pack GGML type {qtype} of shape ({rows}, {n_in})")
  return n


def repack(raw, n_out: int, n_in: int, qtype: int, raw_up=None, out: DeviceBuffer = None, out_offset: int = 0, stream=None) -> PackedWeight:
  """Re-tile raw GGUF blocks of a [n_out, n_in] weight.  With `raw_up` the two
  matrices (gate, up) are interleaved for the fused SwiGLU epilogue.  `out` /
  `out_offset` place the tiles inside a larger buffer (e.g. q|k|v back to back)."""
  if n_in % GGML_QUANT[qtype][0]: raise ValueError(f"n_in={n_in} is not a multiple of the block size")
  raw, raw_up = _as_device(raw), _as_device(raw_up)
  rows = 2 * (-(-n_out // 8) * 8) if raw_up is not None else n_out
  nbytes = packed_bytes(qtype, rows, n_in)
  if out is None: out, out_offset = DeviceBuffer(nbytes), 0
  assert out_offset % 16 == 0 and out_offset + nbytes <= out.nbytes
  check(_lib.load().b200q_repack(qtype, raw.ptr, ptr_of(raw_up), out.ptr + out_offset, n_out, n_in, stream_ptr(stream)))
  if stream is None: check(_lib.load().b200q_device_synchronize())   # raw staging buffers may be freed by the caller
  pw = PackedWeight(qtype, n_out, n_in, out, raw_up is not None)
  pw.offset = out_offset
  return pw


def gemv(w_ptr: int, qtype: int, n_out: int, n_in: int, x, y, m: int = 1, x_dtype=F32, y_dtype=F32, norm_weight=None, norm_eps: float = 0.0,
         epilogue: int = EPI_LINEAR, bias=None, residual=None, flags: int = 0, max_ctas: int = 0, stream=None, xq_in=None, ss_in=None,
         ss_count: int = 0, xq_out=None, xq_out_norm_weight=None, ss_out=None, residual_scale: float = 1.0, peers=None, peer_rank: int = 0,
         xq_out_stage=None) -> None:
  """One launch of the fused dequant-GEMV (all pointers raw device addresses or buffers).  peers: a ctypes array of every rank's
  mailbox pointer (tensor_parallel.PeerMailbox.targets): the output row also goes into slot `peer_rank` of each."""
  a = _lib.GemvArgs(qtype, n_out, n_in, m, w_ptr, ptr_of(x), x_dtype, y_dtype, ptr_of(norm_weight), norm_eps, epilogue, ptr_of(bias),
                    ptr_of(residual), ptr_of(y), flags, max_ctas, ptr_of(xq_in), ptr_of(ss_in), ss_count, ptr_of(xq_out),
                    ptr_of(xq_out_norm_weight), ptr_of(ss_out), residual_scale, peers, len(peers) if peers is not None else 0, peer_rank,
                    ptr_of(xq_out_stage))
  check(_lib.load().b200q_gemv(ctypes.byref(a), stream_ptr(stream)))


import os
PIPELINED_GEMM = os.environ.get("B200Q_PIPELINED_GEMM", "1") == "1"   # qgemm uses the pipelined kernel when it is handed a workspace


def qgemm_workspace_bytes(m: int, n_in: int) -> int:
  return int(_lib.load().b200q_qgemm_workspace_bytes(m, n_in))


def qgemm(w_ptr: int, qtype: int, n_out: int, n_in: int, x, y, m: int, x_dtype=F32, y_dtype=F32, bias=None, residual=None,
          epilogue: int = EPI_LINEAR, stream=None, workspace: DeviceBuffer = None) -> None:
  """Batched / prefill linear on the tcgen05 tensor cores: the weights are streamed once per 128 activation rows.  With a `workspace`
  (qgemm_workspace_bytes(m, n_in) bytes) the pipelined kernel runs: activations pre-split once, bulk-copied operands, MMAs under the unpacking."""
  lib = _lib.load()
  if workspace is not None and PIPELINED_GEMM:
    check(lib.b200q_qgemm_ws(qtype, w_ptr, ptr_of(x), x_dtype, ptr_of(bias), ptr_of(residual), epilogue, ptr_of(y), y_dtype, m, n_out, n_in,
                             workspace.ptr, workspace.nbytes, stream_ptr(stream)))
    return
  check(lib.b200q_qgemm(qtype, w_ptr, ptr_of(x), x_dtype, ptr_of(bias), ptr_of(residual), epilogue, ptr_of(y), y_dtype, m, n_out, n_in,
                        stream_ptr(stream)))


FEW_ROW_FUSED = os.environ.get("B200Q_FEW_ROW_FUSED", "1") == "1"      # batched decode with few rows: the int8-MMA few-row kernel
# ... up to this many rows, 8 per pass over the weights (measured at 16 / 32 sequences of the 7B Q8_0 shape: 5.1 / 10.2 ms per step
# against 10.5 / 11.9 on the tcgen05 few-row GEMM, whose unpacking to fp16 halves costs more than streaming the weights again)
FEW_ROW_MAX = int(os.environ.get("B200Q_FEW_ROW_MAX", "32"))


def qgemv_rows_workspace_bytes(m: int, n_out: int, n_in: int) -> int:
  return int(_lib.load().b200q_qgemv_rows_workspace_bytes(m, n_out, n_in))


def qgemv_rows(w_ptr: int, qtype: int, n_out: int, n_in: int, x, y, m: int, workspace: DeviceBuffer, x_dtype=F32, y_dtype=F32, bias=None, residual=None,
               epilogue: int = EPI_LINEAR, norm_weight=None, norm_eps: float = 0.0, stream=None) -> None:
  """The same Linear for a few activation rows (batched decode) on the int8 tensor cores: weights streamed once per 8 rows.
  norm_weight (fp16 [n_in]): the RMSNorm in front of the Linear, folded into the quantising pre-pass (x is then the un-normed fp32 rows)."""
  check(_lib.load().b200q_qgemv_rows_norm(qtype, w_ptr, ptr_of(x), x_dtype, ptr_of(norm_weight), norm_eps, ptr_of(bias), ptr_of(residual), epilogue, ptr_of(y),
                                          y_dtype, m, n_out, n_in, workspace.ptr, workspace.nbytes, stream_ptr(stream)))


def qgemm_skinny_workspace_bytes(m: int, n_out: int, n_in: int) -> int:
  return int(_lib.load().b200q_qgemm_skinny_workspace_bytes(m, n_out, n_in))


def qgemm_skinny(w_ptr: int, qtype: int, n_out: int, n_in: int, x, y, m: int, workspace: DeviceBuffer, x_dtype=F32, y_dtype=F32, bias=None, residual=None,
                 epilogue: int = EPI_LINEAR, stream=None) -> None:
  """The same Linear for at most 32 activation rows (batched decode): swapped operands, split K, partial sums through `workspace`."""
  check(_lib.load().b200q_qgemm_skinny(qtype, w_ptr, ptr_of(x), x_dtype, ptr_of(bias), ptr_of(residual), epilogue, ptr_of(y), y_dtype, m, n_out, n_in,
                                       workspace.ptr, workspace.nbytes, stream_ptr(stream)))


GEMM_MIN_ROWS = 4   # from this many activation rows on, QuantLinear uses the tensor-core GEMM instead of one GEMV per row


GGML_F32, GGML_F16, GGML_BF16 = 0, 1, 30                # unquantised GGUF tensor types (tinygrad/llm/gguf.py:25-27)
_DENSE_DT = {GGML_F32: (_lib.F32, np.float32), GGML_F16: (_lib.F16, np.float16), GGML_BF16: (_lib.BF16, np.uint16)}


def gemv_dense(w, w_dtype: int, n_out: int, n_in: int, x, y, m: int = 1, x_dtype=F32, y_dtype=F32, norm_weight=None, norm_eps: float = 0.0,
               bias=None, residual=None, flags: int = 0, stream=None) -> None:
  """One launch of the dense-weight GEMV (weight row-major fp16 / bf16 / fp32 on the device)."""
  check(_lib.load().b200q_gemv_dense(ptr_of(w), w_dtype, n_out, n_in, m, ptr_of(x), x_dtype, ptr_of(norm_weight), norm_eps, ptr_of(bias),
                                     ptr_of(residual), ptr_of(y), y_dtype, flags, stream_ptr(stream)))


def _to_bf16_bits(a: np.ndarray) -> np.ndarray:
  """fp32 -> bf16 bit patterns, round to nearest even (tinygrad/dtype.py:222-226)."""
  u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
  return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


class DenseWeight:
  """A [n_out, n_in] weight kept as plain values on the device.  F32 / F16 / BF16 tensors stay as stored; Q6_K blocks are
  dequantised once to fp16 (the cast the reference applies to every loaded tensor, tinygrad/llm/model.py:376)."""
  def __init__(self, raw, n_out: int, n_in: int, ggml_type: int):
    self.n_out, self.n_in = n_out, n_in
    if ggml_type in _DENSE_DT:
      self.dtype, npdt = _DENSE_DT[ggml_type]
      a = np.ascontiguousarray(raw)
      if a.dtype == np.uint8: a = a.view(npdt)                     # raw tensor bytes
      elif ggml_type != GGML_BF16: a = a.astype(npdt)
      elif a.dtype == np.uint16: pass                              # bf16 bit patterns
      else: a = _to_bf16_bits(a.astype(np.float32))                # values (GGUFTensor.numpy widens BF16 to fp32: exact round trip)
      if a.size != n_out * n_in: raise ValueError(f"weight has {a.size} values, expected {n_out}x{n_in}")
      self.buf = DeviceBuffer.from_numpy(a.reshape(n_out, n_in))
    elif ggml_type in GGML_QUANT:
      self.dtype, self.buf = _lib.F16, dequantize(raw, n_out * n_in, ggml_type, np.float16)
    else:
      raise ValueError(f"GGML type '{ggml_type}' is not supported!")

  @property
  def algorithmic_bytes(self) -> int: return self.buf.nbytes


class QuantLinear:
  """Drop-in for `nn.Linear` holding a GGUF weight.

  `QuantLinear(in_features, out_features, ggml_type, raw_blocks, bias)`; calling it
  on activations of shape (..., in_features), fp16 or fp32, returns
  (..., out_features) in the activation dtype, as
  `x.linear(weight.transpose(), bias)` does (tinygrad/nn/__init__.py:177).
  Q4_0 / Q8_0 weights run the fused dequant kernels (GEMV below 4 rows, tcgen05 GEMM from 4 rows on); Q6_K weights (in_features a
  multiple of 256) the fused GEMV for any number of rows; F32 / F16 / BF16 weights the dense GEMV, 4 activation rows per launch."""
  def __init__(self, in_features: int, out_features: int, ggml_type: int, raw, bias=None):
    self.in_features, self.out_features, self.ggml_type = in_features, out_features, ggml_type
    self.fused = ggml_type in (Q4_0, Q8_0) or (ggml_type == Q6_K and in_features % 256 == 0)
    self.weight = repack(raw, out_features, in_features, ggml_type) if self.fused else DenseWeight(raw, out_features, in_features, ggml_type)
    self.bias = None if bias is None else DeviceBuffer.from_numpy(np.asarray(bias, dtype=np.float16))
    self._ws = None      # activation tiles of the pipelined GEMM, grown on demand

  def __call__(self, x: DeviceBuffer, stream=None) -> DeviceBuffer:
    if x.dtype not in _DT: raise TypeError(f"activations must be float16 or float32, got {x.dtype}")
    if x.shape[-1] != self.in_features: raise ValueError(f"Input Tensor shapes {x.shape} cannot be multiplied with in_features={self.in_features}")
    m = int(np.prod(x.shape[:-1], dtype=np.int64))
    y = DeviceBuffer.empty((*x.shape[:-1], self.out_features), x.dtype)
    dt = _DT[x.dtype]
    if not self.fused:
      if m: gemv_dense(self.weight.buf, self.weight.dtype, self.out_features, self.in_features, x, y, m=m, x_dtype=dt, y_dtype=dt, bias=self.bias,
                       stream=stream)
    elif m >= GEMM_MIN_ROWS and self.ggml_type != Q6_K:
      need = qgemm_workspace_bytes(m, self.in_features)
      if self._ws is None or self._ws.nbytes < need: self._ws = DeviceBuffer(need)
      qgemm(self.weight.buf.ptr, self.ggml_type, self.out_features, self.in_features, x, y, m, x_dtype=dt, y_dtype=dt, bias=self.bias, stream=stream,
            workspace=self._ws)
    elif m:
      gemv(self.weight.buf.ptr, self.ggml_type, self.out_features, self.in_features, x, y, m=m, x_dtype=dt, y_dtype=dt, bias=self.bias, stream=stream)
    return y
