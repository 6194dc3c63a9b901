"""`FP8Linear` of extra/fp8/fp8_linear.py:43-63 on the B200 path: per-tensor E4M3 quantisation of weight and activations, the product on
the tcgen05 tensor cores with fp32 accumulation, the two scale factors and the bias applied afterwards.  Inference only: the weight is
quantised once (the reference re-quantises it on every call because it trains it); call `requantize()` after changing `weight`."""
import numpy as np
from . import _lib
from ._lib import check, F32, F16, BF16
from .runtime import DeviceBuffer, stream_ptr

_DT = {np.dtype(np.float32): F32, np.dtype(np.float16): F16}


def quantize_to_fp8(x: DeviceBuffer, n: int, x_dtype: int, stream=None):
  """-> (E4M3 codes [n] uint8, factor: one device float = 1 / scale); `quantize_to_fp8`, extra/fp8/fp8_linear.py:4-16."""
  lib, s = _lib.load(), stream_ptr(stream)
  q, amax, factor = DeviceBuffer.empty((n,), np.uint8), DeviceBuffer.empty((1,), np.float32), DeviceBuffer.empty((1,), np.float32)
  check(lib.b200q_fp8_absmax(x.ptr, x_dtype, n, amax.ptr, s))
  check(lib.b200q_fp8_quantize(x.ptr, x_dtype, n, amax.ptr, q.ptr, factor.ptr, s))
  return q, factor


class FP8Linear:
  """FP8Linear(in_features, out_features, weight [out, in] fp32, bias [out] or None); `__call__(x)` with x (..., in) fp32 / fp16 on the device
  returns (..., out) in x's dtype.  out_features must be a multiple of 256 and in_features of 128 (the tensor-core tile sizes)."""
  def __init__(self, in_features: int, out_features: int, weight: np.ndarray, bias=None):
    if out_features % 256 or in_features % 128: raise ValueError("out_features % 256 == in_features % 128 == 0 is required")
    self.in_features, self.out_features = in_features, out_features
    self.weight = DeviceBuffer.from_numpy(np.ascontiguousarray(weight, dtype=np.float32).reshape(out_features, in_features))
    self.bias = None if bias is None else DeviceBuffer.from_numpy(np.asarray(bias, dtype=np.float32).reshape(out_features))
    self._w_e8 = DeviceBuffer(out_features * in_features // 32)
    check(_lib.load().b200q_memset(self._w_e8.ptr, 127, self._w_e8.nbytes, None))       # E8M0 127 = 2^0: the block scales are all one
    self._ws = {}
    self.requantize()

  def requantize(self) -> None:
    self.w_q, self.w_factor = quantize_to_fp8(self.weight, self.out_features * self.in_features, F32)

  def _workspace(self, m: int):
    w = self._ws.get(m)
    if w is None:
      lib, mp = _lib.load(), -(-m // 256) * 256
      w = dict(mp=mp, x_q=DeviceBuffer.empty((mp, self.in_features), np.uint8, zero=True), x_e8=DeviceBuffer(mp * self.in_features // 32),
               amax=DeviceBuffer.empty((1,), np.float32), factor=DeviceBuffer.empty((1,), np.float32), off=DeviceBuffer.from_numpy(np.array([0, mp], np.int32)),
               acc=DeviceBuffer.empty((mp, self.out_features), np.float32))
      check(lib.b200q_memset(w["x_e8"].ptr, 127, w["x_e8"].nbytes, None))
      self._ws[m] = w
    return w

  def __call__(self, x: DeviceBuffer, stream=None) -> DeviceBuffer:
    if x.dtype not in _DT: raise TypeError(f"activations must be float16 or float32, got {x.dtype}")
    if x.shape[-1] != self.in_features: raise ValueError(f"Input Tensor shapes {x.shape} cannot be multiplied with in_features={self.in_features}")
    m = int(np.prod(x.shape[:-1], dtype=np.int64))
    y = DeviceBuffer.empty((*x.shape[:-1], self.out_features), x.dtype)
    if m == 0: return y
    lib, s, dt, w = _lib.load(), stream_ptr(stream), _DT[x.dtype], self._workspace(m)
    check(lib.b200q_fp8_absmax(x.ptr, dt, m * self.in_features, w["amax"].ptr, s))
    check(lib.b200q_fp8_quantize(x.ptr, dt, m * self.in_features, w["amax"].ptr, w["x_q"].ptr, w["factor"].ptr, s))      # rows past m stay zero
    check(lib.b200q_grouped_mxfp8_gemm_f32(w["x_q"].ptr, w["x_e8"].ptr, self.w_q.ptr, self._w_e8.ptr, w["off"].ptr, 1, w["mp"], self.out_features,
                                           self.in_features, w["acc"].ptr, s))
    check(lib.b200q_fp8_scale_bias(w["acc"].ptr, m, self.out_features, self.w_factor.ptr, w["factor"].ptr, self.bias.ptr if self.bias else None, y.ptr, dt, s))
    return y
