"""ctypes access to the C restatement (test infrastructure / timed CPU baseline)."""
import ctypes, os
import numpy as np
from .build import build_oracle

_lib = None


def lib():
  global _lib
  if _lib is None:
    _lib = ctypes.CDLL(str(build_oracle()))
    _lib.qgemv_cpu.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    _lib.dequant_cpu.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
    _lib.dequant_cpu.restype = ctypes.c_int
    _lib.rmsnorm_cpu.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float]
  return _lib


def qgemv(qtype: int, raw: np.ndarray, x: np.ndarray, n_out: int, n_in: int) -> np.ndarray:
  raw, x = np.ascontiguousarray(raw, dtype=np.uint8), np.ascontiguousarray(x, dtype=np.float32)
  y = np.empty(n_out, dtype=np.float32)
  lib().qgemv_cpu(qtype, raw.ctypes.data, x.ctypes.data, y.ctypes.data, n_out, n_in)
  return y


def dequantize(raw: np.ndarray, n: int, qtype: int) -> np.ndarray:
  """The C restatement of `ggml_data_to_tensor` (fast enough for full-size matrices); same values as oracle.ggml_quant.dequantize."""
  raw = np.ascontiguousarray(raw, dtype=np.uint8)
  out = np.empty(n, dtype=np.float32)
  if lib().dequant_cpu(qtype, raw.ctypes.data, out.ctypes.data, n) != 0: raise ValueError(f"GGML type {qtype} is not restated in C")
  return out


def weight_matrix(raw: np.ndarray, n_out: int, n_in: int, qtype: int) -> np.ndarray:
  return dequantize(raw, n_out * n_in, qtype).reshape(n_out, n_in)


def n_threads() -> int:
  return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
