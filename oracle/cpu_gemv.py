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
    _lib.rmsnorm_cpu.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float]
  return _lib


def qgemv(qtype: int, raw: np.ndarray, x: np.ndarray, n_out: int, n_in: int) -> np.ndarray:
  raw, x = np.ascontiguousarray(raw, dtype=np.uint8), np.ascontiguousarray(x, dtype=np.float32)
  y = np.empty(n_out, dtype=np.float32)
  lib().qgemv_cpu(qtype, raw.ctypes.data, x.ctypes.data, y.ctypes.data, n_out, n_in)
  return y


def n_threads() -> int:
  return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
