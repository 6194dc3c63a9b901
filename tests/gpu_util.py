"""Helpers shared by the GPU parity tests."""
import numpy as np
import pytest


def need_gpu():
  from tinygrad_b200 import build, runtime
  build.build_lib()
  if runtime.device_count() < 1: pytest.fail("a test marked gpu ran without a CUDA device")


def assert_close(got, ref, tol=1e-2, what=""):
  """The path's stated tolerance, read as the reference's own GEMV test reads it
  (test/unit/test_gguf.py:229-231, atol = rtol = 1e-2): |got - ref| <= tol + tol * |ref| elementwise."""
  got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
  err = np.abs(got - ref)
  bad = err > tol + tol * np.abs(ref)
  assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} beyond {tol}: max abs err {err.max():.3e}, at ref {ref.reshape(-1)[err.argmax()]:.4f}"
