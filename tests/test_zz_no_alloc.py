"""The attention entry point for callers that cannot allocate device memory.

Hosts that own every byte of device memory (a frozen serving pool, a planner that replays captured work) have no
scratch buffer to hand to `b200q_attn_decode`; `b200q_attn_decode_static` keeps its scratch in an array built into
the library.  It must give the same result as the ordinary entry point, call after call, although every call reuses
the same array.  This file sorts last so that a run stopping at the first failure has already run everything else."""
import ctypes
import numpy as np
import pytest
from gpu_util import need_gpu, assert_close

pytestmark = pytest.mark.gpu


def _case(n_heads, n_kv, hd, pos, ctx, seed):
  from tinygrad_b200.model import precompute_freqs_cis
  rng = np.random.default_rng(seed)
  qkv = rng.standard_normal((n_heads + 2 * n_kv) * hd).astype(np.float32)
  kc = (rng.standard_normal((n_kv, ctx, hd)) * 0.5).astype(np.float16)
  vc = rng.standard_normal((n_kv, ctx, hd)).astype(np.float16)
  return qkv, kc, vc, precompute_freqs_cis(hd, ctx, 500000.0), np.array([pos], np.int32)


def _run(entry, n_heads, n_kv, hd, ctx, arrays, with_scratch):
  from tinygrad_b200 import _lib
  from tinygrad_b200.runtime import DeviceBuffer
  lib = _lib.load()
  qkv, kc, vc, fc, pos = (DeviceBuffer.from_numpy(a) for a in arrays)
  out = DeviceBuffer.empty((n_heads * hd,), np.float32, zero=True)
  n_split = lib.b200q_attn_min_split(ctx)
  scratch = DeviceBuffer(lib.b200q_attn_scratch_bytes(n_heads, n_kv, hd, n_split), zero=True) if with_scratch else None
  a = _lib.AttnArgs(qkv.ptr, kc.ptr, vc.ptr, _lib.F16, fc.ptr, pos.ptr, out.ptr, scratch.ptr if scratch else None, n_heads, n_kv, hd, hd, ctx,
                    n_split, 0, None)
  _lib.check(getattr(lib, entry)(ctypes.byref(a), None))
  return out.numpy(), kc.numpy()


def test_static_scratch_attention_matches_the_ordinary_entry_point_twice_in_a_row():
  need_gpu()
  # two calls in a row with different geometry: the second finds the first one's leftovers in the shared array
  for n_heads, n_kv, hd, pos, ctx, seed in ((32, 8, 128, 700, 1024, 1), (28, 4, 128, 300, 2048, 2), (32, 8, 128, 701, 1024, 3)):
    arrays = _case(n_heads, n_kv, hd, pos, ctx, seed)
    want, want_k = _run("b200q_attn_decode", n_heads, n_kv, hd, ctx, arrays, True)
    got, got_k = _run("b200q_attn_decode_static", n_heads, n_kv, hd, ctx, arrays, False)
    assert_close(got, want, tol=2e-3, what="static-scratch attention vs ordinary")
    np.testing.assert_array_equal(got_k, want_k)


def test_static_scratch_rejects_what_does_not_fit():
  need_gpu()
  from tinygrad_b200 import _lib
  lib = _lib.load()
  assert lib.b200q_attn_decode_static_capacity() == 2 << 20
  n_split = lib.b200q_attn_min_split(16384)
  assert lib.b200q_attn_scratch_bytes(64, 8, 128, n_split) > lib.b200q_attn_decode_static_capacity()
  a = _lib.AttnArgs(16, 16, 16, _lib.F16, 16, 16, 16, None, 64, 8, 128, 128, 16384, n_split, 0, None)
  assert lib.b200q_attn_decode_static(ctypes.byref(a), None) == -6     # B200Q_ERR_TOO_LARGE, nothing launched
