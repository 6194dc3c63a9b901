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


def _case(n_heads, n_kv, hd, pos, ctx, seed, kv_dtype=np.float16):
  from tinygrad_b200.model import precompute_freqs_cis
  rng = np.random.default_rng(seed)
  qkv = rng.standard_normal((n_heads + 2 * n_kv) * hd).astype(np.float32)
  kc = (rng.standard_normal((n_kv, ctx, hd)) * 0.5).astype(kv_dtype)
  vc = rng.standard_normal((n_kv, ctx, hd)).astype(kv_dtype)
  return qkv, kc, vc, precompute_freqs_cis(hd, ctx, 500000.0), np.array([pos], np.int32)


def _run(entry, n_heads, n_kv, hd, ctx, arrays, with_scratch, record=False):
  from tinygrad_b200 import _lib
  from tinygrad_b200.runtime import DeviceBuffer
  lib = _lib.load()
  qkv, kc, vc, fc, pos = (DeviceBuffer.from_numpy(a) for a in arrays)
  out = DeviceBuffer.empty((n_heads * hd,), np.float32, zero=True)
  n_split = lib.b200q_attn_min_split(ctx)
  scratch = DeviceBuffer(lib.b200q_attn_scratch_bytes(n_heads, n_kv, hd, n_split), zero=True) if with_scratch else None
  xq = DeviceBuffer(lib.b200q_xq_bytes(n_heads * hd), (lib.b200q_xq_bytes(n_heads * hd),), np.uint8, zero=True) if record else None
  a = _lib.AttnArgs(qkv.ptr, kc.ptr, vc.ptr, _lib.F16 if arrays[1].dtype == np.float16 else _lib.F32, fc.ptr, pos.ptr, out.ptr,
                    scratch.ptr if scratch else None, n_heads, n_kv, hd, hd, ctx, n_split, 0, xq.ptr if xq else None)
  _lib.check(getattr(lib, entry)(ctypes.byref(a), None))
  return out.numpy(), kc.numpy(), (xq.numpy() if xq else None)


def test_static_scratch_attention_matches_the_ordinary_entry_point_twice_in_a_row():
  need_gpu()
  # two calls in a row with different geometry: the second finds the first one's leftovers in the shared array
  for n_heads, n_kv, hd, pos, ctx, seed in ((32, 8, 128, 700, 1024, 1), (28, 4, 128, 300, 2048, 2), (32, 8, 128, 701, 1024, 3)):
    arrays = _case(n_heads, n_kv, hd, pos, ctx, seed)
    want, want_k, _ = _run("b200q_attn_decode", n_heads, n_kv, hd, ctx, arrays, True)
    got, got_k, _ = _run("b200q_attn_decode_static", n_heads, n_kv, hd, ctx, arrays, False)
    assert_close(got, want, tol=2e-3, what="static-scratch attention vs ordinary")
    np.testing.assert_array_equal(got_k, want_k)


def test_static_scratch_attention_fp32_cache_and_quantised_record():
  """The other two shapes of the call: an fp32 KV cache, and the output row also handed over as a quantised record."""
  need_gpu()
  for kv_dtype, record in ((np.float32, False), (np.float16, True), (np.float32, True)):
    arrays = _case(16, 4, 128, 333, 512, 7, kv_dtype)
    want, want_k, want_xq = _run("b200q_attn_decode", 16, 4, 128, 512, arrays, True, record)
    got, got_k, got_xq = _run("b200q_attn_decode_static", 16, 4, 128, 512, arrays, False, record)
    assert_close(got, want, tol=2e-3, what="static-scratch attention vs ordinary")
    np.testing.assert_array_equal(got_k, want_k)
    if record: np.testing.assert_array_equal(got_xq, want_xq)      # same kernel, same merge order: the record is bit-identical


def test_static_scratch_validates_before_it_enqueues_anything():
  need_gpu()
  from tinygrad_b200 import _lib
  lib = _lib.load()
  a = _lib.AttnArgs(16, 16, 16, _lib.F16, 16, 16, 16, None, 6, 4, 128, 128, 64, 1, 0, None)      # heads not a multiple of kv heads
  assert lib.b200q_attn_decode_static(ctypes.byref(a), None) == -1


def test_static_scratch_rejects_what_does_not_fit():
  need_gpu()
  from tinygrad_b200 import _lib
  lib = _lib.load()
  assert lib.b200q_attn_decode_static_capacity() == 2 << 20
  n_split = lib.b200q_attn_min_split(16384)
  assert lib.b200q_attn_scratch_bytes(64, 8, 128, n_split) > lib.b200q_attn_decode_static_capacity()
  a = _lib.AttnArgs(16, 16, 16, _lib.F16, 16, 16, 16, None, 64, 8, 128, 128, 16384, n_split, 0, None)
  assert lib.b200q_attn_decode_static(ctypes.byref(a), None) == -6     # B200Q_ERR_TOO_LARGE, nothing launched
