"""GPU parity of the MXFP8 mixture-of-experts path against the oracle (itself pinned on the reference's goldens)."""
import numpy as np
import pytest
from oracle import mxfp8 as mx, llm
from gpu_util import need_gpu, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _gpu(): need_gpu()


def _quant(x, dtype_flag):
  from tinygrad_b200 import moe
  from tinygrad_b200.runtime import DeviceBuffer
  rows, k = x.shape
  q, e8 = moe.quantize_mxfp8(DeviceBuffer.from_numpy(x), rows, k, dtype_flag)
  return q.numpy(), e8.numpy()


def test_quantize_mxfp8_golden_bit_exact(golden):
  from tinygrad_b200 import _lib
  g = golden("mxfp8")
  q, e8 = _quant(g["x"], _lib.F32)
  np.testing.assert_array_equal(e8, g["e8"])
  np.testing.assert_array_equal(q, g["q"])


def test_quantize_mxfp8_random_and_edges_bit_exact():
  from tinygrad_b200 import _lib, moe
  rng = np.random.default_rng(0)
  x = (rng.standard_normal((257, 96)) * np.exp(rng.uniform(-30, 30, (257, 1)))).astype(np.float32)
  x[0, :32] = 0.0                                                  # all-zero block
  x[1, :32] = np.float32(8.0) * (1 - 2.0 ** -24)                   # largest value below a power of two
  x[2, :32] = [448.0, -448.0, 449.0, 1e30] * 8                     # saturation
  x[3, :32] = np.float32(2.0) ** np.arange(-16, 16)                # exact powers of two
  q, e8 = _quant(x, _lib.F32)
  rq, re8 = mx.quantize_mxfp8(x)
  np.testing.assert_array_equal(e8, re8)
  np.testing.assert_array_equal(q, rq)
  xb = moe.to_bf16_bits(x)                                         # bf16 input: same function of the bf16 values
  q, e8 = _quant(xb, _lib.BF16)
  rq, re8 = mx.quantize_mxfp8(moe.from_bf16_bits(xb))
  np.testing.assert_array_equal(e8, re8)
  np.testing.assert_array_equal(q, rq)


def _route(logits, k, mode):
  from tinygrad_b200 import moe
  from tinygrad_b200.runtime import DeviceBuffer
  T, E = logits.shape
  r = moe.Routing(T, E, k, mode).run(DeviceBuffer.from_numpy(logits))
  return r, r.topi.numpy(), r.weights.numpy(), r.dest_row.numpy(), r.off.numpy()


def test_route_golden(golden):
  g = golden("mxfp8")
  r, topi, w, dest, off = _route(g["route_logits"], 2, 0)
  np.testing.assert_array_equal(dest, g["route_dest_row"][0])
  np.testing.assert_array_equal(off, g["route_off"][0])
  np.testing.assert_allclose(w, g["route_weights"][0], rtol=1e-6)
  assert r.m_l == int(g["route_m_l"])


@pytest.mark.parametrize("T,E,k", [(4096, 64, 8), (1000, 8, 2), (37, 128, 6), (3000, 256, 4)])
def test_route_random_matches_oracle(T, E, k):
  logits = np.random.default_rng(T).standard_normal((T, E)).astype(np.float32)
  logits[5, :4] = logits[5, 0]                                      # ties: the lower index ranks higher
  r, topi, w, dest, off = _route(logits, k, 0)
  rw, rtopi, rdest, roff, m_l = mx.route(logits, k, E)
  np.testing.assert_array_equal(topi, rtopi)
  np.testing.assert_array_equal(dest, rdest)
  np.testing.assert_array_equal(off, roff)
  np.testing.assert_allclose(w, rw, rtol=2e-6)
  assert r.m_l == m_l and len(set(dest.tolist())) == T * k           # a permutation into distinct rows
  # mode 1: softmax over all experts, compare-count top-k in ascending order (tinygrad/llm/model.py:35-41)
  _, topi1, w1, dest1, off1 = _route(logits, k, 1)
  scores = llm.softmax(logits)
  _, sel = llm.pairwise_topk(logits[None], k)
  np.testing.assert_array_equal(topi1, sel[0])
  np.testing.assert_allclose(w1, np.take_along_axis(scores, sel[0].astype(np.int64), -1), rtol=2e-6)
  np.testing.assert_array_equal(off1, roff)


@pytest.mark.parametrize("func,norm,scale,with_bias", [("softmax", False, 1.0, False), ("softmax", True, 1.0, False), ("softmax", True, 1.0, True),
                                                       ("sigmoid", True, 2.5, False), ("sigmoid", False, 1.0, True), ("softmax_weight", False, 1.0, False),
                                                       ("sqrt_softplus", True, 1.5, True), ("sqrt_softplus", False, 1.0, False)])
def test_route_gating_matches_oracle(func, norm, scale, with_bias):
  """Every gating of tinygrad's MoE block (tinygrad/llm/model.py:110-128): selection (with ties and a selection bias), weights, placement."""
  from tinygrad_b200 import moe
  from tinygrad_b200.runtime import DeviceBuffer
  T, E, k = 777, 64, 6
  rng = np.random.default_rng(E + k)
  logits = (rng.standard_normal((T, E)) * 2).astype(np.float32)
  logits[3, 10:14] = logits[3, 10]                                  # ties: the lower index ranks higher
  logits[4, :] = 30.0; logits[5, :] = -30.0                         # saturated scores
  bias = (rng.standard_normal(E) * 0.5).astype(np.float32) if with_bias else None
  g = moe.Gating(func, norm, scale, bias)
  r = moe.Routing(T, E, k, g).run(DeviceBuffer.from_numpy(logits))
  sel, probs = llm.moe_gate(logits, moe.GATING[func], norm, k, scale, bias)
  topi, w, dest, off = r.topi.numpy(), r.weights.numpy(), r.dest_row.numpy(), r.off.numpy()
  rows = [t for t in range(T) if t not in (4, 5)]                  # all-equal scores: any consistent order of float ties is checked below
  np.testing.assert_array_equal(topi[rows], sel[rows])
  np.testing.assert_allclose(w[rows], probs[rows], rtol=2e-5, atol=1e-7)
  if not with_bias: np.testing.assert_array_equal(topi[4], np.arange(k)[::-1])      # equal scores: experts k-1 .. 0 in ascending rank
  np.testing.assert_allclose(w[[4, 5]].sum(-1), probs[[4, 5]].sum(-1), rtol=1e-4)
  counts = np.bincount(topi.reshape(-1), minlength=E)
  np.testing.assert_array_equal(off, np.concatenate([[0], np.cumsum((counts + 255) // 256 * 256)]))
  assert len(set(dest.tolist())) == T * k
  e_of_row = np.searchsorted(off, dest, side="right") - 1
  np.testing.assert_array_equal(e_of_row, topi.reshape(-1))         # every pair sits inside its expert's group


def test_grouped_gemm_matches_oracle():
  from tinygrad_b200 import _lib, moe
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(1)
  E, N, K = 4, 256, 384
  off = np.array([0, 256, 256, 768, 1024], np.int32)                # expert 1 got no rows; 1280 rows allocated, 256 unused
  M = 1280
  a = rng.standard_normal((M, K)).astype(np.float32); a[700:768] = 0  # padding rows inside a group are zero
  w = (rng.standard_normal((E, N, K)) * 0.02).astype(np.float32)
  a_q, a_e8 = mx.quantize_mxfp8(a); w_q, w_e8 = mx.quantize_mxfp8(w)
  ref = mx.to_bf16(mx.grouped_mx_gemm(a_q, a_e8, w_q, w_e8, off))
  d = [DeviceBuffer.from_numpy(v) for v in (a_q, a_e8, w_q, w_e8, off)]
  c = DeviceBuffer.from_numpy(np.full((M, N), 0x7FC0, np.uint16))     # NaN canary
  _lib.check(_lib.load().b200q_grouped_mxfp8_gemm(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d[4].ptr, E, M, N, K, c.ptr, None))
  got = c.numpy()
  assert (got[1024:] == 0x7FC0).all()                               # rows past the last group untouched
  assert_close(moe.from_bf16_bits(got[:1024]), ref[:1024], tol=1e-2, what="grouped MXFP8 GEMM")


def test_grouped_gemm_matches_reference_matmul_mx(golden):
  """The contraction against the reference's own portable MXFP8 matmul (matmul_mx, examples/mlperf/models/gpt_oss.py:64-83):
  its inputs, padded with zero rows / columns to the kernel's 256 / 256 / 128 granularity, as one expert group."""
  from tinygrad_b200 import _lib, moe
  from tinygrad_b200.runtime import DeviceBuffer
  g = golden("mxgemm")
  (M, K), N = g["x_bf16"].shape, g["w"].shape[0]
  x, w = np.zeros((256, 128), np.float32), np.zeros((256, 128), np.float32)
  x[:M, :K], w[:N, :K] = g["x_bf16"], g["w"]
  xq, xe = moe.quantize_mxfp8(DeviceBuffer.from_numpy(moe.to_bf16_bits(x)), 256, 128, _lib.BF16)
  wq, we = moe.quantize_mxfp8(DeviceBuffer.from_numpy(w), 256, 128, _lib.F32)
  np.testing.assert_array_equal(wq.numpy()[:N, :K], g["w_q"]); np.testing.assert_array_equal(we.numpy()[:N, :K // 32], g["w_e8"])
  off = DeviceBuffer.from_numpy(np.array([0, 256], np.int32))
  c = DeviceBuffer.empty((256, 256), np.uint16, zero=True)
  _lib.check(_lib.load().b200q_grouped_mxfp8_gemm(xq.ptr, xe.ptr, wq.ptr, we.ptr, off.ptr, 1, 256, 256, 128, c.ptr, None))
  y = moe.from_bf16_bits(c.numpy())[:M, :N]
  np.testing.assert_allclose(y, g["y"], rtol=2 ** -7, atol=1e-6)          # bf16: one unit in the last place (summation order)
  assert (y == g["y"]).mean() > 0.9


def test_moe_ffn_matches_composed_oracle():
  """route -> dispatch+quantise -> GEMM -> SwiGLU+quantise -> GEMM -> combine, against the same chain of oracle pieces."""
  from tinygrad_b200 import moe
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(2)
  T, D, F, E, k = 300, 256, 128, 8, 2
  wg, wu, wd = ((rng.standard_normal(s) * 0.05).astype(np.float32) for s in ((E, F, D), (E, F, D), (E, D, F)))
  x = moe.from_bf16_bits(moe.to_bf16_bits(rng.standard_normal((T, D)).astype(np.float32)))
  logits = rng.standard_normal((T, E)).astype(np.float32)
  for mode in (0, 1):
    m = moe.MxMoE(wg, wu, wd, k, mode)
    out = moe.from_bf16_bits(m(DeviceBuffer.from_numpy(moe.to_bf16_bits(x)), DeviceBuffer.from_numpy(logits), T).numpy())
    # oracle chain
    if mode == 0: w, topi, dest, off, m_l = mx.route(logits, k, E)
    else:
      _, sel = llm.pairwise_topk(logits[None], k); topi = sel[0]
      w = np.take_along_axis(llm.softmax(logits), topi.astype(np.int64), -1)
      _, _, _, off, m_l = mx.route(logits, k, E)
      dest = m.last_routing.dest_row.numpy()                          # placement checked in test_route_random_matches_oracle
    xd = mx.dispatch(x, dest, m_l, k)
    a_q, a_e8 = mx.quantize_mxfp8(xd)
    gu_q, gu_e8 = mx.quantize_mxfp8(np.concatenate([wg, wu], axis=1))
    h = mx.to_bf16(mx.grouped_mx_gemm(a_q, a_e8, gu_q, gu_e8, off))
    act = mx.to_bf16(llm.silu(h[:, :F]) * h[:, F:])
    act_q, act_e8 = mx.quantize_mxfp8(act)
    dn_q, dn_e8 = mx.quantize_mxfp8(wd)
    y = mx.to_bf16(mx.grouped_mx_gemm(act_q, act_e8, dn_q, dn_e8, off))
    ref = mx.to_bf16(mx.combine(y, dest, w))
    assert_close(out, ref, tol=1e-2, what=f"MoE FFN mode {mode}")


@pytest.mark.parametrize("per_slot", [False, True])
def test_expert_weights_call_matches_the_reference_semantics(per_slot):
  """`ExpertWeights.__call__(sel, x)` (tinygrad/llm/model.py:21-27): out[t, j] = x[t, j or 0] @ weight[sel[t, j]].T, here on MXFP8 operands:
  against the dequantised-operands product the reference tests its MX GEMM with (test/backend/test_asm_gemm.py:289-292)."""
  from tinygrad_b200 import moe
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(31)
  T, k, E, n_in, n_out = 37, 3, 6, 256, 512
  w = (rng.standard_normal((E, n_out, n_in)) * 0.05).astype(np.float32)
  sel = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
  sel[5] = [4, 4, 1]                                               # the same expert twice for one token is a legal selection
  x = moe.from_bf16_bits(moe.to_bf16_bits(rng.standard_normal((T, k if per_slot else 1, n_in)).astype(np.float32)))
  ew = moe.ExpertWeights(w)
  out = moe.from_bf16_bits(ew(DeviceBuffer.from_numpy(sel), DeviceBuffer.from_numpy(moe.to_bf16_bits(x))).numpy())
  assert out.shape == (T, k, n_out)
  w_q, w_e8 = mx.quantize_mxfp8(w)
  w_dq = mx.dequantize_mxfp8(w_q, w_e8)
  x_dq = mx.dequantize_mxfp8(*mx.quantize_mxfp8(x))
  ref = np.stack([[x_dq[t, j if per_slot else 0] @ w_dq[sel[t, j]].T for j in range(k)] for t in range(T)])
  assert_close(out, mx.to_bf16(ref), tol=1e-2, what="ExpertWeights(sel, x)")
  with pytest.raises(ValueError): moe.ExpertWeights(np.zeros((2, 100, 128), np.float32))


@pytest.mark.parametrize("dt", [np.float32, np.float16])
def test_fp8_linear_matches_reference_golden_and_oracle(golden, dt):
  """`FP8Linear` (extra/fp8/fp8_linear.py:43-63) through the tcgen05 GEMM with fp32 output: codes and factors bit-exact, outputs like the reference."""
  from tinygrad_b200 import fp8, _lib
  from tinygrad_b200.runtime import DeviceBuffer
  from oracle import fp8_linear as f8
  g = golden("fp8linear")
  for tag in "ab":
    x, w, bias = g[f"{tag}_x"], g[f"{tag}_w"], g[f"{tag}_bias"]
    q, f = fp8.quantize_to_fp8(DeviceBuffer.from_numpy(x), x.size, _lib.F32)
    np.testing.assert_array_equal(q.numpy().reshape(x.shape), g[f"{tag}_xq"])
    assert f.numpy().view(np.uint32)[0] == g[f"{tag}_xf"].view(np.uint32)
    lin = fp8.FP8Linear(w.shape[1], w.shape[0], w, bias)
    np.testing.assert_array_equal(lin.w_q.numpy().reshape(w.shape), g[f"{tag}_wq"])
    xd = x.astype(dt)
    y = lin(DeviceBuffer.from_numpy(xd)).numpy()
    assert y.dtype == dt and y.shape == (x.shape[0], w.shape[0])
    ref = g[f"{tag}_y"] if dt == np.float32 else f8.fp8_linear(xd.astype(np.float32), w, bias)
    assert_close(y, ref, tol=2e-3 if dt == np.float16 else 1e-5, what=f"FP8Linear {tag}")
  # a larger ragged batch against the oracle, no bias
  rng = np.random.default_rng(5)
  x, w = rng.standard_normal((3, 67, 384)).astype(np.float32), (rng.standard_normal((512, 384)) * 0.05).astype(np.float32)
  y = fp8.FP8Linear(384, 512, w)(DeviceBuffer.from_numpy(x)).numpy()
  assert y.shape == (3, 67, 512)
  assert_close(y, f8.fp8_linear(x, w), tol=1e-4, what="FP8Linear, 201 rows")
  with pytest.raises(ValueError): fp8.FP8Linear(100, 256, np.zeros((256, 100), np.float32))


def test_no_tensor_core_wait_ran_out():
  import ctypes
  from tinygrad_b200 import _lib
  st = ctypes.c_int()
  _lib.check(_lib.load().b200q_mx_status_read_clear(ctypes.byref(st)))
  assert st.value == 0
