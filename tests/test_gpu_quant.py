"""GPU parity: dequantisation (bit-exact), packing (lossless) and the fused GEMV, through the C ABI."""
import ctypes
import numpy as np
import pytest
from oracle import ggml_quant as gq, llm
from tinygrad_b200 import synth
from gpu_util import need_gpu, assert_close

pytestmark = pytest.mark.gpu
TAGS = {"q4_0": 2, "q8_0": 8, "q6_k": 14}


@pytest.fixture(scope="module", autouse=True)
def _gpu(): need_gpu()


@pytest.mark.parametrize("tag", list(TAGS))
def test_dequant_golden_bit_exact(golden, tag):
  from tinygrad_b200 import quant
  g = golden("dequant")
  raw, n = g[f"{tag}_raw"], g[f"{tag}_f32"].size
  np.testing.assert_array_equal(quant.dequantize(raw, n, TAGS[tag], np.float32).numpy().view(np.uint32), g[f"{tag}_f32"].reshape(-1).view(np.uint32))
  np.testing.assert_array_equal(quant.dequantize(raw, n, TAGS[tag], np.float16).numpy().view(np.uint16), g[f"{tag}_f16"].reshape(-1).view(np.uint16))


@pytest.mark.parametrize("tag", list(TAGS))
def test_dequant_random_bit_exact(tag):
  from tinygrad_b200 import quant
  typ = TAGS[tag]
  rng = np.random.default_rng(7)
  raw = synth.BLOCK_MAKERS[typ](64, 2048, rng)
  nby = synth.GGML_QUANT[typ][1]
  blocks = raw.reshape(-1, nby)
  sc = 208 if typ == 14 else 0     # every scale bit pattern that is finite, subnormals included
  pats = rng.integers(0, 0x7C00, len(blocks)).astype(np.uint16) | (rng.integers(0, 2, len(blocks)).astype(np.uint16) << 15)
  blocks[:, sc:sc + 2] = pats.view(np.uint8).reshape(-1, 2)
  n = 64 * 2048
  ref = gq.dequantize(raw, n, typ)
  np.testing.assert_array_equal(quant.dequantize(raw, n, typ, np.float32).numpy().view(np.uint32), ref.view(np.uint32))
  np.testing.assert_array_equal(quant.dequantize(raw, n, typ, np.float16).numpy().view(np.uint16), ref.astype(np.float16).view(np.uint16))


def test_dequant_empty_and_errors():
  from tinygrad_b200 import quant, _lib
  assert quant.dequantize(np.zeros(0, np.uint8), 0, 2).numpy().size == 0
  with pytest.raises(ValueError): quant.dequantize(np.zeros(18, np.uint8), 32, 5)
  with pytest.raises(_lib.B200QError): quant.dequantize(np.zeros(18, np.uint8), 31, 2)


@pytest.mark.parametrize("tag,n_out,n_in", [("q4_0", 64, 256), ("q4_0", 40, 96), ("q4_0", 16, 32), ("q8_0", 48, 384), ("q8_0", 17, 160),
                                             ("q6_k", 64, 512), ("q6_k", 40, 256), ("q6_k", 17, 1024)])
def test_repack_is_lossless(tag, n_out, n_in):
  from tinygrad_b200 import quant
  typ = TAGS[tag]
  raw = synth.BLOCK_MAKERS[typ](n_out, n_in, np.random.default_rng(n_out * 1000 + n_in))
  ref = gq.weight_matrix(raw, n_out, n_in, typ)
  pw = quant.repack(raw, n_out, n_in, typ)
  assert pw.buf.nbytes == -(-n_out // 16) * -(-n_in // 128) * {2: 1152, 8: 2176, 14: 1696}[typ]
  np.testing.assert_array_equal(pw.dequantize(np.float32).numpy().view(np.uint32), ref.view(np.uint32))
  np.testing.assert_array_equal(pw.dequantize(np.float16).numpy().view(np.uint16), ref.astype(np.float16).view(np.uint16))


def test_repack_interleaved_gate_up():
  from tinygrad_b200 import quant
  n_out, n_in = 24, 128
  g = synth.q4_0_blocks(n_out, n_in, np.random.default_rng(1)); u = synth.q4_0_blocks(n_out, n_in, np.random.default_rng(2))
  pw = quant.repack(g, n_out, n_in, 2, raw_up=u)
  got = pw.dequantize().numpy().reshape(-1, 2, 8, n_in)        # [tile][gate|up][8 rows]
  np.testing.assert_array_equal(got[:, 0].reshape(-1, n_in)[:n_out], gq.weight_matrix(g, n_out, n_in, 2))
  np.testing.assert_array_equal(got[:, 1].reshape(-1, n_in)[:n_out], gq.weight_matrix(u, n_out, n_in, 2))


def _run_linear(typ, n_out, n_in, x, **kw):
  from tinygrad_b200 import quant
  quant.GEMM_MIN_ROWS = 1 << 30          # these cases test the GEMV kernel, also for a few rows
  from tinygrad_b200.runtime import DeviceBuffer
  raw = synth.BLOCK_MAKERS[typ](n_out, n_in, np.random.default_rng(0))
  lin = quant.QuantLinear(n_in, n_out, typ, raw, **kw)
  return raw, lin(DeviceBuffer.from_numpy(x)).numpy()


def test_single_q4_0_linear_4096_fp16():
  """Config 1: Q4_0 [4096 x 4096], scales |N(0,0.02)|, x fp16 [1,4096] ~ N(0,1), seed 0."""
  rng = np.random.default_rng(0)
  raw = synth.q4_0_blocks(4096, 4096, rng)
  x = rng.standard_normal((1, 4096)).astype(np.float16)
  from tinygrad_b200 import quant
  from tinygrad_b200.runtime import DeviceBuffer
  y = quant.QuantLinear(4096, 4096, 2, raw)(DeviceBuffer.from_numpy(x)).numpy()
  assert y.dtype == np.float16 and y.shape == (1, 4096)
  w = gq.weight_matrix(raw, 4096, 4096, 2)
  assert_close(y, llm.linear_f16(x, w), what="fp16-product reference")
  assert_close(y, llm.linear(x.astype(np.float32), w), what="fp32 reference")


@pytest.mark.parametrize("tag,n_out,n_in,m", [("q4_0", 256, 1024, 1), ("q4_0", 40, 96, 3), ("q4_0", 16, 32, 1), ("q4_0", 4096, 14336, 1),
                                               ("q8_0", 512, 3584, 1), ("q8_0", 33, 160, 2), ("q4_0", 128, 128 * 9, 1),
                                               ("q6_k", 256, 1024, 1), ("q6_k", 33, 256, 3), ("q6_k", 4096, 4096, 1), ("q6_k", 1000, 14336, 2),
                                               ("q6_k", 48, 768, 5)])
def test_linear_fp32_matches_oracle(tag, n_out, n_in, m):
  typ = TAGS[tag]
  x = np.random.default_rng(3).standard_normal((m, n_in)).astype(np.float32)
  raw, y = _run_linear(typ, n_out, n_in, x)
  ref = llm.linear(x, gq.weight_matrix(raw, n_out, n_in, typ))
  assert y.dtype == np.float32
  assert_close(y, ref, tol=1e-2)
  # 15-bit activation quantisation with exact integer block sums: far inside the stated tolerance
  assert np.abs(y - ref).max() <= 5e-4 * np.abs(ref).max()


@pytest.mark.parametrize("tag", ["q4_0", "q8_0", "q6_k"])
def test_linear_golden_from_reference(golden, tag):
  from tinygrad_b200 import quant
  from tinygrad_b200.runtime import DeviceBuffer
  g = golden("linear")
  n_out, n_in = (int(v) for v in g[f"{tag}_shape"])
  lin = quant.QuantLinear(n_in, n_out, TAGS[tag], g[f"{tag}_raw"])
  assert_close(lin(DeviceBuffer.from_numpy(g[f"{tag}_x32"])).numpy(), g[f"{tag}_y32"], what="fp32 activations")
  assert_close(lin(DeviceBuffer.from_numpy(g[f"{tag}_x16"])).numpy(), g[f"{tag}_y16"], what="fp16 activations")


def test_linear_bias_and_empty_batch():
  bias = np.random.default_rng(4).standard_normal(48).astype(np.float16)
  x = np.random.default_rng(5).standard_normal((2, 256)).astype(np.float32)
  raw, y = _run_linear(8, 48, 256, x, bias=bias)
  assert_close(y, llm.linear(x, gq.weight_matrix(raw, 48, 256, 8), bias))
  _, y0 = _run_linear(2, 32, 128, np.zeros((0, 128), np.float32))
  assert y0.shape == (0, 32)


def test_fused_norm_residual_and_swiglu():
  from tinygrad_b200 import quant, _lib
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(6)
  dim, hid = 384, 1000
  x = rng.standard_normal(dim).astype(np.float32) * 3
  nw = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float16)
  g, u, d = (synth.q4_0_blocks(*s, rng) for s in ((hid, dim), (hid, dim), (dim, hid + 24)))
  wg, wu, wd = gq.weight_matrix(g, hid, dim, 2), gq.weight_matrix(u, hid, dim, 2), gq.weight_matrix(d, dim, hid + 24, 2)
  xn = llm.rmsnorm(x[None], nw, 1e-5)
  act_ref = (llm.silu(llm.linear(xn, wg)) * llm.linear(xn, wu))[0]
  pgu = quant.repack(g, hid, dim, 2, raw_up=u)
  dx, dnw, dact = DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(nw), DeviceBuffer.empty((hid + 24,), np.float32, zero=True)
  quant.gemv(pgu.buf.ptr, 2, hid, dim, dx, dact, norm_weight=dnw, norm_eps=1e-5, epilogue=_lib.EPI_SILU_MUL)
  act = dact.numpy()
  assert_close(act[:hid], act_ref, what="norm + gate/up + swiglu")
  assert (act[hid:] == 0).all()                                  # rows past n_out untouched
  act_full = np.concatenate([act_ref, np.zeros(24, np.float32)])
  pd = quant.repack(d, dim, hid + 24, 2)
  dres, dy = DeviceBuffer.from_numpy(x), DeviceBuffer.empty((dim,), np.float32)
  quant.gemv(pd.buf.ptr, 2, dim, hid + 24, dact, dres, residual=dres)   # in place on the residual stream
  assert_close(dres.numpy(), x + llm.linear(act_full[None], wd)[0], what="down + residual")


def test_q6_k_head_with_fused_norm_bias_and_residual():
  """The fused Q6_K GEMV in the role it has in K-quant files (the vocabulary head behind the output RMSNorm), plus bias / residual / fp16."""
  from tinygrad_b200 import quant
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(9)
  n_out, n_in = 1000, 2048
  raw = synth.q6_k_blocks(n_out, n_in, rng)
  w = gq.weight_matrix(raw, n_out, n_in, 14)
  x = rng.standard_normal(n_in).astype(np.float32) * 2
  nw = (1 + 0.1 * rng.standard_normal(n_in)).astype(np.float16)
  bias = rng.standard_normal(n_out).astype(np.float16)
  res = rng.standard_normal(n_out).astype(np.float32)
  pw = quant.repack(raw, n_out, n_in, 14)
  dy = DeviceBuffer.from_numpy(res.copy())
  quant.gemv(pw.buf.ptr, 14, n_out, n_in, DeviceBuffer.from_numpy(x), dy, norm_weight=DeviceBuffer.from_numpy(nw), norm_eps=1e-5,
             bias=DeviceBuffer.from_numpy(bias), residual=dy)
  ref = res + llm.linear(llm.rmsnorm(x[None], nw, 1e-5), w, bias)[0]
  assert_close(dy.numpy(), ref, what="norm + Q6_K linear + bias + residual")
  x16 = x.astype(np.float16)
  y16 = DeviceBuffer.empty((n_out,), np.float16)
  quant.gemv(pw.buf.ptr, 14, n_out, n_in, DeviceBuffer.from_numpy(x16), y16, x_dtype=quant.F16, y_dtype=quant.F16)
  assert_close(y16.numpy(), llm.linear(x16[None].astype(np.float32), w)[0], what="fp16 in / out")
  # what the format cannot do is refused, not approximated
  from tinygrad_b200 import _lib
  with pytest.raises(_lib.B200QError): quant.gemv(pw.buf.ptr, 14, n_out, n_in, DeviceBuffer.from_numpy(x), dy, epilogue=_lib.EPI_SILU_MUL)
  with pytest.raises(ValueError): quant.repack(synth.q6_k_blocks(16, 256, rng), 16, 128, 14)


def test_no_kernel_wait_ran_out():
  """The bounded mbarrier waits of the GEMV pipeline must never expire in normal operation."""
  from tinygrad_b200 import runtime
  assert runtime.device_status() == 0


@pytest.mark.parametrize("tag,m,n_out,n_in,x_dtype,bias", [("q4_0", 4, 64, 128, np.float32, False), ("q4_0", 37, 200, 96, np.float16, True),
                                                           ("q4_0", 130, 4096, 4096, np.float32, False), ("q8_0", 8, 512, 3584, np.float32, True),
                                                           ("q8_0", 32, 48, 160, np.float16, False), ("q4_0", 32, 14336, 4096, np.float32, False)])
def test_tensor_core_gemm_matches_fp16_operand_reference(tag, m, n_out, n_in, x_dtype, bias):
  """tcgen05 path (several activation rows).  fp16 activations: the operands are the activations and the materialised fp16
  weights, as in the reference's fp16 Linear.  fp32 activations: hi + lo halves of both operands, i.e. the fp32 activation times
  the unrounded dequantised weight, as in the reference's fused fp32 kernels."""
  from tinygrad_b200 import quant, _lib
  quant.GEMM_MIN_ROWS = 4
  from tinygrad_b200.runtime import DeviceBuffer
  typ = TAGS[tag]
  rng = np.random.default_rng(m * 7 + n_out)
  raw = synth.BLOCK_MAKERS[typ](n_out, n_in, rng)
  x = rng.standard_normal((m, n_in)).astype(x_dtype)
  b = rng.standard_normal(n_out).astype(np.float16) if bias else None
  lin = quant.QuantLinear(n_in, n_out, typ, raw, bias=b)
  y = lin(DeviceBuffer.from_numpy(x)).numpy()                     # the pipelined kernel (pre-split activations in a workspace)
  assert y.dtype == x_dtype and y.shape == (m, n_out)
  # the single-buffered kernel computes the same products; only the order of the fp32 additions inside the tensor core may differ
  y_old = DeviceBuffer.empty((m, n_out), x_dtype)
  dt = quant.F32 if x_dtype == np.float32 else quant.F16
  quant.qgemm(lin.weight.buf.ptr, typ, n_out, n_in, DeviceBuffer.from_numpy(x), y_old, m, x_dtype=dt, y_dtype=dt, bias=lin.bias)
  np.testing.assert_allclose(y.astype(np.float32), y_old.numpy().astype(np.float32), rtol=0, atol=(2e-3 if x_dtype == np.float16 else 2e-5) * max(1.0, float(np.abs(y).max())))
  ref32 = llm.linear(x.astype(np.float32), gq.weight_matrix(raw, n_out, n_in, typ), b)
  if x_dtype == np.float32:
    assert_close(y, ref32, tol=1e-2, what="tcgen05 GEMM vs fp32 reference")
    assert np.abs(y - ref32).max() <= 2e-5 * max(1.0, np.abs(ref32).max())       # only the accumulation order differs
  else:
    w16 = gq.weight_matrix(raw, n_out, n_in, typ).astype(np.float16).astype(np.float32)
    ref = x.astype(np.float32) @ w16.T + (b.astype(np.float32) if bias else 0.0)
    assert_close(y, ref, tol=4e-3, what="tcgen05 GEMM vs fp16-operand reference")
    # against the exact-weight product the difference is the fp16 rounding of the weight and of the fp16 result
    assert np.abs(y.astype(np.float32) - ref32).max() <= 4e-3 * max(1.0, np.abs(ref32).max())
  st = ctypes.c_int(); _lib.check(_lib.load().b200q_tc_status_read_clear(ctypes.byref(st)))
  assert st.value == 0


@pytest.mark.parametrize("kind,n_out,n_in,m", [("f16", 64, 2048, 1), ("f32", 100, 256, 3), ("bf16", 37, 512, 4), ("q6_k", 48, 1024, 2),
                                              ("f16", 8, 4096, 6)])
def test_dense_weight_linear(kind, n_out, n_in, m):
  """Linears whose weights stay unquantised (F16 / F32 / BF16 tensors): the dense GEMV against the oracle's linear.  Q6_K through the same
  front door takes the fused kernel (exact block values, activations quantised to 15 bits) and, as `DenseWeight`, the fp16 cast."""
  from tinygrad_b200 import quant, moe
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(11)
  if kind == "q6_k":
    raw, typ = synth.q6_k_blocks(n_out, n_in, rng), 14
    w = gq.dequantize(raw, n_out * n_in, 14).reshape(n_out, n_in)
    dw = quant.DenseWeight(raw, n_out, n_in, 14)                 # the reference's own treatment: every tensor cast to fp16 (model.py:376)
    x = rng.standard_normal((m, n_in)).astype(np.float32)
    y = DeviceBuffer.empty((m, n_out), np.float32)
    quant.gemv_dense(dw.buf, dw.dtype, n_out, n_in, DeviceBuffer.from_numpy(x), y, m=m)
    ref16 = llm.linear(x, w.astype(np.float16).astype(np.float32))
    assert np.abs(y.numpy() - ref16).max() <= 1e-5 * max(1.0, np.abs(ref16).max())
  else:
    w = (rng.standard_normal((n_out, n_in)) * 0.05).astype(np.float32)
    if kind == "f16": raw, typ, w = w.astype(np.float16), quant.GGML_F16, w.astype(np.float16).astype(np.float32)
    elif kind == "bf16": raw, typ = moe.to_bf16_bits(w), quant.GGML_BF16; w = moe.from_bf16_bits(raw)
    else: raw, typ = w, quant.GGML_F32
  bias = rng.standard_normal(n_out).astype(np.float16)
  lin = quant.QuantLinear(n_in, n_out, typ, raw, bias=bias)
  for dt in (np.float32, np.float16):
    x = rng.standard_normal((m, n_in)).astype(dt)
    y = lin(DeviceBuffer.from_numpy(x)).numpy()
    assert y.dtype == dt and y.shape == (m, n_out)
    ref = llm.linear(x.astype(np.float32), w, bias)
    assert_close(y, ref, tol=1e-2)
    bound = 2e-3 if dt == np.float16 else (5e-4 if kind == "q6_k" else 1e-5)
    assert np.abs(y.astype(np.float32) - ref).max() <= bound * max(1.0, np.abs(ref).max())


def test_dense_fused_norm_and_residual():
  from tinygrad_b200 import quant, _lib
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(12)
  n_out, n_in = 72, 768
  w = (rng.standard_normal((n_out, n_in)) * 0.05).astype(np.float16)
  x = rng.standard_normal(n_in).astype(np.float32) * 2
  nw = (1 + 0.1 * rng.standard_normal(n_in)).astype(np.float16)
  res = rng.standard_normal(n_out).astype(np.float32)
  dy = DeviceBuffer.from_numpy(res)
  quant.gemv_dense(DeviceBuffer.from_numpy(w), _lib.F16, n_out, n_in, DeviceBuffer.from_numpy(x), dy, norm_weight=DeviceBuffer.from_numpy(nw),
                   norm_eps=1e-5, residual=dy)
  ref = res + llm.linear(llm.rmsnorm(x[None], nw, 1e-5), w.astype(np.float32))[0]
  assert np.abs(dy.numpy() - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("tag,n_out,n_in,m", [("q4_0", 4096, 4096, 1), ("q8_0", 200, 3584, 3), ("q4_0", 48, 14336 + 2048, 2)])
def test_in_graph_kernels_match_oracle(tag, n_out, n_in, m):
  """The entry kernels tinygrad's runtime launches (tinygrad_b200/tg_op.py), run here with the same launch geometry through the library."""
  from tinygrad_b200 import _lib, quant, tg_op
  from tinygrad_b200.runtime import DeviceBuffer
  typ = TAGS[tag]
  rng = np.random.default_rng(n_out)
  raw, x = synth.BLOCK_MAKERS[typ](n_out, n_in, rng), rng.standard_normal((m, n_in)).astype(np.float32)
  w = quant.repack(raw, n_out, n_in, typ)
  y = DeviceBuffer.from_numpy(np.full((m, n_out), np.nan, np.float32))
  meta = DeviceBuffer.from_numpy(np.array([n_out, n_in, m], np.int32))
  (gx, gy, _), _ = tg_op.launch_dims(n_out, m)
  assert gx == -(-(-(-n_out // 16)) // 8) and gy == m
  _lib.check(_lib.load().b200q_tg_gemv(typ, y.ptr, DeviceBuffer.from_numpy(x).ptr, w.buf.ptr, meta.ptr, n_out, m, None))
  ref = llm.linear(x, gq.weight_matrix(raw, n_out, n_in, typ))
  assert_close(y.numpy(), ref, tol=1e-2)
  assert np.abs(y.numpy() - ref).max() <= 5e-4 * np.abs(ref).max()


@pytest.mark.parametrize("tag,typ", [("q4_1", 3), ("q5_0", 6), ("q5_1", 7), ("q4_k", 12), ("q5_k", 13)])
def test_other_block_formats_bit_exact(golden, tag, typ):
  """Q4_1, Q5_0, Q5_1, Q4_K, Q5_K dequantisation: the reference's own output (golden) and random blocks against the oracle, fp32 and fp16."""
  from tinygrad_b200 import quant
  g = golden("dequant2")
  raw, n = g[f"{tag}_raw"], g[f"{tag}_f32"].size
  np.testing.assert_array_equal(quant.dequantize(raw, n, typ, np.float32).numpy().view(np.uint32), g[f"{tag}_f32"].reshape(-1).view(np.uint32))
  np.testing.assert_array_equal(quant.dequantize(raw, n, typ, np.float16).numpy().view(np.uint16), g[f"{tag}_f16"].reshape(-1).view(np.uint16))
  nel, _ = synth.GGML_SIZES[typ]
  blocks = synth.random_blocks(typ, 64, 8 * nel, np.random.default_rng(typ + 1))
  ref = gq.dequantize(blocks, 64 * 8 * nel, typ)
  np.testing.assert_array_equal(quant.dequantize(blocks, ref.size, typ, np.float32).numpy().view(np.uint32), ref.view(np.uint32))
  np.testing.assert_array_equal(quant.dequantize(blocks, ref.size, typ, np.float16).numpy().view(np.uint16), ref.astype(np.float16).view(np.uint16))
