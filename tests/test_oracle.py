"""The oracle against the reference: golden vectors made by running tinygrad
itself (tests/golden/make_golden.py), the reference's known-answer vectors, and
gguf-py (the library tinygrad's own tests compare against)."""
import numpy as np
import pytest
from oracle import ggml_quant as gq, llm, mxfp8
from tinygrad_b200 import synth

TAGS = {"q4_0": 2, "q8_0": 8, "q6_k": 14}


@pytest.mark.parametrize("tag", list(TAGS))
def test_dequant_matches_reference_bit_exact(golden, tag):
  g = golden("dequant")
  raw, typ = g[f"{tag}_raw"], TAGS[tag]
  n = g[f"{tag}_f32"].size
  out = gq.dequantize(raw, n, typ)
  np.testing.assert_array_equal(out.view(np.uint32), g[f"{tag}_f32"].reshape(-1).view(np.uint32))
  np.testing.assert_array_equal(gq.dequantize_f16(raw, n, typ).view(np.uint16), g[f"{tag}_f16"].reshape(-1).view(np.uint16))


def test_dequant_q8_0_known_answer():
  # test/unit/test_gguf.py:36-40
  block = np.frombuffer(np.float16(2.0).tobytes() + np.arange(1, 33, dtype=np.int8).tobytes(), dtype=np.uint8)
  np.testing.assert_array_equal(gq.dequantize(block, 32, 8), np.arange(1, 33, dtype=np.float32) * 2.0)


@pytest.mark.parametrize("tag", list(TAGS))
def test_dequant_matches_gguf_py(tag):
  # test/unit/test_gguf.py:157-170: random blocks, exact equality with gguf.dequantize
  gguf = pytest.importorskip("gguf")
  typ = TAGS[tag]
  raw = synth.BLOCK_MAKERS[typ](8, 512, np.random.default_rng(5))
  qt = gguf.GGMLQuantizationType(typ)
  ref = gguf.dequantize(raw.reshape(-1, synth.GGML_QUANT[typ][1]), qt).reshape(-1)
  np.testing.assert_array_equal(gq.dequantize(raw, 8 * 512, typ), ref.astype(np.float32))


@pytest.mark.parametrize("tag", list(TAGS))
def test_linear_matches_reference(golden, tag):
  g = golden("linear")
  n_out, n_in = g[f"{tag}_shape"]
  w = gq.weight_matrix(g[f"{tag}_raw"], n_out, n_in, TAGS[tag])
  y32 = llm.linear(g[f"{tag}_x32"], w)
  np.testing.assert_allclose(y32, g[f"{tag}_y32"], rtol=1e-5, atol=1e-5)
  y16 = llm.linear_f16(g[f"{tag}_x16"], w)
  np.testing.assert_allclose(y16.astype(np.float32), g[f"{tag}_y16"].astype(np.float32), rtol=2e-3, atol=2e-3)


def test_pairwise_topk_matches_reference(golden):
  g = golden("moe")
  v, s = llm.pairwise_topk(g["topk_x"], 3)
  np.testing.assert_array_equal(s, g["topk_sel"])
  np.testing.assert_array_equal(v, g["topk_v"])


@pytest.mark.parametrize("tag", ["softmax", "softmax_norm", "sigmoid_norm", "softmax_weight"])
def test_moe_ffn_matches_reference(golden, tag):
  g = golden("moe")
  dim, hidden, E, k, gating, norm = (int(v) for v in g[f"{tag}_cfg"])
  cfg = llm.Config(num_blocks=1, dim=dim, hidden_dim=hidden, n_heads=2, n_kv_heads=2, norm_eps=1e-5, vocab_size=32, head_dim=16,
                   rope_theta=10000.0, rope_dim=16, max_context=16, num_experts=E, num_experts_per_tok=k, norm_topk_prob=bool(norm),
                   expert_gating_func=gating, routed_scaling_factor=float(g[f"{tag}_scale"]))
  w = {"blk.0.ffn_gate_exps.weight": g[f"{tag}_gate"], "blk.0.ffn_up_exps.weight": g[f"{tag}_up"],
       "blk.0.ffn_down_exps.weight": g[f"{tag}_down"], "blk.0.ffn_gate_inp.weight": g[f"{tag}_router"]}
  m = llm.Transformer.__new__(llm.Transformer); m.cfg, m.w = cfg, w
  np.testing.assert_allclose(m._feed_forward(0, g[f"{tag}_h"]), g[f"{tag}_y"], rtol=1e-4, atol=1e-5)


def test_e4m3_conversion_matches_reference(golden):
  g = golden("mxfp8")
  np.testing.assert_array_equal(mxfp8.float_to_e4m3(g["e4m3_in"]), g["e4m3_code"])
  t = mxfp8.e4m3_table()
  np.testing.assert_array_equal(np.nan_to_num(t, nan=7777.0), np.nan_to_num(g["e4m3_table"], nan=7777.0))


def test_quantize_mxfp8_matches_reference(golden):
  g = golden("mxfp8")
  q, e8 = mxfp8.quantize_mxfp8(g["x"])
  np.testing.assert_array_equal(e8, g["e8"])
  np.testing.assert_array_equal(q, g["q"])
  np.testing.assert_array_equal(mxfp8.dequantize_mxfp8(q, e8), g["deq"])


def test_route_matches_reference(golden):
  g = golden("mxfp8")
  w, topi, dest, off, m_l = mxfp8.route(g["route_logits"], 2, 8)
  np.testing.assert_allclose(w, g["route_weights"][0], rtol=1e-6)
  np.testing.assert_array_equal(dest, g["route_dest_row"][0])
  np.testing.assert_array_equal(off, g["route_off"][0])
  assert m_l == int(g["route_m_l"])


def _llm_from_golden(g):
  nb, dim, hid, nh, nkv, vocab, hd, rd, ctx, typ, kv_half, bias, seed = (int(v) for v in g["meta"])
  cfg = llm.Config(num_blocks=nb, dim=dim, hidden_dim=hid, n_heads=nh, n_kv_heads=nkv, norm_eps=float(g["norm_eps"]), vocab_size=vocab,
                   head_dim=hd, rope_theta=float(g["rope_theta"]), rope_dim=rd, max_context=ctx, qkv_bias=bool(bias),
                   kv_dtype="float16" if kv_half else "float32")
  w = {}
  for key in g.files:
    if not key.startswith("w:"): continue
    name, a = key[2:], g[key]
    if a.dtype == np.uint8:
      n_out = {n: o for n, o, i in synth.linear_names(cfg)}[name[:-len(".weight")]]
      n_in = {n: i for n, o, i in synth.linear_names(cfg)}[name[:-len(".weight")]]
      a = gq.weight_matrix(a, n_out, n_in, typ)
    w[name] = a
  return cfg, w


@pytest.mark.parametrize("name", ["llm_small_kv32", "llm_q8_bias_kv32", "llm_wide_kv32"])
def test_greedy_token_stream_matches_reference(golden, name):
  g = golden(name)
  cfg, w = _llm_from_golden(g)
  toks = llm.Transformer(cfg, w).generate([int(t) for t in g["prompt"]], len(g["tokens"]))
  assert toks == [int(t) for t in g["tokens"]]


@pytest.mark.parametrize("tag", list(TAGS))
def test_c_dequant_equals_numpy_restatement(golden, tag):
  """The C restatement (used where the numpy one is too slow: full-size matrices, the timed CPU baseline) gives the same
  bits as the numpy restatement, on the reference's golden blocks and on random ones."""
  from oracle import cpu_gemv
  typ, g = TAGS[tag], golden("dequant")
  raw, n = g[f"{tag}_raw"], g[f"{tag}_f32"].size
  np.testing.assert_array_equal(cpu_gemv.dequantize(raw, n, typ).view(np.uint32), g[f"{tag}_f32"].reshape(-1).view(np.uint32))
  raw = synth.BLOCK_MAKERS[typ](16, 1024, np.random.default_rng(9))
  np.testing.assert_array_equal(cpu_gemv.dequantize(raw, 16 * 1024, typ).view(np.uint32), gq.dequantize(raw, 16 * 1024, typ).view(np.uint32))


@pytest.mark.parametrize("tag", list(TAGS))
def test_c_gemv_matches_linear(golden, tag):
  """The timed CPU baseline (oracle/qgemv_cpu.c) against `Linear` as the reference computed it (golden) and against the
  numpy restatement on a larger random case."""
  from oracle import cpu_gemv
  typ, g = TAGS[tag], golden("linear")
  n_out, n_in = (int(v) for v in g[f"{tag}_shape"])
  for row, want in zip(g[f"{tag}_x32"], g[f"{tag}_y32"]):
    np.testing.assert_allclose(cpu_gemv.qgemv(typ, g[f"{tag}_raw"], row, n_out, n_in), want, rtol=1e-5, atol=1e-5)
  rng = np.random.default_rng(4)
  raw, x = synth.BLOCK_MAKERS[typ](64, 2048, rng), rng.standard_normal(2048).astype(np.float32)
  ref = llm.linear(x[None], gq.weight_matrix(raw, 64, 2048, typ))[0]
  np.testing.assert_allclose(cpu_gemv.qgemv(typ, raw, x, 64, 2048), ref, rtol=1e-4, atol=1e-4 * float(np.abs(ref).max()))


def test_mxfp8_matmul_matches_reference(golden):
  """The reference's own runnable MXFP8 contraction (matmul_mx, examples/mlperf/models/gpt_oss.py:64-83) pins the oracle's
  quantise -> dequantise -> matmul chain and the weight quantiser."""
  g = golden("mxgemm")
  w_q, w_e8 = mxfp8.quantize_mxfp8(g["w"])
  np.testing.assert_array_equal(w_q, g["w_q"]); np.testing.assert_array_equal(w_e8, g["w_e8"])
  x_q, x_e8 = mxfp8.quantize_mxfp8(g["x_bf16"])
  y = mxfp8.to_bf16(mxfp8.mxfp8_matmul(x_q, x_e8, w_q, w_e8))
  # bf16 output: at most one unit in the last place apart (fp32 summation order), most entries identical
  np.testing.assert_allclose(y, g["y"], rtol=2 ** -7, atol=1e-6)
  assert (y == g["y"]).mean() > 0.9


@pytest.mark.parametrize("tag", ["softplus_bias", "softmax_bias_norm", "sigmoid_shared", "softmax_shared_plain"])
def test_moe_ffn_gating_paths_match_reference(golden, tag):
  """sqrt(softplus) scores, a selection bias, scaling factor, shared expert with and without its gate (tinygrad/llm/model.py:110-134)."""
  g = golden("moe2")
  dim, hidden, E, k, gating, norm = (int(v) for v in g[f"{tag}_cfg"])
  cfg = llm.Config(num_blocks=1, dim=dim, hidden_dim=hidden, n_heads=2, n_kv_heads=2, norm_eps=1e-5, vocab_size=32, head_dim=16,
                   rope_theta=10000.0, rope_dim=16, max_context=16, num_experts=E, num_experts_per_tok=k, norm_topk_prob=bool(norm),
                   expert_gating_func=gating, routed_scaling_factor=float(g[f"{tag}_scale"]))
  names = {"gate": "ffn_gate_exps.weight", "up": "ffn_up_exps.weight", "down": "ffn_down_exps.weight", "router": "ffn_gate_inp.weight",
           "bias": "exp_probs_b.bias", "sh_gate": "ffn_gate_shexp.weight", "sh_up": "ffn_up_shexp.weight", "sh_down": "ffn_down_shexp.weight",
           "sh_inp": "ffn_gate_inp_shexp.weight"}
  w = {"blk.0." + full: g[f"{tag}_{short}"] for short, full in names.items() if f"{tag}_{short}" in g.files}
  m = llm.Transformer.__new__(llm.Transformer); m.cfg, m.w = cfg, w
  np.testing.assert_allclose(m._feed_forward(0, g[f"{tag}_h"]), g[f"{tag}_y"], rtol=1e-4, atol=1e-5)


TAGS2 = {"q4_1": 3, "q5_0": 6, "q5_1": 7, "q4_k": 12, "q5_k": 13}


@pytest.mark.parametrize("tag", list(TAGS2))
def test_other_block_formats_match_reference_and_gguf_py(golden, tag):
  """Q4_1, Q5_0, Q5_1, Q4_K, Q5_K (tinygrad/llm/gguf.py:47-67): the numpy and the C restatement against the reference's own output,
  bit for bit, and against gguf-py on random blocks as the reference's tests do (test/unit/test_gguf.py:50-62)."""
  from oracle import cpu_gemv
  typ, g = TAGS2[tag], golden("dequant2")
  raw, n = g[f"{tag}_raw"], g[f"{tag}_f32"].size
  want = g[f"{tag}_f32"].reshape(-1).view(np.uint32)
  np.testing.assert_array_equal(gq.dequantize(raw, n, typ).view(np.uint32), want)
  np.testing.assert_array_equal(cpu_gemv.dequantize(raw, n, typ).view(np.uint32), want)
  np.testing.assert_array_equal(gq.dequantize_f16(raw, n, typ).view(np.uint16), g[f"{tag}_f16"].reshape(-1).view(np.uint16))
  gguf = pytest.importorskip("gguf")
  nel, nby = synth.GGML_SIZES[typ]
  blocks = synth.random_blocks(typ, 16, 2 * nel, np.random.default_rng(typ))
  ref = gguf.dequantize(blocks.reshape(-1, nby), gguf.GGMLQuantizationType(typ)).reshape(-1).astype(np.float32)
  np.testing.assert_array_equal(gq.dequantize(blocks, 32 * nel, typ), ref)
  np.testing.assert_array_equal(cpu_gemv.dequantize(blocks, 32 * nel, typ), ref)


def test_fp8_linear_matches_the_reference(golden):
  """`quantize_to_fp8` and the forward of `FP8Linear` (extra/fp8/fp8_linear.py:4-16,43-63): codes and factors bit-exact, outputs to fp32 rounding."""
  from oracle import fp8_linear as f8
  g = golden("fp8linear")
  for tag in "ab":
    for nm in ("x", "w"):
      q, f = f8.quantize_to_fp8(g[f"{tag}_{nm}"])
      np.testing.assert_array_equal(q, g[f"{tag}_{nm}q"])
      assert f.view(np.uint32) == g[f"{tag}_{nm}f"].view(np.uint32)
    y = f8.fp8_linear(g[f"{tag}_x"], g[f"{tag}_w"], g[f"{tag}_bias"])
    np.testing.assert_allclose(y, g[f"{tag}_y"], rtol=0, atol=2e-6 * np.abs(g[f"{tag}_y"]).max())      # the sum order is free
