"""GPU parity of prompt processing: batched causal attention with cache append, the GEMM epilogues it uses, and the
whole prefill path against token-by-token steps and the numpy oracle."""
import numpy as np
import pytest
from oracle import ggml_quant as gq, llm
from tinygrad_b200 import synth
from gpu_util import need_gpu, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _gpu(): need_gpu()


@pytest.mark.parametrize("kv_dtype,n_heads,n_kv,hd,rope_dim,start,T", [
  (np.float16, 8, 2, 128, 128, 0, 70), (np.float16, 4, 4, 64, 64, 37, 130), (np.float32, 4, 2, 16, 16, 5, 9), (np.float16, 6, 2, 32, 16, 64, 64),
  (np.float16, 32, 8, 128, 128, 300, 1), (np.float32, 2, 1, 128, 64, 0, 200)])
def test_prefill_attention_matches_oracle(kv_dtype, n_heads, n_kv, hd, rope_dim, start, T):
  from tinygrad_b200 import _lib
  from tinygrad_b200._lib import check, F16, F32
  from tinygrad_b200.runtime import DeviceBuffer
  from tinygrad_b200.model import precompute_freqs_cis
  rng = np.random.default_rng(hd + T)
  ctx = start + T + 3
  fc = precompute_freqs_cis(rope_dim, ctx, 10000.0)
  qkv = rng.standard_normal((T, (n_heads + 2 * n_kv) * hd)).astype(np.float32)
  k_old, v_old = (rng.standard_normal((n_kv, ctx, hd)).astype(kv_dtype) for _ in range(2))
  k_old[:, start:], v_old[:, start:] = 0, 0
  dk, dv = DeviceBuffer.from_numpy(k_old), DeviceBuffer.from_numpy(v_old)
  q16, out = DeviceBuffer.empty((T, n_heads * hd), np.float32), DeviceBuffer.empty((T, n_heads * hd), np.float16)
  dqkv, dfc = DeviceBuffer.from_numpy(qkv), DeviceBuffer.from_numpy(fc)
  check(_lib.load().b200q_attn_prefill(dqkv.ptr, dk.ptr, dv.ptr, F16 if kv_dtype == np.float16 else F32, dfc.ptr, start, T, n_heads, n_kv, hd,
                                       rope_dim, ctx, q16.ptr, out.ptr, F16, None))
  # oracle: model.py:167-198 on the same projections
  q = qkv[:, :n_heads * hd].reshape(1, T, n_heads, hd).transpose(0, 2, 1, 3)
  k = qkv[:, n_heads * hd:(n_heads + n_kv) * hd].reshape(1, T, n_kv, hd).transpose(0, 2, 1, 3)
  v = qkv[:, (n_heads + n_kv) * hd:].reshape(1, T, n_kv, hd).transpose(0, 2, 1, 3)
  f = fc[start:start + T]
  q = np.concatenate([llm.apply_rope(q[..., :rope_dim], f), q[..., rope_dim:]], -1)
  k = np.concatenate([llm.apply_rope(k[..., :rope_dim], f), k[..., rope_dim:]], -1)
  kc, vc = k_old.copy(), v_old.copy()
  kc[:, start:start + T], vc[:, start:start + T] = k[0].astype(kv_dtype), v[0].astype(kv_dtype)
  np.testing.assert_array_equal(dv.numpy(), vc)                       # v rows are stored as cast
  assert_close(dk.numpy().astype(np.float32), kc.astype(np.float32), tol=2e-3, what="k cache")
  rep = n_heads // n_kv
  kk, vv = np.repeat(kc[None, :, :start + T].astype(np.float32), rep, 1), np.repeat(vc[None, :, :start + T].astype(np.float32), rep, 1)
  qk = (q.astype(np.float32) @ kk.transpose(0, 1, 3, 2)) / np.float32(np.sqrt(hd))
  qk = qk + np.triu(np.full((T, start + T), -np.inf, dtype=np.float32), start + 1)
  ref = (llm.softmax(qk) @ vv).transpose(0, 2, 1, 3).reshape(T, -1)
  assert_close(out.numpy().astype(np.float32), ref, tol=2e-3, what="attention")


def test_gemm_epilogues_residual_and_swiglu():
  from tinygrad_b200 import quant, _lib
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(3)
  m, dim, hid = 150, 256, 392
  g, u, d = synth.q4_0_blocks(hid, dim, rng), synth.q4_0_blocks(hid, dim, rng), synth.q8_0_blocks(dim, hid + 24, rng)
  wg, wu = (gq.weight_matrix(r, hid, dim, 2).astype(np.float16).astype(np.float32) for r in (g, u))
  wd = gq.weight_matrix(d, dim, hid + 24, 8).astype(np.float16).astype(np.float32)
  x = rng.standard_normal((m, dim)).astype(np.float16)
  pgu = quant.repack(g, hid, dim, 2, raw_up=u)
  act = DeviceBuffer.empty((m, hid), np.float16)
  dx = DeviceBuffer.from_numpy(x)
  quant.qgemm(pgu.buf.ptr, 2, 2 * hid, dim, dx, act, m, x_dtype=_lib.F16, y_dtype=_lib.F16, epilogue=_lib.EPI_SILU_MUL)
  xf = x.astype(np.float32)
  ref_act = llm.silu(xf @ wg.T) * (xf @ wu.T)
  assert_close(act.numpy().astype(np.float32), ref_act, tol=4e-3, what="swiglu epilogue")
  a16 = np.concatenate([act.numpy(), np.zeros((m, 24), np.float16)], axis=1)
  res = rng.standard_normal((m, dim)).astype(np.float32)
  y = DeviceBuffer.from_numpy(res)
  pd, da16 = quant.repack(d, dim, hid + 24, 8), DeviceBuffer.from_numpy(a16)
  quant.qgemm(pd.buf.ptr, 8, dim, hid + 24, da16, y, m, x_dtype=_lib.F16, y_dtype=_lib.F32, residual=y)
  ref_y = res + a16.astype(np.float32) @ wd.T
  assert np.abs(y.numpy() - ref_y).max() <= 2e-4 * max(1.0, np.abs(ref_y).max())


@pytest.mark.parametrize("typ,kv,hd,chunk", [(2, "float16", 128, 512), (8, "float16", 64, 32), (2, "float32", 64, 50)])
def test_prefill_path_matches_steps_and_oracle(typ, kv, hd, chunk):
  """The same prompt through the GEMM prefill (several chunks, so start_pos > 0 inside it) and through one-token steps:
  logits within the end-to-end tolerance of the oracle, identical greedy continuation on both paths, and the cache prefix is
  reused by a following call."""
  from tinygrad_b200.model import Transformer, TransformerConfig
  kw = dict(num_blocks=3, dim=512, hidden_dim=1408, n_heads=512 // hd, n_kv_heads=2, norm_eps=1e-5, vocab_size=2000, head_dim=hd, rope_theta=500000.0,
            rope_dim=hd, max_context=256, qkv_bias=(typ == 8), kv_dtype=kv)
  cfg = TransformerConfig(**kw)
  sd = synth.dense_model_raw(cfg, typ, seed=13, embd_std=0.3, scale_std=0.02 if typ == 2 else 0.0015)
  shapes = {n: (o, i) for n, o, i in synth.linear_names(cfg)}
  w = {k: (gq.weight_matrix(v, *shapes[k[:-len(".weight")]], typ) if v.dtype == np.uint8 else v) for k, v in sd.items()}
  prompt = [int(t) for t in np.random.default_rng(2).integers(0, 2000, 150)]
  want, want_logits = llm.Transformer(llm.Config(**kw), w).generate(prompt, 12, keep_logits=True)
  fast = Transformer(cfg, sd, ggml_type=typ, prefill_rows=16, prefill_chunk=chunk)
  slow = Transformer(cfg, sd, ggml_type=typ, prefill_rows=0)
  got_fast, got_slow = [], []
  gf, gs = fast.generate(list(prompt)), slow.generate(list(prompt))
  for i in range(12):
    got_fast.append(next(gf)); got_slow.append(next(gs))
    # (the one-token path is held to the oracle by test_gpu_model; position 10 of this seed amplifies its 15-bit activation
    # quantisation past 3e-2, which is why the two device paths are not compared with each other here)
    assert_close(fast.read_logits(), want_logits[i], tol=3e-2, what=f"prefill-path logits at step {i}")
  assert got_slow == want
  assert got_fast == want
  again = []
  for tok in fast.generate(prompt + got_fast[:4] + [7, 8, 9] * 10):    # 150 + 4 cached, 30 new tokens -> a second prefill at start_pos > 0
    again.append(tok)
    if len(again) == 4: break
  ref_again = []
  for tok in slow.generate(prompt + got_fast[:4] + [7, 8, 9] * 10):
    ref_again.append(tok)
    if len(ref_again) == 4: break
  assert again == ref_again


class _MxOracle(llm.Transformer):
  """The oracle Transformer with the expert FFN of the MXFP8 path: bf16 activations, E4M3 + E8M0 operands on both sides of both
  expert GEMMs, bf16 results (the chain tests/test_gpu_moe.py checks piece by piece), routing as tinygrad/llm/model.py:110-124."""
  def _feed_forward(self, i, x):
    from oracle import mxfp8 as mx
    c = self.cfg
    B, T, D = x.shape
    xr = x.reshape(T, D).astype(np.float32)
    logits = llm.linear(xr, self.w[f"blk.{i}.ffn_gate_inp.weight"].astype(np.float32))
    sel, probs = llm.moe_gate(logits, c.expert_gating_func, c.norm_topk_prob, c.num_experts_per_tok, c.routed_scaling_factor,
                              self.w.get(f"blk.{i}.exp_probs_b.bias"))
    xa = mx.dequantize_mxfp8(*mx.quantize_mxfp8(mx.to_bf16(xr)))
    wg, wu, wd = (self.w[f"blk.{i}.ffn_{n}_exps.weight"] for n in ("gate", "up", "down"))
    if not hasattr(self, "_deq"): self._deq = {}
    if i not in self._deq:
      self._deq[i] = (mx.dequantize_mxfp8(*mx.quantize_mxfp8(np.concatenate([wg, wu], axis=1))), mx.dequantize_mxfp8(*mx.quantize_mxfp8(wd)))
    gu, dn = self._deq[i]
    F = wg.shape[1]
    out = np.zeros((T, D), np.float32)
    for t in range(T):
      acc = np.zeros(D, np.float32)
      for j in range(c.num_experts_per_tok):
        e = int(sel[t, j])
        h = mx.to_bf16(gu[e] @ xa[t])
        act = mx.to_bf16(llm.silu(h[:F]) * h[F:])
        aq = mx.dequantize_mxfp8(*mx.quantize_mxfp8(act[None]))[0]
        acc += probs[t, j] * mx.to_bf16(dn[e] @ aq)
      out[t] = mx.to_bf16(acc)
    return out.reshape(B, T, D) + self._shared_expert(i, x)


@pytest.mark.parametrize("variant", ["softmax", "softmax_norm", "sigmoid_norm_scaled_shared_gate", "sqrt_softplus_bias_shared"])
def test_moe_transformer_matches_mx_oracle(variant):
  """A routed-experts model (MXFP8 expert GEMMs inside the Transformer): prompt through the row path, then one-token steps; the gating
  functions, selection bias, scaling factor and shared expert of tinygrad/llm/model.py:110-134."""
  from tinygrad_b200.model import Transformer, TransformerConfig
  from tinygrad_b200 import moe
  extra = {"softmax": dict(), "softmax_norm": dict(norm_topk_prob=True),
           "sigmoid_norm_scaled_shared_gate": dict(expert_gating_func="sigmoid", norm_topk_prob=True, routed_scaling_factor=2.0, shared_expert_dim=128),
           "sqrt_softplus_bias_shared": dict(expert_gating_func="sqrt_softplus", expert_bias=True, shared_expert_dim=96, shared_expert_gate=False)}[variant]
  kw = dict(num_blocks=2, dim=256, hidden_dim=128, n_heads=4, n_kv_heads=2, norm_eps=1e-5, vocab_size=500, head_dim=64, rope_theta=10000.0, rope_dim=64,
            max_context=96, num_experts=8, num_experts_per_tok=2, **extra)
  cfg = TransformerConfig(**kw)
  sd = {k: v for k, v in synth.dense_model_raw(cfg, 8, seed=17, embd_std=0.3, scale_std=0.0015).items() if ".ffn_gate." not in k and ".ffn_up." not in k
        and ".ffn_down." not in k}
  rng = np.random.default_rng(5)
  for i in range(cfg.num_blocks):
    sd[f"blk.{i}.ffn_gate_inp.weight"] = (rng.standard_normal((8, 256)) * 0.1).astype(np.float32)
    for n, shape in (("gate", (8, 128, 256)), ("up", (8, 128, 256)), ("down", (8, 256, 128))):
      sd[f"blk.{i}.ffn_{n}_exps.weight"] = (rng.standard_normal(shape) * 0.08).astype(np.float32)
    if cfg.expert_bias: sd[f"blk.{i}.exp_probs_b.bias"] = (rng.standard_normal(8) * 0.3).astype(np.float32)
  shapes = {n: (o, i) for n, o, i in synth.linear_names(cfg)}
  sh = cfg.shared_expert_dim
  for i in range(cfg.num_blocks if sh else 0):       # the shared expert: Q8_0 blocks like the attention Linears
    for n, (o, ii) in (("ffn_gate_shexp", (sh, 256)), ("ffn_up_shexp", (sh, 256)), ("ffn_down_shexp", (256, sh))):
      sd[f"blk.{i}.{n}.weight"] = synth.q8_0_blocks(o, ii, np.random.default_rng(synth.name_seed(f"{i}{n}", 3)), scale_std=0.0015)
      shapes[f"blk.{i}.{n}"] = (o, ii)
    if cfg.shared_expert_gate: sd[f"blk.{i}.ffn_gate_inp_shexp.weight"] = (rng.standard_normal(256) * 0.1).astype(np.float32)
  w = {k: (gq.weight_matrix(v, *shapes[k[:-len(".weight")]], 8) if v.dtype == np.uint8 else v) for k, v in sd.items()}
  okw = {k: v for k, v in kw.items() if k not in ("shared_expert_dim", "shared_expert_gate", "expert_bias")}
  okw["expert_gating_func"] = moe.GATING[cfg.expert_gating_func]
  oracle = _MxOracle(llm.Config(**okw, kv_dtype="float16"), w)
  prompt = [int(t) for t in np.random.default_rng(6).integers(0, 500, 40)]
  want, want_logits = oracle.generate(prompt, 6, chunk_size=64, keep_logits=True)
  m = Transformer(cfg, sd, ggml_type=8)
  assert m.is_moe
  got = []
  for i, tok in enumerate(m.generate(list(prompt))):
    # fp8 operands: a different summation order can move a bf16 rounding across an E4M3 boundary (a 6 % step of that element), so
    # the end-to-end bound is wider than the dense model's: elementwise 1.5e-1, and 3e-2 of the logit vector's norm
    lg = m.read_logits()
    assert_close(lg, want_logits[i], tol=1.5e-1, what=f"MoE model logits at step {i}")
    assert np.linalg.norm(lg - want_logits[i]) <= 3e-2 * np.linalg.norm(want_logits[i])
    top2 = np.sort(want_logits[i])[-2:]
    if top2[1] - top2[0] > 0.25: assert tok == want[i]
    if tok != want[i]: break
    got.append(tok)
    if len(got) == 6: break


@pytest.mark.parametrize("typ,B", [(2, 3), (8, 5), (2, 11)])
def test_batched_decode_matches_oracle_per_sequence(typ, B):
  """B sequences in lock-step (tokens [B, 1] per step): each stream equals the oracle's own run of that sequence.  11 sequences: two
  passes of the few-row kernel (8 + 3 rows) per Linear."""
  from tinygrad_b200.model import Transformer, TransformerConfig
  kw = dict(num_blocks=2, dim=512, hidden_dim=1408, n_heads=8, n_kv_heads=2, norm_eps=1e-5, vocab_size=2000, head_dim=64, rope_theta=500000.0,
            rope_dim=64, max_context=96, qkv_bias=(typ == 8), kv_dtype="float16")
  cfg = TransformerConfig(**kw)
  sd = synth.dense_model_raw(cfg, typ, seed=19, embd_std=0.3, scale_std=0.02 if typ == 2 else 0.0015)
  shapes = {n: (o, i) for n, o, i in synth.linear_names(cfg)}
  w = {k: (gq.weight_matrix(v, *shapes[k[:-len(".weight")]], typ) if v.dtype == np.uint8 else v) for k, v in sd.items()}
  # prompts whose greedy choices are decided by a margin: with this seed the top-2 logit gap of every step is >= 3.7e-3 of the logit scale
  # (seed 4 has a step with a gap of 3e-6, which no arithmetic other than the oracle's own can be expected to reproduce)
  rng = np.random.default_rng(6)
  prompts = [[int(t) for t in rng.integers(0, 2000, 24)] for _ in range(B)]
  want = [llm.Transformer(llm.Config(**kw), w).generate(p, 10) for p in prompts]
  m = Transformer(cfg, sd, ggml_type=typ, batch=B)
  got = [[] for _ in range(B)]
  for step, toks in enumerate(m.generate_batch(prompts)):
    for i, t in enumerate(toks): got[i].append(t)
    if step == 9: break
  assert got == want


@pytest.mark.parametrize("tag,m,n_out,n_in,x_dtype,epi", [("q4_0", 8, 4096, 4096, np.float32, "res"), ("q8_0", 32, 512, 18944, np.float32, "bias"),
                                                        ("q4_0", 5, 200, 96, np.float16, "lin"), ("q8_0", 17, 48, 1536, np.float32, "silu"),
                                                        ("q4_0", 1, 14336 * 2, 4096, np.float32, "silu")])
def test_skinny_split_k_gemm(tag, m, n_out, n_in, x_dtype, epi):
  """Few-row GEMM (swapped operands, split K, fixed-order reduction) against the fp32 product; bit-reproducible across runs."""
  from tinygrad_b200 import quant, _lib
  from tinygrad_b200.runtime import DeviceBuffer
  typ = {"q4_0": 2, "q8_0": 8}[tag]
  rng = np.random.default_rng(m + n_out)
  x = rng.standard_normal((m, n_in)).astype(x_dtype)
  dx = DeviceBuffer.from_numpy(x)
  ws = DeviceBuffer(quant.qgemm_skinny_workspace_bytes(m, n_out, n_in))
  if epi == "silu":
    hid = n_out // 2
    g, u = synth.BLOCK_MAKERS[typ](hid, n_in, rng), synth.BLOCK_MAKERS[typ](hid, n_in, rng)
    pw = quant.repack(g, hid, n_in, typ, raw_up=u)
    y = DeviceBuffer.empty((m, hid), np.float32)
    quant.qgemm_skinny(pw.buf.ptr, typ, n_out, n_in, dx, y, m, ws, x_dtype=quant._DT[np.dtype(x_dtype)], epilogue=_lib.EPI_SILU_MUL)
    xf = x.astype(np.float32)
    ref = llm.silu(xf @ gq.weight_matrix(g, hid, n_in, typ).T) * (xf @ gq.weight_matrix(u, hid, n_in, typ).T)
  else:
    raw = synth.BLOCK_MAKERS[typ](n_out, n_in, rng)
    pw = quant.repack(raw, n_out, n_in, typ)
    bias = rng.standard_normal(n_out).astype(np.float16) if epi == "bias" else None
    res = rng.standard_normal((m, n_out)).astype(np.float32) if epi == "res" else None
    db = DeviceBuffer.from_numpy(bias) if bias is not None else None
    y = DeviceBuffer.from_numpy(res) if res is not None else DeviceBuffer.empty((m, n_out), np.float32)
    quant.qgemm_skinny(pw.buf.ptr, typ, n_out, n_in, dx, y, m, ws, x_dtype=quant._DT[np.dtype(x_dtype)], bias=db, residual=y if res is not None else None)
    w = gq.weight_matrix(raw, n_out, n_in, typ)
    if x_dtype == np.float16: w = w.astype(np.float16).astype(np.float32)
    ref = x.astype(np.float32) @ w.T + (bias.astype(np.float32) if bias is not None else 0.0) + (res if res is not None else 0.0)
  got = y.numpy()
  assert np.abs(got - ref).max() <= 3e-5 * max(1.0, np.abs(ref).max())
  if epi == "lin":
    y2 = DeviceBuffer.empty((m, n_out), np.float32)
    quant.qgemm_skinny(pw.buf.ptr, typ, n_out, n_in, dx, y2, m, ws, x_dtype=quant._DT[np.dtype(x_dtype)])
    np.testing.assert_array_equal(y2.numpy(), got)


@pytest.mark.parametrize("tag,m,n_out,n_in,x_dtype,epi", [("q4_0", 8, 4096, 4096, np.float32, "res"), ("q8_0", 8, 512, 18944, np.float32, "bias"),
                                                        ("q4_0", 5, 200, 96, np.float32, "lin"), ("q8_0", 17, 48, 1536, np.float32, "silu"),
                                                        ("q4_0", 1, 14336 * 2, 4096, np.float32, "silu"), ("q4_0", 3, 4096, 14336, np.float16, "lin"),
                                                        ("q8_0", 32, 3584, 3584, np.float32, "res")])
def test_few_row_fused_gemv(tag, m, n_out, n_in, x_dtype, epi):
  """Few activation rows on the int8 tensor cores (8 rows per pass over the weights, K chunks summed in a fixed order) against the fp32
  product: the one-row GEMV's arithmetic (15-bit activation integers, exact sums inside a block), so its error bound; bit-reproducible."""
  from tinygrad_b200 import quant, _lib
  from tinygrad_b200.runtime import DeviceBuffer
  typ = {"q4_0": 2, "q8_0": 8}[tag]
  rng = np.random.default_rng(m + n_out)
  x = rng.standard_normal((m, n_in)).astype(x_dtype)
  dx, xdt = DeviceBuffer.from_numpy(x), quant._DT[np.dtype(x_dtype)]
  ws = DeviceBuffer(quant.qgemv_rows_workspace_bytes(m, n_out, n_in))
  xf = x.astype(np.float32)
  if epi == "silu":
    hid = n_out // 2
    g, u = synth.BLOCK_MAKERS[typ](hid, n_in, rng), synth.BLOCK_MAKERS[typ](hid, n_in, rng)
    pw = quant.repack(g, hid, n_in, typ, raw_up=u)
    y = DeviceBuffer.empty((m, hid), np.float32)
    quant.qgemv_rows(pw.buf.ptr, typ, n_out, n_in, dx, y, m, ws, x_dtype=xdt, epilogue=_lib.EPI_SILU_MUL)
    ref = llm.silu(xf @ gq.weight_matrix(g, hid, n_in, typ).T) * (xf @ gq.weight_matrix(u, hid, n_in, typ).T)
  else:
    raw = synth.BLOCK_MAKERS[typ](n_out, n_in, rng)
    pw = quant.repack(raw, n_out, n_in, typ)
    bias = rng.standard_normal(n_out).astype(np.float16) if epi == "bias" else None
    res = rng.standard_normal((m, n_out)).astype(np.float32) if epi == "res" else None
    db = DeviceBuffer.from_numpy(bias) if bias is not None else None
    y = DeviceBuffer.from_numpy(res) if res is not None else DeviceBuffer.empty((m, n_out), np.float32)
    quant.qgemv_rows(pw.buf.ptr, typ, n_out, n_in, dx, y, m, ws, x_dtype=xdt, bias=db, residual=y if res is not None else None)
    ref = xf @ gq.weight_matrix(raw, n_out, n_in, typ).T + (bias.astype(np.float32) if bias is not None else 0.0) + (res if res is not None else 0.0)
  got = y.numpy()
  assert np.abs(got - ref).max() <= 5e-4 * max(1.0, np.abs(ref).max())
  if epi == "lin":
    y2 = DeviceBuffer.empty((m, n_out), np.float32)
    quant.qgemv_rows(pw.buf.ptr, typ, n_out, n_in, dx, y2, m, ws, x_dtype=xdt)
    np.testing.assert_array_equal(got.view(np.uint32), y2.numpy().view(np.uint32))
  from tinygrad_b200 import runtime
  assert runtime.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("tag,m,n_out,n_in", [("q8_0", 8, 512, 3584), ("q4_0", 5, 272, 8192), ("q8_0", 19, 160, 4096)])
def test_few_row_fused_gemv_folds_rmsnorm(tag, m, n_out, n_in):
  """`Linear(norm(x))` (tinygrad/llm/model.py:159,167): the RMSNorm inside the quantising pre-pass against the norm applied in fp32."""
  from tinygrad_b200 import quant, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  typ = {"q4_0": 2, "q8_0": 8}[tag]
  rng = np.random.default_rng(n_in)
  x = (rng.standard_normal((m, n_in)) * rng.uniform(0.2, 5.0, (m, 1))).astype(np.float32)
  nw = rng.uniform(0.5, 1.5, n_in).astype(np.float16)
  raw = synth.BLOCK_MAKERS[typ](n_out, n_in, rng)
  pw = quant.repack(raw, n_out, n_in, typ)
  ws = DeviceBuffer(quant.qgemv_rows_workspace_bytes(m, n_out, n_in))
  y = DeviceBuffer.empty((m, n_out), np.float32)
  quant.qgemv_rows(pw.buf.ptr, typ, n_out, n_in, DeviceBuffer.from_numpy(x), y, m, ws, norm_weight=DeviceBuffer.from_numpy(nw), norm_eps=1e-5)
  xn = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5).astype(np.float32) * nw.astype(np.float32)
  ref = xn @ gq.weight_matrix(raw, n_out, n_in, typ).T
  assert np.abs(y.numpy() - ref).max() <= 5e-4 * max(1.0, np.abs(ref).max())
  assert runtime.device_status() == 0
