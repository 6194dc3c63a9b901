"""Generate the golden vectors under tests/golden/ by running the REFERENCE.

Usage:  python tests/golden/make_golden.py <path-to-tinygrad-checkout> [group ...]

The reference is imported from the given checkout and executed on its uop
interpreter device (DEV=PYTHON), which runs the real ``ggml_data_to_tensor``,
``Linear``, ``Transformer`` and ``quantize_mxfp8`` code -- slowly, so every
case is tiny.  Inputs come from ``tinygrad_b200.synth`` (seeded numpy); inputs
AND reference outputs are stored, so the tests never depend on the generators
staying bit-stable.  Groups: dequant linear llm_small llm_wide llm_q8 moe mxfp8.
"""
import os, sys, pathlib, time
os.environ.setdefault("DEV", "PYTHON")
ref = sys.argv[1]
sys.path.insert(0, ref)
HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
import numpy as np
from tinygrad import Tensor, dtypes, nn
from tinygrad.llm.gguf import ggml_data_to_tensor
from tinygrad.llm.model import Transformer, TransformerConfig, TransformerBlock, pairwise_topk, ExpertGating
from tinygrad_b200 import synth

groups = sys.argv[2:] or ["dequant", "linear", "llm_small", "moe", "mxfp8"]


def save(name, **arrs):
  np.savez_compressed(HERE / f"{name}.npz", **arrs)
  print("wrote", name, {k: (v.shape, str(v.dtype)) for k, v in arrs.items()}, flush=True)


def ref_weight(raw, n_out, n_in, typ):
  return ggml_data_to_tensor(Tensor(raw), n_out * n_in, typ).reshape(n_out, n_in)


if "dequant" in groups:
  out = {}
  for typ, tag in ((2, "q4_0"), (8, "q8_0"), (14, "q6_k")):
    nel, nby = synth.GGML_QUANT[typ]
    rng = np.random.default_rng(100 + typ)
    raw = synth.BLOCK_MAKERS[typ](1, 4 * nel, rng)                # 4 blocks with sane scales
    wild = rng.integers(0, 256, 2 * nby, dtype=np.uint8)          # 2 blocks of arbitrary bytes ...
    sc_off = 208 if typ == 14 else 0
    for b in range(2): wild[b * nby + sc_off: b * nby + sc_off + 2] = np.array([rng.uniform(-4, 4)], dtype=np.float16).view(np.uint8)  # ... finite scale
    raw = np.concatenate([raw, wild])
    t = ggml_data_to_tensor(Tensor(raw), 6 * nel, typ)
    out[f"{tag}_raw"], out[f"{tag}_f32"] = raw, t.numpy()
    out[f"{tag}_f16"] = t.cast(dtypes.float16).numpy()
  save("dequant", **out)

if "linear" in groups:
  out = {}
  for typ, tag, n_out, n_in in ((2, "q4_0", 32, 128), (8, "q8_0", 32, 64), (14, "q6_k", 16, 256)):
    rng = np.random.default_rng(200 + typ)
    raw = synth.BLOCK_MAKERS[typ](n_out, n_in, rng)
    x16 = rng.standard_normal((1, n_in)).astype(np.float16)
    x32 = rng.standard_normal((3, n_in)).astype(np.float32)
    w = ref_weight(raw, n_out, n_in, typ).cast(dtypes.float16)   # lazy, as Transformer.from_gguf leaves it
    out[f"{tag}_raw"], out[f"{tag}_x16"], out[f"{tag}_x32"] = raw, x16, x32
    out[f"{tag}_y16"] = Tensor(x16).linear(w.T).numpy()           # fp16 activations: fp16 out
    out[f"{tag}_y32"] = Tensor(x32).linear(w.T).numpy()           # fp32 activations: fp32 out
    out[f"{tag}_shape"] = np.array([n_out, n_in])
  save("linear", **out)


def run_llm(tag, cfg, typ, kv_half, prompt, n_new, seed):
  sd_raw = synth.dense_model_raw(cfg, typ, seed=seed, embd_std=0.5)
  model = Transformer(cfg)
  new = {}
  for k, v in sd_raw.items():
    if v.dtype == np.uint8:
      tgt = nn.state.get_state_dict(model)[k]
      new[k] = ref_weight(v, tgt.shape[0], tgt.shape[1], typ).cast(dtypes.float16)
    else: new[k] = Tensor(v)
  nn.state.load_state_dict(model, new, verbose=False, realize=False)
  # The cache dtype is the reference's default float (fp32).  Handing the block an fp16 cache up front does not run on the
  # interpreter device (its store of fp32 rows into a fp16 buffer raises), so fp16-cache streams cannot be generated here.
  assert not kv_half
  toks, t0 = [], time.time()
  for tok in model.generate(list(prompt), chunk_size=32, temperature=0.0):
    toks.append(tok); print(tag, len(toks), tok, f"{time.time()-t0:.0f}s", flush=True)
    if len(toks) >= n_new: break
  meta = np.array([cfg.num_blocks, cfg.dim, cfg.hidden_dim, cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size, cfg.head_dim,
                   cfg.rope_dim, cfg.max_context, typ, int(kv_half), int(cfg.qkv_bias), seed])
  save(tag, meta=meta, norm_eps=np.array(cfg.norm_eps), rope_theta=np.array(cfg.rope_theta), prompt=np.array(prompt), tokens=np.array(toks),
       **{"w:" + k: v for k, v in sd_raw.items()})


def tiny_cfg(**kw):
  base = dict(num_blocks=2, dim=64, hidden_dim=128, n_heads=4, n_kv_heads=2, norm_eps=1e-5, vocab_size=96, head_dim=16,
              rope_theta=10000.0, rope_dim=16, v_head_dim=16, max_context=80)
  base.update(kw)
  return TransformerConfig(**base)


if "llm_small" in groups:
  run_llm("llm_small_kv32", tiny_cfg(), 2, False, [1, 5, 9, 13, 17, 21, 25, 29], 64, seed=1)
if "llm_q8" in groups:
  run_llm("llm_q8_bias_kv32", tiny_cfg(qkv_bias=True, n_heads=2, n_kv_heads=1, head_dim=32, rope_dim=32, v_head_dim=32), 8, False,
          [7, 7, 3, 90, 41], 32, seed=3)
if "llm_wide" in groups:
  run_llm("llm_wide_kv32", tiny_cfg(dim=128, hidden_dim=384, n_heads=4, n_kv_heads=1, head_dim=32, rope_dim=32, v_head_dim=32, vocab_size=160,
                                    max_context=112), 2, False, list(range(2, 42)), 64, seed=4)

if "moe" in groups:
  rng = np.random.default_rng(300)
  x = np.concatenate([rng.standard_normal((2, 3, 8)), np.array([[[1., 1, 2, 2, 0, 0, 2, 1]] * 3] * 1)], axis=0).astype(np.float32)  # last rows: ties
  v, s = pairwise_topk(Tensor(x), 3)
  out = {"topk_x": x, "topk_v": v.numpy(), "topk_sel": s.numpy()}
  for gating, norm, tag in ((ExpertGating.SOFTMAX, False, "softmax"), (ExpertGating.SOFTMAX, True, "softmax_norm"),
                            (ExpertGating.SIGMOID, True, "sigmoid_norm"), (ExpertGating.SOFTMAX_WEIGHT, False, "softmax_weight")):
    dim, hidden, E, k = 32, 64, 8, 2
    cfg = TransformerConfig(num_blocks=1, dim=dim, hidden_dim=hidden, n_heads=2, n_kv_heads=2, norm_eps=1e-5, vocab_size=32, head_dim=16,
                            rope_theta=10000, rope_dim=16, v_head_dim=16, max_context=16, num_experts=E, num_experts_per_tok=k,
                            norm_topk_prob=norm, expert_gating_func=gating, routed_scaling_factor=1.5 if norm else 1.0)
    blk = TransformerBlock(cfg)
    ws = {n: (rng.standard_normal(shape) * 0.3).astype(np.float32) for n, shape in
          (("gate", (E, hidden, dim)), ("up", (E, hidden, dim)), ("down", (E, dim, hidden)), ("router", (E, dim)))}
    blk.ffn_gate_exps.weight, blk.ffn_up_exps.weight = Tensor(ws["gate"]), Tensor(ws["up"])
    blk.ffn_down_exps.weight, blk.ffn_gate_inp.weight = Tensor(ws["down"]), Tensor(ws["router"])
    h = rng.standard_normal((1, 5, dim)).astype(np.float32)
    y = blk._feed_forward(Tensor(h)).numpy()
    out.update({f"{tag}_{n}": a for n, a in ws.items()})
    out.update({f"{tag}_h": h, f"{tag}_y": y, f"{tag}_cfg": np.array([dim, hidden, E, k, int(gating), int(norm)]),
                f"{tag}_scale": np.array(cfg.routed_scaling_factor)})
  save("moe", **out)

if "mxfp8" in groups:
  from extra.gemm.cdna_asm_gemm import quantize_mxfp8, _mx_block_scale
  from extra.gemm.moe_routing import route
  from tinygrad.dtype import float_to_fp8, fp8_to_float
  rng = np.random.default_rng(400)
  x = (rng.standard_normal((6, 64)) * np.array([1e-3, 0.02, 1.0, 37.0, 1e4, 0.0])[:, None]).astype(np.float32)
  x[2, :4] = [448.0, -448.0, 0.0, 1e-30]
  q, e8, _ = quantize_mxfp8(Tensor(x))
  out = {"x": x, "q": q.bitcast(dtypes.uint8).numpy(), "e8": e8.numpy(),
         "deq": (q.cast(dtypes.float32) * _mx_block_scale(e8)).numpy()}
  # the scalar E4M3 conversions of tinygrad/dtype.py:237-274 over a sweep of values and every code
  vals = np.concatenate([np.linspace(-500, 500, 4001), np.logspace(-12, 3, 600), -np.logspace(-12, 3, 600),
                         rng.standard_normal(4000) * 3, np.array([0.0, -0.0])]).astype(np.float32)
  out["e4m3_in"] = vals
  out["e4m3_code"] = np.array([float_to_fp8(float(v), dtypes.fp8e4m3) for v in vals], dtype=np.uint8)
  out["e4m3_table"] = np.array([fp8_to_float(c, dtypes.fp8e4m3) for c in range(256)], dtype=np.float32)
  logits = rng.standard_normal((12, 8)).astype(np.float32)
  r = route(Tensor(logits), 2, 8)
  out.update({"route_logits": logits, "route_weights": r.weights.numpy(), "route_dest_row": r.dest_row.numpy(),
              "route_off": r.off.numpy(), "route_m_l": np.array(r.m_l)})
  save("mxfp8", **out)

if "gguf" in groups:
  # a GGUF file image of a tiny llama-family model: the reference's parser output and its greedy stream from Transformer.from_gguf
  # (which applies the family's q/k RoPE row permutation and the fp16 cast of every tensor)
  import json
  from tinygrad.llm.gguf import gguf_load
  cfg = tiny_cfg()
  img = synth.dense_model_gguf(cfg, 2, seed=5, embd_std=0.5, output="f16")
  kv, sd = gguf_load(Tensor(np.frombuffer(img, dtype=np.uint8)))
  out = {"image": np.frombuffer(img, dtype=np.uint8), "kv_json": np.frombuffer(json.dumps({k: v for k, v in kv.items()}).encode(), dtype=np.uint8)}
  for name in ("blk.0.attn_q.weight", "blk.1.ffn_down.weight", "token_embd.weight", "output.weight", "blk.0.attn_norm.weight"):
    out["t:" + name] = sd[name].numpy()
  model, _ = Transformer.from_gguf(Tensor(np.frombuffer(img, dtype=np.uint8)), max_context=80)
  toks, t0 = [], time.time()
  for tok in model.generate([3, 14, 15, 92, 65, 35], chunk_size=32, temperature=0.0):
    toks.append(tok); print("gguf", len(toks), tok, f"{time.time()-t0:.0f}s", flush=True)
    if len(toks) >= 48: break
  out["prompt"], out["tokens"] = np.array([3, 14, 15, 92, 65, 35]), np.array(toks)
  save("gguf_llama_tiny", **out)

if "mxgemm" in groups:
  # The reference's one MXFP8 contraction that runs without AMD hardware: matmul_mx of examples/mlperf/models/gpt_oss.py:64-83
  # (its portable branch: quantise-dequantise the activations per 32, dequantise the weight, bf16 matmul with fp32 accumulation).
  from extra.gemm.cdna_asm_gemm import quantize_mxfp8
  from examples.mlperf.models.gpt_oss import matmul_mx
  rng = np.random.default_rng(500)
  M, N, K = 6, 16, 96
  x = (rng.standard_normal((M, K)) * np.array([0.05, 1.0, 1.0, 30.0, 1.0, 1.0])[:, None]).astype(np.float32)
  w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
  xb = Tensor(x).cast(dtypes.bfloat16)
  w_q, w_e8, _ = quantize_mxfp8(Tensor(w))
  y = matmul_mx(xb, w_q, w_e8)
  save("mxgemm", x_bf16=xb.float().numpy(), w=w, w_q=w_q.bitcast(dtypes.uint8).numpy(), w_e8=w_e8.numpy(), y=y.float().numpy())


if "moe2" in groups:
  # the remaining gating paths of tinygrad/llm/model.py:110-134: sqrt(softplus) scores, a selection bias, a (gated) shared expert
  rng = np.random.default_rng(600)
  out = {}
  for tag, kwargs in (("softplus_bias", dict(expert_gating_func=ExpertGating.SQRT_SOFTPLUS, norm_topk_prob=True, routed_scaling_factor=2.5, expert_bias=True)),
                      ("softmax_bias_norm", dict(expert_gating_func=ExpertGating.SOFTMAX, norm_topk_prob=True, expert_bias=True)),
                      ("sigmoid_shared", dict(expert_gating_func=ExpertGating.SIGMOID, norm_topk_prob=True, shared_expert_dim=48, shared_expert_gate=True)),
                      ("softmax_shared_plain", dict(expert_gating_func=ExpertGating.SOFTMAX, shared_expert_dim=32, shared_expert_gate=False))):
    dim, hidden, E, k = 32, 64, 8, 3
    cfg = TransformerConfig(num_blocks=1, dim=dim, hidden_dim=hidden, n_heads=2, n_kv_heads=2, norm_eps=1e-5, vocab_size=32, head_dim=16,
                            rope_theta=10000, rope_dim=16, v_head_dim=16, max_context=16, num_experts=E, num_experts_per_tok=k, **kwargs)
    blk = TransformerBlock(cfg)
    sh = cfg.shared_expert_dim
    ws = {n: (rng.standard_normal(shape) * 0.3).astype(np.float32) for n, shape in
          (("gate", (E, hidden, dim)), ("up", (E, hidden, dim)), ("down", (E, dim, hidden)), ("router", (E, dim)))}
    blk.ffn_gate_exps.weight, blk.ffn_up_exps.weight = Tensor(ws["gate"]), Tensor(ws["up"])
    blk.ffn_down_exps.weight, blk.ffn_gate_inp.weight = Tensor(ws["down"]), Tensor(ws["router"])
    if cfg.expert_bias:
      ws["bias"] = (rng.standard_normal(E) * 0.5).astype(np.float32)
      blk.exp_probs_b["bias"] = Tensor(ws["bias"])
    if sh:
      for n, shape in (("sh_gate", (sh, dim)), ("sh_up", (sh, dim)), ("sh_down", (dim, sh))): ws[n] = (rng.standard_normal(shape) * 0.3).astype(np.float32)
      blk.ffn_gate_shexp.weight, blk.ffn_up_shexp.weight, blk.ffn_down_shexp.weight = Tensor(ws["sh_gate"]), Tensor(ws["sh_up"]), Tensor(ws["sh_down"])
      if cfg.shared_expert_gate:
        ws["sh_inp"] = (rng.standard_normal(dim) * 0.3).astype(np.float32)
        blk.ffn_gate_inp_shexp["weight"] = Tensor(ws["sh_inp"])
    h = rng.standard_normal((1, 5, dim)).astype(np.float32)
    y = blk._feed_forward(Tensor(h)).numpy()
    out.update({f"{tag}_{n}": a for n, a in ws.items()})
    out.update({f"{tag}_h": h, f"{tag}_y": y, f"{tag}_cfg": np.array([dim, hidden, E, k, int(cfg.expert_gating_func), int(cfg.norm_topk_prob)]),
                f"{tag}_scale": np.array(cfg.routed_scaling_factor)})
  save("moe2", **out)


if "dequant2" in groups:
  # the other block formats of real GGUF files: Q4_1, Q5_0, Q5_1, Q4_K, Q5_K (tinygrad/llm/gguf.py:47-67), 3 blocks each
  out = {}
  for typ, tag in ((3, "q4_1"), (6, "q5_0"), (7, "q5_1"), (12, "q4_k"), (13, "q5_k")):
    nel, nby = synth.GGML_SIZES[typ]
    raw = synth.random_blocks(typ, 1, 3 * nel, np.random.default_rng(700 + typ), scale_std=0.05)
    t = ggml_data_to_tensor(Tensor(raw), 3 * nel, typ)
    out[f"{tag}_raw"], out[f"{tag}_f32"] = raw, t.numpy()
    out[f"{tag}_f16"] = t.cast(dtypes.float16).numpy()
  save("dequant2", **out)


if "fp8linear" in groups:
  # `quantize_to_fp8` and the forward of `FP8Linear` (extra/fp8/fp8_linear.py:4-16,43-63).  The class's custom kernel does not build at this
  # revision of the reference (`output.size // SEQ` on a method, fp8_linear.py:23), so the contraction it states -- the product of the two
  # FP8 tensors cast to float, summed over the input features -- is evaluated with ordinary tensor ops; everything else is the class's code.
  from extra.fp8.fp8_linear import quantize_to_fp8
  rng = np.random.default_rng(900)
  out = {}
  for tag, (m, n_in, n_out) in (("a", (5, 128, 256)), ("b", (1, 256, 256))):
    # values on coarse grids (the file compresses; the FP8 rounding still has all its cases: the scales are not powers of two)
    x = (rng.integers(-400, 401, (m, n_in)) / 128).astype(np.float32)
    w = (rng.integers(-90, 91, (n_out, n_in)) / 1024).astype(np.float32)
    bias = rng.standard_normal(n_out).astype(np.float32)
    xq, xf = quantize_to_fp8(Tensor(x))
    wq, wf = quantize_to_fp8(Tensor(w))
    y = (xq.cast(dtypes.float).reshape(m, 1, n_in) * wq.cast(dtypes.float).reshape(1, n_out, n_in)).sum(axis=-1)
    y = y * wf * xf + Tensor(bias)
    out.update({f"{tag}_x": x, f"{tag}_w": w, f"{tag}_bias": bias, f"{tag}_xq": xq.bitcast(dtypes.uint8).numpy(), f"{tag}_wq": wq.bitcast(dtypes.uint8).numpy(),
                f"{tag}_xf": xf.numpy(), f"{tag}_wf": wf.numpy(), f"{tag}_y": y.numpy()})
  save("fp8linear", **out)
