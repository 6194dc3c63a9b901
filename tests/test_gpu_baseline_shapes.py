"""GPU parity at the sizes the benchmark configurations name (one transformer block of each model shape with its head,
one whole mixture-of-experts layer), against the oracle on the same seeded inputs.  The oracle's dequantisation runs
through its C restatement here (bit-identical to the numpy one, see tests/test_oracle.py) because the matrices hold
hundreds of millions of weights."""
import numpy as np
import pytest
from oracle import cpu_gemv, llm, mxfp8 as mx
from tinygrad_b200 import synth
from gpu_util import need_gpu, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _gpu(): need_gpu()


def _conditioned_model(cfg, typ, seed):
  """The benchmark's block distribution (uniform quants, half-normal fp16 scales) makes every weight matrix strongly biased
  (Q4_0: mean -0.4 sigma against an rms of 4.6 sigma, times thousands of inputs) and, at sigma 0.02, gives each Linear a gain of
  several: attention scores of tens, a softmax that is an arg-max, logits whose common part dwarfs their spread.  Elementwise
  comparison of such a network measures its conditioning, not the kernels.  For parity the same blocks get a random SIGN on the
  scale (a legal fp16 scale) and sigma = 1 / (rms of the quants * sqrt(n_in)): zero-mean weights, unit gain per Linear."""
  sd = synth.dense_model_raw(cfg, typ, seed=seed, embd_std=1.0)
  nby, qrms = synth.GGML_QUANT[typ][1], (4.61 if typ == 2 else 73.3)
  for name, n_out, n_in in synth.linear_names(cfg):
    rng = np.random.default_rng(synth.name_seed(name, seed + 1))
    blk = synth.BLOCK_MAKERS[typ](n_out, n_in, rng, scale_std=1.0 / (qrms * np.sqrt(n_in))).reshape(-1, nby)
    blk[:, 1] ^= (rng.integers(0, 2, blk.shape[0], dtype=np.uint8) << 7)          # sign bit of the fp16 scale (little endian: byte 1)
    sd[name + ".weight"] = blk.reshape(-1)
  return sd


def _oracle_weights(cfg, sd, typ):
  shapes = {n: (o, i) for n, o, i in synth.linear_names(cfg)}
  return {k: (cpu_gemv.weight_matrix(v, *shapes[k[:-len(".weight")]], typ) if v.dtype == np.uint8 else v) for k, v in sd.items()}


def _decode_logits(m, prompt, n_steps):
  toks, logits = [], []
  for tok in m.generate(list(prompt)):
    toks.append(tok); logits.append(m.read_logits().copy())
    if len(toks) == n_steps: break
  return toks, logits


def _assert_same_or_tied(got, want, ref_logits, what):
  """Greedy tokens must agree unless the oracle's own top two logits are closer than the path's tolerance."""
  for i, (g, w) in enumerate(zip(got, want)):
    if g == w: continue
    gap = abs(float(ref_logits[i][w]) - float(ref_logits[i][g]))
    assert gap <= 1e-2 * (1 + abs(float(ref_logits[i][w]))), f"{what}: step {i} chose {g}, oracle {w} (logit gap {gap:.3e})"
    break      # after a tie broken the other way the streams legitimately differ


@pytest.mark.parametrize("prompt_path", ["gemm", "steps"])
def test_llama3_8b_shape_block_and_head(prompt_path):
  """configs[1] shape (dim 4096, 32 / 8 heads of 128, FFN 14336, vocab 128256, Q4_0, fp16 cache) with one block: logits of 4 decode
  steps after a 64-token prompt, the prompt going through the tensor-core GEMMs or through one-token steps."""
  from tinygrad_b200.model import Transformer, TransformerConfig
  kw = dict(num_blocks=1, dim=4096, hidden_dim=14336, n_heads=32, n_kv_heads=8, norm_eps=1e-5, vocab_size=128256, head_dim=128,
            rope_theta=500000.0, rope_dim=128, max_context=128)
  cfg = TransformerConfig(**kw, kv_dtype="float16")
  sd = _conditioned_model(cfg, 2, seed=3)
  prompt = [int(t) for t in np.random.default_rng(8).integers(0, cfg.vocab_size, 64)]
  want, want_logits = llm.Transformer(llm.Config(**kw, kv_dtype="float16"), _oracle_weights(cfg, sd, 2)).generate(prompt, 4, keep_logits=True)
  m = Transformer(cfg, sd, ggml_type=2, prefill_rows=(32 if prompt_path == "gemm" else 0))
  got, logits = _decode_logits(m, prompt, 4)
  for i in range(4):
    assert_close(logits[i], want_logits[i], tol=3e-2, what=f"8B-shape logits, step {i}")
    if got[i] != want[i]: break
  _assert_same_or_tied(got, want, want_logits, "8B-shape block")


@pytest.mark.parametrize("batch", [1, 8])
def test_qwen2_7b_shape_block_and_head(batch):
  """configs[2] shape (dim 3584, 28 / 4 heads of 128, FFN 18944, vocab 152064, Q8_0, q/k/v bias) with one block, at batch 1 through the
  one-token kernels and at batch 8 through the lock-step batched step: logits against the oracle run per sequence."""
  from tinygrad_b200.model import Transformer, TransformerConfig
  kw = dict(num_blocks=1, dim=3584, hidden_dim=18944, n_heads=28, n_kv_heads=4, norm_eps=1e-6, vocab_size=152064, head_dim=128,
            rope_theta=1000000.0, rope_dim=128, max_context=96, qkv_bias=True)
  cfg = TransformerConfig(**kw, kv_dtype="float16")
  sd = _conditioned_model(cfg, 8, seed=5)
  w = _oracle_weights(cfg, sd, 8)
  rng = np.random.default_rng(12)
  prompts = [[int(t) for t in rng.integers(0, cfg.vocab_size, 40)] for _ in range(batch)]
  refs = [llm.Transformer(llm.Config(**kw, kv_dtype="float16"), w).generate(p, 3, keep_logits=True) for p in prompts]
  m = Transformer(cfg, sd, ggml_type=8, batch=batch)
  if batch == 1:
    got, logits = _decode_logits(m, prompts[0], 3)
    for i in range(3): assert_close(logits[i], refs[0][1][i], tol=3e-2, what=f"7B-shape logits, step {i}")
    _assert_same_or_tied(got, refs[0][0], refs[0][1], "7B-shape block")
    return
  gen = m.generate_batch(prompts)
  alive = [True] * batch
  for step in range(3):
    toks = next(gen)
    lg = m._batch_logits.numpy().reshape(batch, cfg.vocab_size)
    for b in range(batch):
      if not alive[b]: continue
      assert_close(lg[b], refs[b][1][step], tol=3e-2, what=f"7B-shape batched logits, sequence {b}, step {step}")
      if toks[b] != refs[b][0][step]:
        _assert_same_or_tied([toks[b]], [refs[b][0][step]], [refs[b][1][step]], f"sequence {b}")
        alive[b] = False


def test_llama3_70b_shape_block():
  """configs[4] shape (dim 8192, 64 / 8 heads of 128, FFN 28672, Q4_0) with one block.  The vocabulary is cut to 8192 rows so that the
  oracle's fp32 head fits comfortably; the block is the full size."""
  from tinygrad_b200.model import Transformer, TransformerConfig
  kw = dict(num_blocks=1, dim=8192, hidden_dim=28672, n_heads=64, n_kv_heads=8, norm_eps=1e-5, vocab_size=8192, head_dim=128,
            rope_theta=500000.0, rope_dim=128, max_context=128)
  cfg = TransformerConfig(**kw, kv_dtype="float16")
  sd = _conditioned_model(cfg, 2, seed=7)
  prompt = [int(t) for t in np.random.default_rng(9).integers(0, cfg.vocab_size, 70)]
  want, want_logits = llm.Transformer(llm.Config(**kw, kv_dtype="float16"), _oracle_weights(cfg, sd, 2)).generate(prompt, 3, keep_logits=True)
  m = Transformer(cfg, sd, ggml_type=2)
  got, logits = _decode_logits(m, prompt, 3)
  for i in range(3): assert_close(logits[i], want_logits[i], tol=3e-2, what=f"70B-shape logits, step {i}")
  _assert_same_or_tied(got, want, want_logits, "70B-shape block")


def _assert_rel(got, ref, tol, what):
  """|got - ref| <= tol * (rms(ref) + |ref|): the path's tolerance with the absolute part scaled to the data (MoE outputs are small numbers)."""
  got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
  err, scale = np.abs(got - ref), float(np.sqrt((ref * ref).mean()))
  bad = err > tol * (scale + np.abs(ref))
  assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} beyond {tol}; max err {err.max():.3e} at rms {scale:.3e}"
  assert np.sqrt((err * err).mean()) <= 0.3 * tol * scale, f"{what}: rms error {np.sqrt((err * err).mean()):.3e} vs rms {scale:.3e}"


def test_grouped_mxfp8_gemm_olmoe_size():
  """`grouped_mx_gemm` alone at the expert-GEMM size of configs[3]: N 2048, K 2048, 64 groups of uneven size, one of them empty."""
  from tinygrad_b200 import _lib, moe
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(21)
  E, N, K = 64, 2048, 2048
  sizes = rng.integers(1, 4, E) * 256
  sizes[5] = 0
  off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
  M = int(off[-1]) + 256                                                  # 256 rows past the last group
  a = rng.standard_normal((M, K)).astype(np.float32)
  a_q, a_e8 = mx.quantize_mxfp8(a)
  w = DeviceBuffer.from_numpy((rng.standard_normal((E * N, K), dtype=np.float32) * 0.02))
  w_q, w_e8 = moe.quantize_mxfp8(w, E * N, K, _lib.F32)                   # the device quantiser is pinned bit-exact elsewhere
  wq_h, we_h = w_q.numpy().reshape(E, N, K), w_e8.numpy().reshape(E, N, K // 32)
  ref = mx.to_bf16(mx.grouped_mx_gemm(a_q, a_e8, wq_h, we_h, off))
  d = [DeviceBuffer.from_numpy(v) for v in (a_q, a_e8, off)]
  c = DeviceBuffer.from_numpy(np.full((M, N), 0x7FC0, np.uint16))
  _lib.check(_lib.load().b200q_grouped_mxfp8_gemm(d[0].ptr, d[1].ptr, w_q.ptr, w_e8.ptr, d[2].ptr, E, M, N, K, c.ptr, None))
  got = c.numpy()
  assert (got[off[-1]:] == 0x7FC0).all()
  _assert_rel(moe.from_bf16_bits(got[:off[-1]]), ref[:off[-1]], 1e-2, "grouped MXFP8 GEMM, 64 groups")


@pytest.mark.parametrize("mode", [1, 0])
def test_olmoe_shape_moe_layer(mode):
  """One whole configs[3] layer: 4096 tokens, 64 experts, top-8, d_model 2048, expert FFN 1024, against the composed oracle
  (route -> dispatch -> quantise -> grouped GEMM -> SwiGLU -> quantise -> grouped GEMM -> combine)."""
  from tinygrad_b200 import moe
  from tinygrad_b200.runtime import DeviceBuffer
  rng = np.random.default_rng(31)
  T, D, F, E, k = 4096, 2048, 1024, 64, 8
  wg, wu, wd = ((rng.standard_normal(s, dtype=np.float32) * 0.02) for s in ((E, F, D), (E, F, D), (E, D, F)))
  xb = moe.to_bf16_bits(rng.standard_normal((T, D), dtype=np.float32))
  x = moe.from_bf16_bits(xb)
  logits = rng.standard_normal((T, E), dtype=np.float32)
  m = moe.MxMoE(wg, wu, wd, k, mode)
  out = moe.from_bf16_bits(m(DeviceBuffer.from_numpy(xb), DeviceBuffer.from_numpy(logits), T).numpy())
  # ---- oracle chain; expert weights are quantised by the device quantiser (bit-exact against the reference's golden elsewhere)
  w, topi, dest, off, m_l = mx.route(logits, k, E)
  if mode == 1:      # softmax over all experts, ascending compare-count order (tinygrad/llm/model.py:35-41,118,123-124)
    _, sel = llm.pairwise_topk(logits[None], k); topi = sel[0]
    w = np.take_along_axis(llm.softmax(logits), topi.astype(np.int64), -1)
    dest = m.last_routing.dest_row.numpy()                               # placement is checked in test_gpu_moe.py
  np.testing.assert_array_equal(m.last_routing.off.numpy(), off)
  np.testing.assert_array_equal(m.last_routing.topi.numpy(), topi)
  xq, xe = mx.quantize_mxfp8(x)                                           # quantise once per token, then dispatch the quantised rows
  a_q, a_e8 = np.zeros((m_l, D), np.uint8), np.zeros((m_l, D // 32), np.uint8)
  a_q[dest], a_e8[dest] = np.repeat(xq, k, axis=0), np.repeat(xe, k, axis=0)
  gu_q = np.stack([m.gu_q.numpy().reshape(E, F // 128, 2, 128, D)[:, :, i].reshape(E, F, D) for i in (0, 1)], axis=1).reshape(E, 2 * F, D)
  gu_e8 = np.stack([m.gu_e8.numpy().reshape(E, F // 128, 2, 128, D // 32)[:, :, i].reshape(E, F, D // 32) for i in (0, 1)], axis=1).reshape(E, 2 * F, D // 32)
  h = mx.to_bf16(mx.grouped_mx_gemm(a_q, a_e8, gu_q, gu_e8, off))
  act = mx.to_bf16(llm.silu(h[:, :F]) * h[:, F:])
  act_q, act_e8 = mx.quantize_mxfp8(act)
  y = mx.to_bf16(mx.grouped_mx_gemm(act_q, act_e8, m.dn_q.numpy().reshape(E, D, F), m.dn_e8.numpy().reshape(E, D, F // 32), off))
  ref = mx.to_bf16(mx.combine(y, dest, w))
  _assert_rel(out, ref, 1e-2, f"OLMoE-shape MoE layer, routing mode {mode}")
