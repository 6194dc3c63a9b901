"""GPU parity of the decode step: attention, arg-max, and greedy token streams
against the reference's golden streams and against the numpy oracle."""
import ctypes
import numpy as np
import pytest
from oracle import ggml_quant as gq, llm
from tinygrad_b200 import synth
from gpu_util import need_gpu, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _gpu(): need_gpu()


def _oracle_weights(cfg, sd, typ):
  shapes = {n: (o, i) for n, o, i in synth.linear_names(cfg)}
  return {k: (gq.weight_matrix(v, *shapes[k[:-len(".weight")]], typ) if v.dtype == np.uint8 else v) for k, v in sd.items()}


def _cfgs(g):
  from tinygrad_b200.model import TransformerConfig
  nb, dim, hid, nh, nkv, vocab, hd, rd, ctx, typ, kv_half, bias, seed = (int(v) for v in g["meta"])
  kw = dict(num_blocks=nb, dim=dim, hidden_dim=hid, n_heads=nh, n_kv_heads=nkv, norm_eps=float(g["norm_eps"]), vocab_size=vocab, head_dim=hd,
            rope_theta=float(g["rope_theta"]), rope_dim=rd, max_context=ctx, qkv_bias=bool(bias), kv_dtype="float16" if kv_half else "float32")
  return TransformerConfig(**kw), llm.Config(**kw), typ


@pytest.mark.parametrize("name", ["llm_small_kv32", "llm_q8_bias_kv32", "llm_wide_kv32"])
@pytest.mark.parametrize("mode", ["step", "graph_pdl", "eager"])
def test_greedy_stream_identical_to_reference(golden, name, mode):
  """Identical greedy token stream to tinygrad's own run of the same seeded model (64 tokens where the fixture holds 64), through the
  whole-step kernel (the models whose head_dim it takes), the chained launches replayed as a graph, and the same launches eagerly."""
  from tinygrad_b200.model import Transformer
  g = golden(name)
  cfg, _, typ = _cfgs(g)
  sd = {k[2:]: g[k] for k in g.files if k.startswith("w:")}
  m = Transformer(cfg, sd, ggml_type=typ, use_pdl=(mode == "graph_pdl"), use_graph=(mode == "graph_pdl"), engine="step" if mode == "step" and cfg.head_dim % 32 == 0 else "chain")
  assert m.engine == ("step" if mode == "step" and cfg.head_dim % 32 == 0 else "chain")
  want = [int(t) for t in g["tokens"]]
  got = []
  for tok in m.generate([int(t) for t in g["prompt"]]):
    got.append(tok)
    if len(got) == len(want): break
  assert got == want


@pytest.mark.parametrize("typ,kv,hd,handover", [(2, "float16", 64, None), (8, "float16", 64, None), (2, "float32", 64, None),
                                                 (2, "float16", 128, True), (8, "float16", 128, True), (2, "float16", 128, False),
                                                 (2, "float16", 128, None), (2, "float16", 128, "gateup_down,down_qkv"),
                                                 (2, "float16", 128, "unstaged"), (8, "float16", 128, "unstaged"),
                                                 (2, "float16", 64, "step"), (8, "float16", 64, "step"), (2, "float32", 64, "step"),
                                                 (2, "float16", 128, "step"), (8, "float32", 128, "step"), (8, "float16", 32, "step")])
def test_mid_size_model_matches_oracle(typ, kv, hd, handover, monkeypatch):
  """A model too big for the reference's interpreter: logits within tolerance of the oracle at every step,
  identical greedy stream, and KV-prefix reuse gives the same continuation.  handover True: every GEMV hands its output row to the
  next one as a quantised record, blocks collected through the staging row; "unstaged": the same with runs of row tiles per CTA."""
  from tinygrad_b200 import model as model_mod
  from tinygrad_b200.model import Transformer, TransformerConfig
  if handover == "unstaged":
    monkeypatch.setattr(model_mod, "STAGED_HANDOVER", False)
    handover = True
  kw = dict(num_blocks=3, dim=512, hidden_dim=1408, n_heads=512 // hd, n_kv_heads=2, norm_eps=1e-5, vocab_size=2000, head_dim=hd, rope_theta=500000.0,
            rope_dim=hd, max_context=160, qkv_bias=(typ == 8), kv_dtype=kv)
  cfg = TransformerConfig(**kw)
  sd = synth.dense_model_raw(cfg, typ, seed=11, embd_std=0.3, scale_std=0.02 if typ == 2 else 0.0015)   # weights of rms ~0.1 either way
  prompt = [int(t) for t in np.random.default_rng(1).integers(0, 2000, 70)]
  want, want_logits = llm.Transformer(llm.Config(**kw), _oracle_weights(cfg, sd, typ)).generate(prompt, 24, keep_logits=True)
  if handover == "step":      # the whole-step kernel instead of the chained launches
    m = Transformer(cfg, sd, ggml_type=typ, engine="step")
  else:
    m = Transformer(cfg, sd, ggml_type=typ, handover=handover, engine="chain")
    if handover is not None: assert m.handover == bool(handover)
  got = []
  for i, tok in enumerate(m.generate(list(prompt))):
    # logits after several blocks: the 15-bit activation quantisation (like the fp16 rounding of the KV cache, which moves
    # these logits by as much) is amplified by the random-weight network, so the end-to-end bound is looser than one GEMV's
    assert_close(m.read_logits(), want_logits[i], tol=3e-2, what=f"logits at step {i}")
    got.append(tok)
    if len(got) == 24: break
  assert got == want
  again = []
  for tok in m.generate(prompt + got[:8]):          # reuses the cached prefix (get_start_pos)
    again.append(tok)
    if len(again) == 8: break
  assert again == got[8:16]


@pytest.mark.parametrize("kv_dtype,n_heads,n_kv,hd,rope_dim,pos,n_split", [
  (np.float16, 32, 8, 128, 128, 0, 16), (np.float16, 32, 8, 128, 128, 700, 16), (np.float16, 28, 4, 128, 128, 300, 16),
  (np.float32, 4, 2, 16, 16, 33, 16), (np.float16, 8, 1, 64, 32, 517, 20), (np.float16, 64, 8, 128, 128, 1023, 16),
  (np.float16, 32, 8, 128, 128, 63, 16), (np.float16, 32, 8, 128, 128, 64, 16), (np.float32, 16, 4, 128, 64, 127, 16)])
def test_attention_decode_matches_oracle(kv_dtype, n_heads, n_kv, hd, rope_dim, pos, n_split):
  from tinygrad_b200 import _lib
  from tinygrad_b200.runtime import DeviceBuffer
  from tinygrad_b200.model import precompute_freqs_cis
  rng = np.random.default_rng(pos + n_heads)
  ctx = 1024
  qkv = rng.standard_normal((n_heads + 2 * n_kv) * hd).astype(np.float32)
  kc = (rng.standard_normal((n_kv, ctx, hd)) * 0.5).astype(kv_dtype); vc = rng.standard_normal((n_kv, ctx, hd)).astype(kv_dtype)
  fc = precompute_freqs_cis(rope_dim, ctx, 10000.0)
  # oracle: tinygrad/llm/model.py:167-198 with T == 1
  q = qkv[:n_heads * hd].reshape(1, n_heads, 1, hd); k = qkv[n_heads * hd:(n_heads + n_kv) * hd].reshape(1, n_kv, 1, hd)
  v = qkv[(n_heads + n_kv) * hd:].reshape(1, n_kv, 1, hd)
  rope = lambda t: np.concatenate([llm.apply_rope(t[..., :rope_dim], fc[pos:pos + 1]), t[..., rope_dim:]], axis=-1)
  kc_ref, vc_ref = kc.copy(), vc.copy()
  kc_ref[:, pos] = rope(k)[0, :, 0].astype(kv_dtype); vc_ref[:, pos] = v[0, :, 0].astype(kv_dtype)
  kk = np.repeat(kc_ref[:, :pos + 1].astype(np.float32), n_heads // n_kv, axis=0); vv = np.repeat(vc_ref[:, :pos + 1].astype(np.float32), n_heads // n_kv, axis=0)
  s = np.einsum("hd,hpd->hp", rope(q)[0, :, 0], kk) / np.float32(np.sqrt(hd))
  ref = np.einsum("hp,hpd->hd", llm.softmax(s), vv).reshape(-1)
  lib = _lib.load()
  d = {n: DeviceBuffer.from_numpy(a) for n, a in (("qkv", qkv), ("kc", kc), ("vc", vc), ("fc", fc), ("pos", np.array([pos], np.int32)))}
  out = DeviceBuffer.empty((n_heads * hd,), np.float32)
  scratch = DeviceBuffer(lib.b200q_attn_scratch_bytes(n_heads, n_kv, hd, n_split), zero=True)
  a = _lib.AttnArgs(d["qkv"].ptr, d["kc"].ptr, d["vc"].ptr, _lib.F16 if kv_dtype == np.float16 else _lib.F32, d["fc"].ptr, d["pos"].ptr, out.ptr,
                    scratch.ptr, n_heads, n_kv, hd, rope_dim, ctx, n_split, 0, None)
  for _ in range(2):   # the scratch counters must reset themselves
    _lib.check(lib.b200q_attn_decode(ctypes.byref(a), None))
    assert_close(out.numpy(), ref, tol=2e-3, what="attention output")
  if kv_dtype == np.float16:   # appended rows, rounded once to the cache dtype
    np.testing.assert_array_equal(d["kc"].numpy()[:, pos], kc_ref[:, pos])
  else:                        # fp32 cache: the rotation may be contracted into FMAs (last-bit differences)
    np.testing.assert_allclose(d["kc"].numpy()[:, pos], kc_ref[:, pos], rtol=1e-6, atol=1e-6)
  np.testing.assert_array_equal(d["vc"].numpy()[:, pos], vc_ref[:, pos])
  mask = np.ones(ctx, bool); mask[pos] = False
  np.testing.assert_array_equal(d["kc"].numpy()[:, mask], kc[:, mask])        # nothing else touched


def test_attention_of_several_sequences_in_one_launch():
  """b200q_attn_decode_seqs (sequences in lock-step, each at its own position of its own cache) gives, bit for bit, what one
  b200q_attn_decode per sequence gives: outputs and appended cache rows."""
  from tinygrad_b200 import _lib, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  from tinygrad_b200.model import precompute_freqs_cis
  lib = _lib.load()
  rng = np.random.default_rng(11)
  B, n_heads, n_kv, hd, ctx = 3, 14, 2, 128, 200
  n_split = lib.b200q_attn_min_split(ctx)
  row = (n_heads + 2 * n_kv) * hd
  qkv = rng.standard_normal((B, row)).astype(np.float32)
  kc = (rng.standard_normal((B, n_kv, ctx, hd)) * 0.5).astype(np.float16); vc = rng.standard_normal((B, n_kv, ctx, hd)).astype(np.float16)
  pos = np.array([150, 3, 64], np.int32)
  fc = DeviceBuffer.from_numpy(precompute_freqs_cis(hd, ctx, 10000.0))
  # one launch per sequence
  outs, kcs, vcs = [], [], []
  for s in range(B):
    d = {n: DeviceBuffer.from_numpy(np.ascontiguousarray(a)) for n, a in (("qkv", qkv[s]), ("kc", kc[s]), ("vc", vc[s]), ("pos", pos[s:s + 1]))}
    out = DeviceBuffer.empty((n_heads * hd,), np.float32)
    scratch = DeviceBuffer(lib.b200q_attn_scratch_bytes(n_heads, n_kv, hd, n_split), zero=True)
    a = _lib.AttnArgs(d["qkv"].ptr, d["kc"].ptr, d["vc"].ptr, _lib.F16, fc.ptr, d["pos"].ptr, out.ptr, scratch.ptr, n_heads, n_kv, hd, hd, ctx, n_split, 0, None)
    _lib.check(lib.b200q_attn_decode(ctypes.byref(a), None))
    outs.append(out.numpy()); kcs.append(d["kc"].numpy()); vcs.append(d["vc"].numpy())
  # all of them at once
  d = {n: DeviceBuffer.from_numpy(a) for n, a in (("qkv", qkv), ("kc", kc), ("vc", vc), ("pos", pos))}
  out = DeviceBuffer.empty((B, n_heads * hd), np.float32)
  scratch = DeviceBuffer(B * lib.b200q_attn_seq_scratch_stride(n_heads, n_kv, hd, n_split), zero=True)
  a = _lib.AttnArgs(d["qkv"].ptr, d["kc"].ptr, d["vc"].ptr, _lib.F16, fc.ptr, d["pos"].ptr, out.ptr, scratch.ptr, n_heads, n_kv, hd, hd, ctx, n_split, 0, None)
  for _ in range(2):
    _lib.check(lib.b200q_attn_decode_seqs(ctypes.byref(a), B, None))
    np.testing.assert_array_equal(out.numpy().view(np.uint32), np.stack(outs).view(np.uint32))
  np.testing.assert_array_equal(d["kc"].numpy(), np.stack(kcs)); np.testing.assert_array_equal(d["vc"].numpy(), np.stack(vcs))
  assert runtime.device_status() == 0
  a.xq_out = 16
  assert lib.b200q_attn_decode_seqs(ctypes.byref(a), B, None) == -1      # no quantised record in the multi-sequence form


def test_attention_at_the_last_cache_row_and_refusal_past_it():
  """pos == max_context - 1 with a context that is not a multiple of the 64-position slice is served; pos == max_context
  touches nothing (cache and output unchanged) and raises status 2; embed / arg-max / advance stop at the table's end."""
  from tinygrad_b200 import _lib, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  from tinygrad_b200.model import precompute_freqs_cis
  lib = _lib.load()
  rng = np.random.default_rng(3)
  n_heads, n_kv, hd, ctx = 8, 2, 128, 100
  n_split = lib.b200q_attn_min_split(ctx)
  qkv = rng.standard_normal((n_heads + 2 * n_kv) * hd).astype(np.float32)
  kc = (rng.standard_normal((n_kv, ctx, hd)) * 0.5).astype(np.float16); vc = rng.standard_normal((n_kv, ctx, hd)).astype(np.float16)
  fc = precompute_freqs_cis(hd, ctx, 10000.0)
  assert runtime.device_status() == 0
  for pos in (ctx - 1, ctx):
    d = {n: DeviceBuffer.from_numpy(a) for n, a in (("qkv", qkv), ("kc", kc), ("vc", vc), ("fc", fc), ("pos", np.array([pos], np.int32)))}
    out = DeviceBuffer.from_numpy(np.full(n_heads * hd, 7.0, np.float32))
    scratch = DeviceBuffer(lib.b200q_attn_scratch_bytes(n_heads, n_kv, hd, n_split), zero=True)
    a = _lib.AttnArgs(d["qkv"].ptr, d["kc"].ptr, d["vc"].ptr, _lib.F16, d["fc"].ptr, d["pos"].ptr, out.ptr, scratch.ptr, n_heads, n_kv, hd, hd, ctx, n_split,
                      0, None)
    _lib.check(lib.b200q_attn_decode(ctypes.byref(a), None))
    if pos == ctx:
      assert runtime.device_status() == 2
      np.testing.assert_array_equal(d["kc"].numpy(), kc); np.testing.assert_array_equal(d["vc"].numpy(), vc)
      np.testing.assert_array_equal(out.numpy(), np.full(n_heads * hd, 7.0, np.float32))
      continue
    q = qkv[:n_heads * hd].reshape(1, n_heads, 1, hd); k = qkv[n_heads * hd:(n_heads + n_kv) * hd].reshape(1, n_kv, 1, hd)
    v = qkv[(n_heads + n_kv) * hd:].reshape(n_kv, hd)
    kr, vr = kc.copy(), vc.copy()
    kr[:, pos] = llm.apply_rope(k, fc[pos:pos + 1])[0, :, 0].astype(np.float16); vr[:, pos] = v.astype(np.float16)
    kk, vv = np.repeat(kr.astype(np.float32), n_heads // n_kv, axis=0), np.repeat(vr.astype(np.float32), n_heads // n_kv, axis=0)
    sc = np.einsum("hd,hpd->hp", llm.apply_rope(q, fc[pos:pos + 1])[0, :, 0], kk) / np.float32(np.sqrt(hd))
    assert_close(out.numpy(), np.einsum("hp,hpd->hd", llm.softmax(sc), vv).reshape(-1), tol=2e-3, what="attention at the last row")
    # the rotation may be contracted into FMAs on the device: the appended row is the oracle's up to one fp16 rounding step
    np.testing.assert_allclose(d["kc"].numpy()[:, pos].astype(np.float32), kr[:, pos].astype(np.float32), rtol=1e-3, atol=1e-6)
    np.testing.assert_array_equal(d["vc"].numpy()[:, pos], vr[:, pos])
    assert runtime.device_status() == 0
  # token table of max_context + 1 entries: the arg-max writes entry max_context at most
  toks, logits = DeviceBuffer.from_numpy(np.arange(9, dtype=np.int32)), DeviceBuffer.from_numpy(np.array([0.0, 3.0, 1.0], np.float32))
  scratch = DeviceBuffer(lib.b200q_argmax_scratch_bytes(), zero=True)
  p = DeviceBuffer.from_numpy(np.array([7], np.int32))
  _lib.check(lib.b200q_argmax_advance(logits.ptr, 3, toks.ptr, p.ptr, 8, scratch.ptr, 0, None))
  assert int(p.numpy()[0]) == 8 and int(toks.numpy()[8]) == 1 and runtime.device_status() == 0
  _lib.check(lib.b200q_argmax_advance(logits.ptr, 3, toks.ptr, p.ptr, 8, scratch.ptr, 0, None))
  _lib.check(lib.b200q_advance(p.ptr, 8, 0, None))
  assert int(p.numpy()[0]) == 8 and runtime.device_status() == 2
  np.testing.assert_array_equal(toks.numpy(), [0, 1, 2, 3, 4, 5, 6, 7, 1])


def test_argmax_lowest_index_wins_ties_and_advances():
  from tinygrad_b200 import _lib
  from tinygrad_b200.runtime import DeviceBuffer
  lib = _lib.load()
  rng = np.random.default_rng(0)
  scratch = DeviceBuffer(lib.b200q_argmax_scratch_bytes(), zero=True)
  for n in (1, 96, 128256, 152064):
    logits = rng.standard_normal(n).astype(np.float32)
    if n > 1000: logits[[77777, 5000, 90000]] = logits.max() + 1.0          # a three-way tie
    d, toks, pos = DeviceBuffer.from_numpy(logits), DeviceBuffer.empty((8,), np.int32, zero=True), DeviceBuffer.from_numpy(np.array([3], np.int32))
    _lib.check(lib.b200q_argmax_advance(d.ptr, n, toks.ptr, pos.ptr, 7, scratch.ptr, 0, None))
    assert int(pos.numpy()[0]) == 4
    assert int(toks.numpy()[4]) == int(np.argmax(logits))


def test_no_kernel_wait_ran_out():
  from tinygrad_b200 import runtime
  assert runtime.device_status() == 0


def test_from_gguf_stream_identical_to_reference(golden):
  """A GGUF file image through the loader (metadata -> config, llama q/k RoPE row permutation, F16 head on the dense GEMV):
  the same greedy stream as the reference's Transformer.from_gguf on the same image."""
  from tinygrad_b200 import gguf
  g = golden("gguf_llama_tiny")
  m, kv = gguf.transformer_from_gguf(g["image"].tobytes(), max_context=80, kv_dtype="float32")
  assert kv["general.architecture"] == "llama" and m.output_type == 1
  want, got = [int(t) for t in g["tokens"]], []
  for tok in m.generate([int(t) for t in g["prompt"]]):
    got.append(tok)
    if len(got) == len(want): break
  assert got == want


@pytest.mark.parametrize("output", ["q6_k", "tied", "same", "bf16", "f32"])
def test_from_gguf_output_head_variants(output):
  """Q6_K, tied (token_embd) and same-type output heads of a qwen2-family file against the oracle."""
  from tinygrad_b200 import gguf
  from tinygrad_b200.model import TransformerConfig
  kw = dict(num_blocks=2, dim=256, hidden_dim=512, n_heads=4, n_kv_heads=2, norm_eps=1e-6, vocab_size=320, head_dim=64, rope_theta=10000.0,
            rope_dim=64, max_context=64, qkv_bias=True)
  cfg = TransformerConfig(**kw)
  img = synth.dense_model_gguf(cfg, 8, seed=21, arch="qwen2", embd_std=0.3, output=output)
  kv, t = gguf.gguf_load(img)
  sd = synth.dense_model_raw(cfg, 8, seed=21, embd_std=0.3)
  w = _oracle_weights(cfg, sd, 8)
  head = t.get("output.weight", t["token_embd.weight"])
  if output != "same":
    w["output.weight"] = (gq.dequantize(head.data, head.n_elems, 14).astype(np.float16) if head.ggml_type == 14 else head.numpy()) \
                           .astype(np.float32).reshape(cfg.vocab_size, cfg.dim)
  prompt = [5, 17, 300, 2, 9]
  want = llm.Transformer(llm.Config(**kw, kv_dtype="float16"), w).generate(prompt, 16)
  m, _ = gguf.transformer_from_gguf(img)
  assert m.config.qkv_bias and m.output_type == {"q6_k": 14, "tied": 1, "same": 8, "bf16": 30, "f32": 0}[output]
  got = []
  for tok in m.generate(prompt):
    got.append(tok)
    if len(got) == 16: break
  assert got == want


def test_from_gguf_mixed_block_formats():
  """A file that mixes block formats like the K-quant files of the reference's model zoo (Q4_K blocks with Q6_K for attn_v / ffn_down / the
  head, a Q5_K output projection, Q4_1 / Q5_0 / Q5_1 elsewhere, a Q4_K embedding): loads onto the dense fp16 path and decodes like the oracle."""
  from tinygrad_b200 import gguf
  from tinygrad_b200.model import TransformerConfig
  kw = dict(num_blocks=2, dim=256, hidden_dim=512, n_heads=4, n_kv_heads=2, norm_eps=1e-6, vocab_size=320, head_dim=64, rope_theta=10000.0,
            rope_dim=64, max_context=64)
  cfg = TransformerConfig(**kw)
  mixed = {"attn_q": 12, "attn_k": 3, "attn_v": 14, "attn_output": 13, "ffn_gate": 6, "ffn_up": 7, "ffn_down": 14}
  img = synth.dense_model_gguf(cfg, 12, seed=23, arch="qwen2", embd_std=0.3, output="q6_k", mixed=mixed, embd_type=12)
  kv, t = gguf.gguf_load(img)
  assert {t[f"blk.0.{n}.weight"].ggml_type for n in mixed} == set(mixed.values())
  w = {}
  for name, g in t.items():
    if g.ggml_type in (0, 1, 30): w[name] = g.numpy().astype(np.float32)
    else: w[name] = gq.dequantize(g.data, g.n_elems, g.ggml_type).astype(np.float16).astype(np.float32).reshape(g.shape)      # model.py:376: every tensor is cast to fp16
  prompt = [5, 17, 300, 2, 9, 44]
  want, want_logits = llm.Transformer(llm.Config(**kw, kv_dtype="float16"), w).generate(prompt, 12, keep_logits=True)
  m, _ = gguf.transformer_from_gguf(img)
  assert m.dense_blocks and m.output_type == 14
  got = []
  for i, tok in enumerate(m.generate(prompt)):
    assert_close(m.read_logits(), want_logits[i], tol=3e-2, what=f"mixed-format logits at step {i}")
    got.append(tok)
    if len(got) == 12: break
  assert got == want
