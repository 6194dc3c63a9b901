"""GGUF container reader against the reference's parser output (golden) and the format's error cases; no GPU needed."""
import json, struct
import numpy as np
import pytest
from oracle import ggml_quant as gq
from tinygrad_b200 import gguf, synth
from tinygrad_b200.model import TransformerConfig


def _tiny():
  return TransformerConfig(num_blocks=2, dim=64, hidden_dim=128, n_heads=4, n_kv_heads=2, norm_eps=1e-5, vocab_size=96, head_dim=16,
                           rope_theta=10000.0, rope_dim=16, v_head_dim=16, max_context=80)


def test_parse_matches_reference_parser(golden):
  g = golden("gguf_llama_tiny")
  kv, t = gguf.gguf_load(g["image"].tobytes())
  want_kv = json.loads(bytes(g["kv_json"]).decode())
  assert set(kv) == set(want_kv)
  for k, v in want_kv.items():
    if isinstance(v, float): assert kv[k] == pytest.approx(v, rel=1e-7)      # fp32 metadata printed through JSON
    else: assert kv[k] == v
  for key in g.files:
    if not key.startswith("t:"): continue
    ten, ref = t[key[2:]], g[key]
    assert ten.shape == ref.shape
    got = gq.dequantize(ten.data, ten.n_elems, ten.ggml_type).reshape(ten.shape) if ten.ggml_type in (2, 8, 14) else ten.numpy().astype(np.float32)
    np.testing.assert_array_equal(got.view(np.uint32), ref.astype(np.float32).view(np.uint32))


def test_write_parse_round_trip_all_types():
  rng = np.random.default_rng(0)
  tensors = [("a.weight", (8, 64), 2, synth.q4_0_blocks(8, 64, rng)), ("b.weight", (4, 32), 8, synth.q8_0_blocks(4, 32, rng)),
             ("c.weight", (2, 256), 14, synth.q6_k_blocks(2, 256, rng)), ("d", (5,), 0, rng.standard_normal(5).astype(np.float32)),
             ("e", (3, 7), 1, rng.standard_normal((3, 7)).astype(np.float16))]
  kv = {"general.architecture": "llama", "general.alignment": 64, "x.f": 1.5, "x.i": 7, "x.neg": -3, "x.b": True, "x.s": "hello", "x.l": ["a", "bc"],
        "x.li": [1, 2, 3]}
  for version in (2, 3):
    kv2, t = gguf.gguf_parse(synth.write_gguf(kv, tensors, version=version))
    assert kv2 == kv
    for name, shape, typ, data in tensors:
      assert t[name].shape == shape and t[name].ggml_type == typ
      np.testing.assert_array_equal(t[name].data, np.ascontiguousarray(data).view(np.uint8).reshape(-1))
    assert t["e"].numpy().dtype == np.float16 and t["a.weight"].rows().shape == (8, 36)
    with pytest.raises(ValueError): t["a.weight"].numpy()


def test_invalid_files_raise_like_the_reference():
  img = synth.write_gguf({"general.architecture": "llama"}, [("d", (4,), 0, np.zeros(4, np.float32))])
  for bad in (b"GGML" + img[4:], img[:4] + struct.pack("<i", 1) + img[8:], img[:10], img[:-20]):
    with pytest.raises(ValueError, match="Invalid GGUF format!"): gguf.gguf_parse(bad)
  with pytest.raises(ValueError, match="is not supported"):                       # a block type outside this path (IQ3_XXS = 18)
    gguf.gguf_parse(synth.write_gguf({}, [("w", (256,), 18, np.zeros(98, np.uint8))]))
  kv, t = gguf.gguf_parse(synth.write_gguf({}, [("w", (256,), 12, np.zeros(144, np.uint8))]))      # Q4_K: sized and listed
  assert t["w"].ggml_type == 12 and t["w"].data.size == 144


def test_split_file_names():
  import pathlib
  p = pathlib.Path("/m/model-00001-of-00003.gguf")
  assert [x.name for x in gguf._split_paths(p, {"split.count": 3})] == [f"model-0000{i}-of-00003.gguf" for i in (1, 2, 3)]
  assert gguf._split_paths(p, {}) == [p]
  with pytest.raises(ValueError): gguf._split_paths(p, {"split.count": 3, "split.no": 1})
  with pytest.raises(ValueError): gguf._split_paths(pathlib.Path("/m/model.gguf"), {"split.count": 2})


def test_split_files_merge_when_loaded_by_path(tmp_path):
  a = synth.write_gguf({"general.architecture": "llama", "split.count": 2, "split.no": 0}, [("a", (4,), 0, np.arange(4, dtype=np.float32))])
  b = synth.write_gguf({"split.count": 2, "split.no": 1}, [("b", (2,), 0, np.ones(2, np.float32))])
  (tmp_path / "m-00001-of-00002.gguf").write_bytes(a)
  (tmp_path / "m-00002-of-00002.gguf").write_bytes(b)
  kv, t = gguf.gguf_load(tmp_path / "m-00001-of-00002.gguf")
  assert set(t) == {"a", "b"} and t["b"].numpy().tolist() == [1.0, 1.0]
  with pytest.raises(ValueError): gguf.gguf_load(a)


def test_rope_row_permutation_is_the_reference_rearrange():
  # "n (h two) d -> n (two h) d" after the first `prefix` rows of every head (tinygrad/llm/model.py:405-413)
  n_heads, per, d, prefix = 3, 8, 5, 2
  w = np.arange(n_heads * per * d).reshape(n_heads * per, d)
  got = gguf._permute_rope_rows(w, n_heads, prefix).reshape(n_heads, per, d)
  src = w.reshape(n_heads, per, d)
  for h in range(n_heads):
    np.testing.assert_array_equal(got[h, :prefix], src[h, :prefix])
    rot = src[h, prefix:]
    np.testing.assert_array_equal(got[h, prefix:], np.concatenate([rot[0::2], rot[1::2]]))


def test_lazy_state_answers_membership_without_making_tensors():
  sd = synth.LazyDenseState(_tiny(), 2, seed=0)
  assert "blk.1.ffn_down.weight" in sd and "output.weight" in sd and "token_embd.weight" in sd and "blk.0.attn_norm.weight" in sd
  assert "blk.0.attn_q.bias" not in sd and "blk.0.ffn_gate_inp.weight" not in sd and 3 not in sd
  assert sd["blk.1.ffn_down.weight"].dtype == np.uint8
