"""Seeded synthetic inputs: raw GGUF quant blocks, activations, model weights.

Pure numpy.  The benchmark configurations name no dataset: weights, token ids
and activations are random with stated distributions, so every generator here
takes an explicit seed (or derives one from the tensor's name with crc32, which
is stable across processes, unlike Python's salted ``hash``).
"""
import zlib
import numpy as np

Q4_0, Q8_0, Q6_K = 2, 8, 14
# {ggml_type: (elements per block, bytes per block)}; same table as tinygrad/llm/gguf.py:20-21
GGML_QUANT = {Q4_0: (32, 18), Q8_0: (32, 34), Q6_K: (256, 210)}


def name_seed(name: str, base: int = 0) -> int:
  return (zlib.crc32(name.encode()) + base) & 0xFFFFFFFF


def q4_0_blocks(n_out: int, n_in: int, rng, scale_std: float = 0.02) -> np.ndarray:
  """(n_out, n_in) weight as raw Q4_0 bytes: per 32 elements an fp16 scale
  |N(0, scale_std)| followed by 16 bytes of uniform nibbles (value=(q-8)*d)."""
  nb = n_out * n_in // 32
  out = np.empty((nb, 18), dtype=np.uint8)
  out[:, :2] = np.abs(rng.standard_normal(nb, dtype=np.float32) * scale_std).astype(np.float16).view(np.uint8).reshape(nb, 2)
  out[:, 2:] = rng.integers(0, 256, (nb, 16), dtype=np.uint8)
  return out.reshape(-1)


def q8_0_blocks(n_out: int, n_in: int, rng, scale_std: float = 0.01) -> np.ndarray:
  """Raw Q8_0 bytes: fp16 scale |N(0, scale_std)| + 32 int8 uniform in [-127,127]."""
  nb = n_out * n_in // 32
  out = np.empty((nb, 34), dtype=np.uint8)
  out[:, :2] = np.abs(rng.standard_normal(nb, dtype=np.float32) * scale_std).astype(np.float16).view(np.uint8).reshape(nb, 2)
  out[:, 2:] = rng.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
  return out.reshape(-1)


def q6_k_blocks(n_out: int, n_in: int, rng, scale_std: float = 0.001) -> np.ndarray:
  """Raw Q6_K bytes: 128 B low nibbles, 64 B high 2-bit fields, 16 int8
  sub-block scales, fp16 super-block scale."""
  nb = n_out * n_in // 256
  out = np.empty((nb, 210), dtype=np.uint8)
  out[:, :192] = rng.integers(0, 256, (nb, 192), dtype=np.uint8)
  out[:, 192:208] = rng.integers(-64, 64, (nb, 16), dtype=np.int8).view(np.uint8)
  out[:, 208:] = np.abs(rng.standard_normal(nb, dtype=np.float32) * scale_std).astype(np.float16).view(np.uint8).reshape(nb, 2)
  return out.reshape(-1)


def random_blocks(ggml_type: int, n_out: int, n_in: int, rng, scale_std: float = 0.01) -> np.ndarray:
  """Raw blocks of any of the sized block types: random bytes, with sane (finite, small) fp16 values where the format keeps scales."""
  nel, nby = GGML_SIZES[ggml_type]
  nb = n_out * n_in // nel
  out = rng.integers(0, 256, (nb, nby), dtype=np.uint8)
  for off in F16_FIELDS[ggml_type]:
    out[:, off:off + 2] = np.abs(rng.standard_normal(nb, dtype=np.float32) * scale_std).astype(np.float16).view(np.uint8).reshape(nb, 2)
  return out.reshape(-1)


# {ggml_type: (elements, bytes)} of every block format the dequantisers cover (tinygrad/llm/gguf.py:20-21), and where their fp16 fields sit
GGML_SIZES = {2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}
F16_FIELDS = {2: (0,), 3: (0, 2), 6: (0,), 7: (0, 2), 8: (0,), 12: (0, 2), 13: (0, 2), 14: (208,)}
BLOCK_MAKERS = {Q4_0: q4_0_blocks, Q8_0: q8_0_blocks, Q6_K: q6_k_blocks}


def linear_names(cfg) -> list:
  """(state-dict name, out, in) of every quantised Linear of a dense model,
  named as tinygrad/llm/model.py:105-107,161-164,350 name them."""
  qd, kvd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
  names = []
  for i in range(cfg.num_blocks):
    names += [(f"blk.{i}.attn_q", qd, cfg.dim), (f"blk.{i}.attn_k", kvd, cfg.dim), (f"blk.{i}.attn_v", kvd, cfg.dim),
              (f"blk.{i}.attn_output", cfg.dim, qd), (f"blk.{i}.ffn_gate", cfg.hidden_dim, cfg.dim),
              (f"blk.{i}.ffn_up", cfg.hidden_dim, cfg.dim), (f"blk.{i}.ffn_down", cfg.dim, cfg.hidden_dim)]
  names.append(("output", cfg.vocab_size, cfg.dim))
  return names


def dense_model_raw(cfg, ggml_type: int = Q4_0, seed: int = 0, embd_std: float = 0.02, bias_std: float = 0.02, scale_std=None) -> dict:
  """Random-init dense model as the loader would see it: every Linear weight
  as raw quant bytes (key ``name.weight``, uint8), embeddings / norm weights /
  biases as fp16 arrays.  One seed per tensor, derived from its name."""
  sd = {}
  for name, n_out, n_in in linear_names(cfg):
    kw = {} if scale_std is None else {"scale_std": scale_std}
    make = BLOCK_MAKERS.get(ggml_type) or (lambda o, i, rng, **k: random_blocks(ggml_type, o, i, rng, **k))
    sd[name + ".weight"] = make(n_out, n_in, np.random.default_rng(name_seed(name, seed)), **kw)
    if cfg.qkv_bias and name.split(".")[-1] in ("attn_q", "attn_k", "attn_v"):
      sd[name + ".bias"] = (np.random.default_rng(name_seed(name + ".bias", seed)).standard_normal(n_out, dtype=np.float32) * bias_std).astype(np.float16)
  rng = np.random.default_rng(name_seed("token_embd", seed))
  sd["token_embd.weight"] = (rng.standard_normal((cfg.vocab_size, cfg.dim), dtype=np.float32) * embd_std).astype(np.float16)
  for name in [f"blk.{i}.{n}" for i in range(cfg.num_blocks) for n in ("attn_norm", "ffn_norm")] + ["output_norm"]:
    rng = np.random.default_rng(name_seed(name, seed))
    sd[name + ".weight"] = (1.0 + 0.05 * rng.standard_normal(cfg.dim, dtype=np.float32)).astype(np.float16)
  return sd


class LazyDenseState:
  """Mapping view of `dense_model_raw` that makes each tensor when it is asked for, so a
  multi-GB model never sits in host memory as a whole."""
  def __init__(self, cfg, ggml_type: int = Q4_0, seed: int = 0, embd_std: float = 0.02, bias_std: float = 0.02, embd_vocab: int = 0,
               linear_seed: int = None, distinct_blocks: int = 0):
    """embd_vocab: rows of the embedding table when it differs from cfg.vocab_size (a tensor-parallel shard keeps the whole
    table but only a slice of the vocabulary head); linear_seed: seed of the Linear weights / biases only (per-rank shards
    differ, replicated tensors must not); distinct_blocks > 0: block i takes the values of block i % distinct_blocks (memoised), which
    bounds the host time of generating a very large model; every block still gets its own device memory."""
    self.distinct_blocks, self._memo = distinct_blocks, {}
    self.cfg, self.ggml_type, self.seed, self.embd_std, self.bias_std = cfg, ggml_type, seed, embd_std, bias_std
    self.embd_vocab, self.linear_seed = embd_vocab or cfg.vocab_size, seed if linear_seed is None else linear_seed
    self.shapes = {n: (o, i) for n, o, i in linear_names(cfg)}

  def __contains__(self, key) -> bool:
    if not isinstance(key, str) or "." not in key: return False
    name, kind = key.rsplit(".", 1)
    if kind == "bias": return self.cfg.qkv_bias and name in self.shapes and name.split(".")[-1] in ("attn_q", "attn_k", "attn_v")
    return kind == "weight" and (name in self.shapes or name == "token_embd" or name.endswith("_norm"))

  def __getitem__(self, key: str) -> np.ndarray:
    if self.distinct_blocks and key.startswith("blk."):
      _, i, rest = key.split(".", 2)
      src = f"blk.{int(i) % self.distinct_blocks}.{rest}"
      if src not in self._memo: self._memo[src] = self._make(src)
      return self._memo[src]
    return self._make(key)

  def _make(self, key: str) -> np.ndarray:
    name, kind = key.rsplit(".", 1)
    is_linear = (kind == "weight" and name in self.shapes) or kind == "bias"
    rng = np.random.default_rng(name_seed(name if kind == "weight" else key, self.linear_seed if is_linear else self.seed))
    if kind == "weight" and name in self.shapes: return BLOCK_MAKERS[self.ggml_type](*self.shapes[name], rng)
    if kind == "bias": return (rng.standard_normal(self.shapes[name][0], dtype=np.float32) * self.bias_std).astype(np.float16)
    if name == "token_embd": return (rng.standard_normal((self.embd_vocab, self.cfg.dim), dtype=np.float32) * self.embd_std).astype(np.float16)
    if name.endswith("_norm"): return (1.0 + 0.05 * rng.standard_normal(self.cfg.dim, dtype=np.float32)).astype(np.float16)
    raise KeyError(key)


# ---- GGUF container images of synthetic models (the file format of tinygrad/llm/gguf.py:132-149) ----
def _gguf_value(v) -> bytes:
  import struct
  if isinstance(v, bool): return struct.pack("<i?", 7, v)
  if isinstance(v, int): return struct.pack("<iI", 4, v) if 0 <= v < 2**32 else struct.pack("<iq", 11, v)
  if isinstance(v, float): return struct.pack("<if", 6, v)
  if isinstance(v, str): b = v.encode(); return struct.pack("<iQ", 8, len(b)) + b
  if isinstance(v, (list, tuple)):
    items = [_gguf_value(x) for x in v]
    typ = items[0][:4] if items else struct.pack("<i", 4)
    assert all(it[:4] == typ for it in items), "GGUF arrays hold one value type"
    return struct.pack("<i", 9) + typ + struct.pack("<Q", len(items)) + b"".join(it[4:] for it in items)
  raise TypeError(f"no GGUF value type for {type(v)}")


def write_gguf(kv: dict, tensors: list, version: int = 3) -> bytes:
  """kv: metadata; tensors: (name, shape outermost-first, ggml_type, raw bytes / array).  Returns the file image."""
  import struct
  align = kv.get("general.alignment", 32)
  head = b"GGUF" + struct.pack("<iqq", version, len(tensors), len(kv))
  for k, v in kv.items(): head += struct.pack("<Q", len(k.encode())) + k.encode() + _gguf_value(v)
  blobs, off = [], 0
  for name, shape, typ, data in tensors:
    raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1).tobytes()
    head += struct.pack("<Q", len(name.encode())) + name.encode() + struct.pack("<I", len(shape))
    head += b"".join(struct.pack("<Q", d) for d in reversed(shape)) + struct.pack("<iQ", typ, off)     # dims innermost-first
    pad = (-len(raw)) % align
    blobs.append(raw + b"\0" * pad)
    off += len(raw) + pad
  return head + b"\0" * ((-len(head)) % align) + b"".join(blobs)


def dense_model_gguf(cfg, ggml_type: int = Q4_0, seed: int = 0, arch: str = "llama", embd_std: float = 0.02, output: str = "same", mixed: dict = None,
                     embd_type: int = 1) -> bytes:
  """A random-init dense model as a GGUF file image.  output: "same" (head in ggml_type), "f16", "bf16", "f32", "q6_k", or "tied" (no output.weight).
  For arch "llama" the q/k rows are stored as given; the loader applies the family's RoPE row permutation.
  mixed: Linear short name ("attn_v", "ffn_down", "output", ...) -> GGML type for those Linears (random blocks of that format), as real
  files mix K-quants; embd_type: GGML type of token_embd (1 = F16; a block format: random blocks)."""
  sd = dense_model_raw(cfg, ggml_type, seed=seed, embd_std=embd_std)
  shapes = {n + ".weight": (o, i) for n, o, i in linear_names(cfg)}
  kv = {"general.architecture": arch, "general.alignment": 32, f"{arch}.context_length": cfg.max_context, f"{arch}.block_count": cfg.num_blocks,
        f"{arch}.embedding_length": cfg.dim, f"{arch}.feed_forward_length": cfg.hidden_dim, f"{arch}.attention.head_count": cfg.n_heads,
        f"{arch}.attention.head_count_kv": cfg.n_kv_heads, f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.norm_eps),
        f"{arch}.rope.freq_base": float(cfg.rope_theta), f"{arch}.rope.dimension_count": cfg.rope_dim,
        f"{arch}.attention.key_length": cfg.head_dim, f"{arch}.attention.value_length": cfg.head_dim,
        "tokenizer.ggml.tokens": [f"t{i}" for i in range(cfg.vocab_size)]}
  tensors = []
  for name, arr in sd.items():
    if name == "output.weight" and output != "same":
      if output == "tied": continue
      rng = np.random.default_rng(name_seed("output", seed))
      if output == "q6_k": arr, typ = q6_k_blocks(cfg.vocab_size, cfg.dim, rng), Q6_K
      elif output == "f32": arr, typ = rng.standard_normal((cfg.vocab_size, cfg.dim), dtype=np.float32) * 0.05, 0
      elif output == "bf16":      # bf16 bit patterns (type 30): the upper halves of random fp32 values
        arr, typ = ((rng.standard_normal((cfg.vocab_size, cfg.dim), dtype=np.float32) * 0.05).view(np.uint32) >> 16).astype(np.uint16), 30
      else: arr, typ = (rng.standard_normal((cfg.vocab_size, cfg.dim), dtype=np.float32) * 0.05).astype(np.float16), 1
      tensors.append((name, (cfg.vocab_size, cfg.dim), typ, arr))
    elif name in shapes:
      short = name[:-len(".weight")].split(".")[-1]
      if mixed and short in mixed:
        typ = mixed[short]
        arr = random_blocks(typ, *shapes[name], np.random.default_rng(name_seed(name, seed + 7)), scale_std=0.004 if typ in (12, 13) else (0.0008 if typ == 14 else 0.02))
        tensors.append((name, shapes[name], typ, arr))
      else: tensors.append((name, shapes[name], ggml_type, arr))
    elif name == "token_embd.weight" and embd_type != 1:
      arr = random_blocks(embd_type, cfg.vocab_size, cfg.dim, np.random.default_rng(name_seed(name, seed + 7)), scale_std=0.05)
      tensors.append((name, (cfg.vocab_size, cfg.dim), embd_type, arr))
    else: tensors.append((name, arr.shape, 1, arr))                  # fp16 embeddings / norms / biases
  return write_gguf(kv, tensors)
