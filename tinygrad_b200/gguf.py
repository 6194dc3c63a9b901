"""GGUF container reader: host-side mirror of `gguf_load` (tinygrad/llm/gguf.py:132-176).

`gguf_load(path_or_bytes)` returns `(kv_data, tensors)` like the reference, except that a tensor is not a lazy
dequantisation expression but a `GGUFTensor`: its shape in the reference's order (GGUF stores dims innermost-first,
gguf.py:148 reverses them), its GGML type and a zero-copy view of its raw block bytes, which is what the device-side
`repack` / `dequantize` take.  `transformer_from_gguf` is `Transformer.from_gguf` (tinygrad/llm/model.py:369-452) for the
dense llama / qwen2 families: same metadata keys, same RoPE row permutation, same output.weight tying.
"""
from __future__ import annotations
import io, mmap, pathlib, re, struct
from dataclasses import dataclass
import numpy as np

# (elements per block, bytes per block) of the tensor types this path handles (gguf.py:20-21,25-27); other types parse
# (so that a file can be listed) but cannot be sized here and raise like the reference's ggml_data_to_tensor does
GGML_SIZES = {0: (1, 4), 1: (1, 2), 30: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 12: (256, 144), 13: (256, 176),
              14: (256, 210)}
GGML_NAMES = {0: "F32", 1: "F16", 30: "BF16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}


@dataclass
class GGUFTensor:
  name: str
  shape: tuple          # outermost first, as the reference reshapes it
  ggml_type: int
  data: np.ndarray      # uint8 view of the raw bytes inside the file buffer

  @property
  def n_elems(self) -> int: return int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1

  def rows(self) -> np.ndarray:
    """Raw bytes as [shape[0], bytes per row] (blocks run along the innermost dim)."""
    return self.data.reshape(self.shape[0], -1) if len(self.shape) > 1 else self.data.reshape(1, -1)

  def numpy(self) -> np.ndarray:
    """Values of an unquantised tensor (F32 / F16; BF16 widened to fp32)."""
    if self.ggml_type == 0: return self.data.view(np.float32).reshape(self.shape)
    if self.ggml_type == 1: return self.data.view(np.float16).reshape(self.shape)
    if self.ggml_type == 30: return (self.data.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(self.shape)
    raise ValueError(f"tensor {self.name} is quantised ({GGML_NAMES.get(self.ggml_type, self.ggml_type)}): dequantise it on the device")


class _Reader:
  def __init__(self, buf): self.buf, self.pos = memoryview(buf).cast("B"), 0
  def take(self, fmt: str, n: int):
    if self.pos + n > len(self.buf): raise ValueError("Invalid GGUF format!")
    v = struct.unpack_from("<" + fmt, self.buf, self.pos)[0]
    self.pos += n
    return v
  def string(self) -> str:
    n = self.take("Q", 8)
    if self.pos + n > len(self.buf): raise ValueError("Invalid GGUF format!")
    s = str(bytes(self.buf[self.pos:self.pos + n]), "utf-8")
    self.pos += n
    return s
  def value(self, typ: int):
    if typ == 8: return self.string()
    if typ == 9:
      item, n = self.take("i", 4), self.take("Q", 8)
      return [self.value(item) for _ in range(n)]
    if typ not in _SCALARS: raise ValueError(f"unknown GGUF metadata value type {typ}")
    return self.take(*_SCALARS[typ])


# metadata value types of the GGUF spec, as the reference's `readers` table (gguf.py:125-129)
_SCALARS = {0: ("c", 1), 1: ("b", 1), 2: ("H", 2), 3: ("h", 2), 4: ("I", 4), 5: ("i", 4), 6: ("f", 4), 7: ("?", 1), 10: ("Q", 8), 11: ("q", 8),
            12: ("d", 8)}


def gguf_parse(buf) -> tuple:
  """bytes-like -> (kv_data, {name: GGUFTensor}); raises ValueError("Invalid GGUF format!") like gguf.py:136."""
  r = _Reader(buf)
  if len(r.buf) < 24 or bytes(r.buf[:4]) != b"GGUF": raise ValueError("Invalid GGUF format!")
  r.pos = 4
  version, n_tensors, n_kv = r.take("i", 4), r.take("q", 8), r.take("q", 8)
  if version not in (2, 3): raise ValueError("Invalid GGUF format!")
  kv = {}
  for _ in range(n_kv):
    k, typ = r.string(), r.take("i", 4)
    kv[k] = r.value(typ)
  infos = []
  for _ in range(n_tensors):
    name = r.string()
    dims = tuple(r.take("Q", 8) for _ in range(r.take("I", 4)))
    infos.append((name, dims, r.take("i", 4), r.take("Q", 8)))
  align = kv.get("general.alignment", 32)
  data_start = (r.pos + align - 1) // align * align
  raw = np.frombuffer(r.buf, dtype=np.uint8)
  tensors = {}
  for name, dims, typ, off in infos:
    n = int(np.prod(dims, dtype=np.int64)) if dims else 1
    if typ not in GGML_SIZES: raise ValueError(f"GGML type '{typ}' is not supported!")      # gguf.py:119
    nel, nby = GGML_SIZES[typ]
    if n % nel: raise ValueError(f"tensor {name}: {n} elements is not a whole number of {GGML_NAMES[typ]} blocks")
    nbytes = n // nel * nby
    if data_start + off + nbytes > raw.size: raise ValueError("Invalid GGUF format!")
    tensors[name] = GGUFTensor(name, tuple(reversed(dims)), typ, raw[data_start + off:data_start + off + nbytes])
  return kv, tensors


def _split_paths(path: pathlib.Path, kv: dict) -> list:
  """Multi-part files (gguf.py:151-155): <base>-00001-of-NNNNN.gguf lists all parts; loading starts from the first."""
  total = kv.get("split.count", 1)
  if total <= 1: return [path]
  if kv.get("split.no", 0) != 0: raise ValueError(f"multi-part GGUF must be loaded from the first split, got split.no={kv['split.no']}")
  m = re.match(r"^(.*)-00001-of-\d{5}\.gguf$", str(path))
  if not m: raise ValueError(f"first split path must end with -00001-of-NNNNN.gguf: {path}")
  return [pathlib.Path(f"{m.group(1)}-{i:05d}-of-{total:05d}.gguf") for i in range(1, total + 1)]


def _map_file(path) -> mmap.mmap:
  with open(path, "rb") as f: return mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)


def gguf_load(fn) -> tuple:
  """Path or bytes-like -> (kv_data, tensors); multi-part splits are merged when loaded by path (gguf.py:157-176)."""
  by_path = isinstance(fn, (str, pathlib.Path))
  kv, sd = gguf_parse(_map_file(fn) if by_path else fn)
  if kv.get("split.count", 1) <= 1: return kv, sd
  if not by_path: raise ValueError("multi-part GGUF requires a path argument (got bytes)")
  for pp in _split_paths(pathlib.Path(fn), kv)[1:]: sd.update(gguf_parse(_map_file(pp))[1])
  return kv, sd


def _permute_rope_rows(rows: np.ndarray, n_heads: int, prefix: int = 0) -> np.ndarray:
  """Interleaved -> half-split RoPE layout on the ROWS of a q/k weight (model.py:405-413): inside each head, rows
  (2i, 2i+1) after the first `prefix` become (i, i + half).  A row of a quantised weight is a run of whole blocks, so the
  permutation applies to the raw bytes unchanged."""
  per = rows.shape[0] // n_heads
  w = rows.reshape(n_heads, per, -1)
  rot = w[:, prefix:].reshape(n_heads, (per - prefix) // 2, 2, -1).transpose(0, 2, 1, 3).reshape(n_heads, per - prefix, -1)
  return np.ascontiguousarray(np.concatenate([w[:, :prefix], rot], axis=1).reshape(rows.shape[0], -1))


SUPPORTED_ARCH = ("llama", "qwen2")


def transformer_from_gguf(fn, max_context: int = None, kv_dtype: str = "float16", **kwargs):
  """-> (Transformer, kv_data), the dense decoder families this path covers (model.py:369-452).  Files whose block Linears are all
  Q4_0 or all Q8_0 run the fused dequant kernels; files that mix block formats or use Q4_1 / Q5_0 / Q5_1 / Q4_K / Q5_K / Q6_K / F16 /
  BF16 / F32 Linears (what the reference's model zoo mostly ships, tinygrad/llm/cli.py:76-94) run on dense fp16 blocks, every weight
  dequantised once on the device.  The output head may be of any of these types.  kv_dtype is the
  cache dtype (the reference takes it from DEFAULT_FLOAT, model.py:202-203); other keyword arguments go to Transformer."""
  from .model import Transformer, TransformerConfig
  kv, t = gguf_load(fn)
  arch = kv["general.architecture"]
  if arch not in SUPPORTED_ARCH: raise NotImplementedError(f"architecture '{arch}' is outside this path (dense {SUPPORTED_ARCH} only)")
  ctx = kv[f"{arch}.context_length"]
  max_context = min(max_context, ctx) if max_context is not None else ctx
  n_heads, n_kv = kv[f"{arch}.attention.head_count"], kv[f"{arch}.attention.head_count_kv"]
  head_dim = kv.get(f"{arch}.attention.key_length", kv[f"{arch}.embedding_length"] // n_heads)
  rope_dim = kv.get(f"{arch}.rope.dimension_count", head_dim)
  cfg = TransformerConfig(num_blocks=kv[f"{arch}.block_count"], dim=kv[f"{arch}.embedding_length"], hidden_dim=kv[f"{arch}.feed_forward_length"],
                          n_heads=n_heads, n_kv_heads=n_kv, norm_eps=kv[f"{arch}.attention.layer_norm_rms_epsilon"],
                          vocab_size=len(kv["tokenizer.ggml.tokens"]), head_dim=head_dim, rope_theta=kv[f"{arch}.rope.freq_base"], rope_dim=rope_dim,
                          v_head_dim=kv.get(f"{arch}.attention.value_length", head_dim), max_context=max_context,
                          qkv_bias="blk.0.attn_q.bias" in t, kv_dtype=kv_dtype)
  lin_names = [f"blk.{i}.{n}.weight" for i in range(cfg.num_blocks) for n in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")]
  lin_types = {n: t[n].ggml_type for n in lin_names}
  unknown = sorted({GGML_NAMES.get(x, x) for x in lin_types.values() if x not in GGML_SIZES})
  if unknown: raise NotImplementedError(f"block Linears in formats without a dequantiser here: {unknown}")
  # one fused type for every block Linear -> the fused kernels; anything else (mixed files, K-quants, F16 models) -> dense fp16 blocks
  kinds = set(lin_types.values())
  block_type = kinds.pop() if len(kinds) == 1 and kinds <= {2, 8} else max(set(lin_types.values()), key=list(lin_types.values()).count)
  quantised = {k for k, (nel, _) in GGML_SIZES.items() if nel > 1}
  sd = {}
  for name, g in t.items():
    if name.endswith(".weight") and g.ggml_type in quantised and len(g.shape) == 2:
      rows = g.rows()
      if arch == "llama" and "attn_q.weight" in name: rows = _permute_rope_rows(rows, n_heads, head_dim - rope_dim)
      elif arch == "llama" and "attn_k.weight" in name: rows = _permute_rope_rows(rows, n_kv)
      sd[name] = rows.reshape(-1)
    elif g.ggml_type in (0, 1, 30):
      a = g.numpy()
      if arch == "llama" and len(g.shape) == 2 and "attn_q.weight" in name: a = _permute_rope_rows(a, n_heads, head_dim - rope_dim)
      elif arch == "llama" and len(g.shape) == 2 and "attn_k.weight" in name: a = _permute_rope_rows(a, n_kv)
      sd[name] = a
    else:
      sd[name] = g
  # models without output.weight tie it to token_embd.weight (model.py:378-379)
  out_t = t.get("output.weight", t["token_embd.weight"])
  emb = t["token_embd.weight"]
  if emb.ggml_type not in (0, 1, 30):
    from .quant import dequantize
    sd["token_embd.weight"] = dequantize(np.ascontiguousarray(emb.data), emb.n_elems, emb.ggml_type, np.float16).numpy().reshape(emb.shape)
  if "output.weight" not in t: sd["output.weight"] = np.ascontiguousarray(out_t.data) if out_t.ggml_type in quantised else out_t.numpy()
  model = Transformer(cfg, sd, ggml_type=block_type, output_type=out_t.ggml_type, linear_types=lin_types, **kwargs)
  return model, kv
