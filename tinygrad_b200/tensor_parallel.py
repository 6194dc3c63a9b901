"""Tensor-parallel decode: column-split QKV / gate / up / vocab head, row-split O / down, all-reduce over NCCL.

A rank's shard of a dense Transformer is itself a dense Transformer with fewer heads and a narrower FFN (same model
dim): `local_config` gives its shape, `shard_state_dict` cuts the reference-named tensors (raw GGUF blocks) for one rank
the way tinygrad shards them by axis (examples/llama3.py:233-243: attention and w1/w3 by output rows, wo/w2 by input
columns, output by vocabulary rows).  The row-split linears add residual / n_ranks, so the NCCL all-reduce of the shards
yields W x + residual; the vocabulary slices are all-gathered before the arg-max.  torch.distributed is the plumbing
(process group, NCCL calls, the two buffers NCCL touches); every kernel is the library's own.
"""
from dataclasses import replace
import numpy as np


def local_config(cfg, tp_size: int):
  assert cfg.n_heads % tp_size == 0 and cfg.n_kv_heads % tp_size == 0, "heads must split evenly (whole KV groups per rank)"
  assert cfg.hidden_dim % (tp_size * 128) == 0 and cfg.vocab_size % (tp_size * 16) == 0
  return replace(cfg, n_heads=cfg.n_heads // tp_size, n_kv_heads=cfg.n_kv_heads // tp_size, hidden_dim=cfg.hidden_dim // tp_size,
                 vocab_size=cfg.vocab_size // tp_size)


def _rows(raw: np.ndarray, n_out: int, lo: int, hi: int) -> np.ndarray:
  return np.ascontiguousarray(raw.reshape(n_out, -1)[lo:hi]).reshape(-1)


def _cols(raw: np.ndarray, n_out: int, n_in: int, blk_bytes: int, lo: int, hi: int) -> np.ndarray:
  return np.ascontiguousarray(raw.reshape(n_out, n_in // 32, blk_bytes)[:, lo // 32:hi // 32]).reshape(-1)


def shard_state_dict(sd: dict, cfg, rank: int, tp_size: int, blk_bytes: int = 18) -> dict:
  """The tensors of rank `rank`, named as in the full model.  `blk_bytes`: 18 for Q4_0, 34 for Q8_0."""
  qd, kvd, hid = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim, cfg.hidden_dim
  ql, kvl, hl, vl = qd // tp_size, kvd // tp_size, hid // tp_size, cfg.vocab_size // tp_size
  out = {}
  for k, v in sd.items():
    name = k.split(".")[-2] if "." in k else k
    if k.endswith(".weight") and v.dtype == np.uint8:
      if name == "attn_q": v = _rows(v, qd, rank * ql, (rank + 1) * ql)
      elif name in ("attn_k", "attn_v"): v = _rows(v, kvd, rank * kvl, (rank + 1) * kvl)
      elif name in ("ffn_gate", "ffn_up"): v = _rows(v, hid, rank * hl, (rank + 1) * hl)
      elif name == "attn_output": v = _cols(v, cfg.dim, qd, blk_bytes, rank * ql, (rank + 1) * ql)
      elif name == "ffn_down": v = _cols(v, cfg.dim, hid, blk_bytes, rank * hl, (rank + 1) * hl)
      elif name == "output": v = _rows(v, cfg.vocab_size, rank * vl, (rank + 1) * vl)
    elif k.endswith(".bias"):
      n = qd if name == "attn_q" else kvd
      v = v[rank * (n // tp_size):(rank + 1) * (n // tp_size)]
    out[k] = v
  return out


class TorchBuffer:
  """A torch CUDA tensor seen through the DeviceBuffer interface (the buffers NCCL reduces / gathers)."""
  def __init__(self, tensor):
    self.t, self.ptr, self.nbytes = tensor, tensor.data_ptr(), tensor.numel() * tensor.element_size()
    self.shape, self.dtype = tuple(tensor.shape), np.dtype(np.float32)
  def numpy(self, *a, **k): return self.t.detach().cpu().numpy()
  def zero_(self, stream=None): self.t.zero_()


class TPGroup:
  """Rank bookkeeping + the two collectives of tensor-parallel decode, on torch.distributed (backend nccl)."""
  def __init__(self, ranks):
    import torch
    self.torch, self.dist, self.rank, self.size = torch, ranks.dist, ranks.rank, ranks.world
    self.tstream = torch.cuda.Stream()          # every launch of the model and every NCCL call goes on this stream
    # NCCL sets up its connections at the first collective of each kind: do that now, never inside a stream capture
    warm, part = torch.zeros(1024, device="cuda"), torch.zeros(1024 // self.size, device="cuda")
    with torch.cuda.stream(self.tstream):
      self.dist.all_reduce(warm)
      self.dist.all_gather_into_tensor(warm, part)
    self.tstream.synchronize()

  kind = "NCCL all-reduce per row-parallel linear (torch.distributed), captured into the step's CUDA graph"

  def stream_ptr(self) -> int: return int(self.tstream.cuda_stream)

  def empty_f32(self, n: int) -> TorchBuffer:
    return TorchBuffer(self.torch.zeros(n, dtype=self.torch.float32, device="cuda"))

  def all_reduce(self, buf: TorchBuffer) -> None:
    with self.torch.cuda.stream(self.tstream): self.dist.all_reduce(buf.t)

  def all_gather(self, full: TorchBuffer, part: TorchBuffer) -> None:
    with self.torch.cuda.stream(self.tstream): self.dist.all_gather_into_tensor(full.t, part.t)
