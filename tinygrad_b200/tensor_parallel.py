"""Tensor-parallel decode: column-split QKV / gate / up / vocab head, row-split O / down, all-reduce over NCCL.

A rank's shard of a dense Transformer is itself a dense Transformer with fewer heads and a narrower FFN (same model
dim): `local_config` gives its shape, `shard_state_dict` cuts the reference-named tensors (raw GGUF blocks) for one rank
the way tinygrad shards them by axis (examples/llama3.py:233-243: attention and w1/w3 by output rows, wo/w2 by input
columns, output by vocabulary rows).  The row-split linears add residual / n_ranks, so the NCCL all-reduce of the shards
yields W x + residual; the vocabulary slices are all-gathered before the arg-max.  The collectives are the library's own by default
(mailboxes in peer memory, `PeerMailbox`); torch.distributed is the plumbing (process group, the IPC handles at set-up), and offers
NCCL as the alternative data path.
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


def share_buffer(group, buf) -> list:
  """Device pointers to every rank's counterpart of `buf` (a b200q_malloc allocation), as mapped into this process: the buffer's CUDA IPC
  handle goes to all ranks through the group's host channel and theirs are opened here.  Entry `group.rank` is the local pointer."""
  import ctypes
  from . import _lib
  from ._lib import check
  lib = _lib.load()
  handle = ctypes.create_string_buffer(64)
  check(lib.b200q_ipc_export(buf.ptr, handle))
  ptrs = []
  for r, h in enumerate(group.exchange(bytes(handle.raw))):
    if r == group.rank: ptrs.append(buf.ptr)
    else:
      p = ctypes.c_void_p()
      check(lib.b200q_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
      ptrs.append(int(p.value))
  return ptrs


class PeerMailbox:
  """A mailbox [n_slots][n] of fp32 words on every rank, each rank holding pointers to all of them (CUDA IPC): what the sharded
  GEMVs store their output rows into and `b200q_mailbox_reduce` consumes.  `targets` is the ctypes pointer array a GEMV takes."""
  def __init__(self, group: "TPGroup", n_slots: int, n: int):
    import ctypes
    from . import _lib
    from ._lib import check
    from .runtime import DeviceBuffer, synchronize
    lib = _lib.load()
    self.n_slots, self.n, self.group = n_slots, n, group
    self.local = DeviceBuffer(4 * n_slots * n)
    check(lib.b200q_memset(self.local.ptr, 0xFF, self.local.nbytes, None))      # every word empty
    synchronize()
    self.ptrs = share_buffer(group, self.local)
    self.targets = (ctypes.c_void_p * group.size)(*self.ptrs)
    group.barrier()                                  # nobody stores into a mailbox that is not yet filled with the empty pattern

  def reduce(self, out, residual=None, flags: int = 0, stream=None, spin_limit: int = 0) -> None:
    from . import _lib
    from .runtime import ptr_of, stream_ptr
    _lib.check(_lib.load().b200q_mailbox_reduce(self.local.ptr, self.n_slots, self.n, ptr_of(residual), ptr_of(out), spin_limit, flags, stream_ptr(stream)))


class TPGroup:
  """Rank bookkeeping + the collectives of tensor-parallel decode.  kind "peer" (default): the library's own mailboxes in peer memory,
  filled by the sharded GEMVs and summed by a small kernel -- no communication library in the data path; torch.distributed only carries
  the IPC handles at set-up.  kind "nccl": torch.distributed all-reduce / all-gather on NCCL, captured into the step's CUDA graph."""
  def __init__(self, ranks, kind: str = "peer"):
    assert kind in ("peer", "nccl")
    self.kind_id, self.ranks, self.dist, self.rank, self.size = kind, ranks, ranks.dist, ranks.rank, ranks.world
    self.kind = ("mailboxes in peer memory: sharded GEMVs store into every rank's mailbox over NVLink, one small kernel sums them (no library call)"
                 if kind == "peer" else "NCCL all-reduce per row-parallel linear (torch.distributed), captured into the step's CUDA graph")
    self.tstream = None
    if kind == "nccl":
      import torch
      self.torch = torch
      self.tstream = torch.cuda.Stream()          # every launch of the model and every NCCL call goes on this stream
      # NCCL sets up its connections at the first collective of each kind: do that now, never inside a stream capture
      warm, part = torch.zeros(1024, device="cuda"), torch.zeros(1024 // self.size, device="cuda")
      with torch.cuda.stream(self.tstream):
        self.dist.all_reduce(warm)
        self.dist.all_gather_into_tensor(warm, part)
      self.tstream.synchronize()

  def stream_ptr(self): return int(self.tstream.cuda_stream) if self.tstream is not None else None

  def exchange(self, blob: bytes) -> list:
    """Every rank's blob, by rank (host side, set-up only)."""
    if self.dist is None: return [blob]
    out = [None] * self.size
    self.dist.all_gather_object(out, blob)
    return out

  def barrier(self) -> None:
    if self.dist is not None: self.dist.barrier()

  def empty_f32(self, n: int):
    if self.kind_id == "nccl": return TorchBuffer(self.torch.zeros(n, dtype=self.torch.float32, device="cuda"))
    from .runtime import DeviceBuffer
    return DeviceBuffer.empty((n,), np.float32, zero=True)

  def all_reduce(self, buf: TorchBuffer) -> None:
    with self.torch.cuda.stream(self.tstream): self.dist.all_reduce(buf.t)

  def all_gather(self, full: TorchBuffer, part: TorchBuffer) -> None:
    with self.torch.cuda.stream(self.tstream): self.dist.all_gather_into_tensor(full.t, part.t)
