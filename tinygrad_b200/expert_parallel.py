"""Expert-parallel MXFP8 MoE FFN: experts split contiguously over the ranks, tokens split over the ranks at the input.

The reference's grouped path on one device is route -> dispatch -> grouped_mx_gemm -> activation -> grouped_mx_gemm -> combine
(extra/gemm/moe_routing.py:109-131, examples/mlperf/models/gpt_oss.py:215-226).  Across ranks `dispatch` and `combine` become an
all-to-all each: a rank routes its own tokens over ALL experts, quantises every routed row once (E4M3 + E8M0, so the wire carries
33/32 bytes per value instead of 2), lays the rows out sorted by expert (= sorted by destination rank, experts being contiguous),
and exchanges them; the receiver regroups what it got by local expert (groups padded to 256 rows), runs the two grouped GEMMs on
its expert shard and sends the bf16 results back the same way; the sender combines them with its routing weights.
Every row's arithmetic is the single-GPU path's, so the result equals `MxMoE` on the concatenated tokens bit for bit.

`exchange_plan` is the host-side index arithmetic (pure numpy, tested on CPU); the payload exchange is torch.distributed
(`all_to_all_single` on NCCL; point-to-point sends elsewhere, for the CPU tests); all compute is in libb200q.so.
"""
from __future__ import annotations
import numpy as np

BLOCK_ROW = 256   # extra/gemm/moe_routing.py:4


def exchange_plan(counts: np.ndarray, rank: int) -> dict:
  """counts[s, e] = rows rank s routes to expert e (every rank holds the whole matrix after an all-gather).
  Experts are split contiguously: rank r owns experts r*E_l .. (r+1)*E_l-1.  Returns for `rank`:
    send_rows[r]   rows this rank sends to rank r (its compact expert-sorted buffer is cut at these sizes)
    recv_rows[s]   rows it receives from rank s (arrival order: by source rank, inside a source by expert)
    off_local      [E_l+1] group starts of the local expert groups, each padded to 256 rows
    place          [sum(recv_rows)] row of the grouped buffer for every received row (a stable placement: source-major inside an expert)
    m_local        rows of the grouped buffer (= off_local[-1])"""
  counts = np.asarray(counts, dtype=np.int64)
  n_ranks, n_experts = counts.shape
  assert n_experts % n_ranks == 0, "experts must split evenly over the ranks"
  e_l = n_experts // n_ranks
  send_rows = counts[rank].reshape(n_ranks, e_l).sum(1)
  mine = counts[:, rank * e_l:(rank + 1) * e_l]                  # [source, local expert]
  recv_rows = mine.sum(1)
  tot = mine.sum(0)
  off_local = np.concatenate([[0], np.cumsum((tot + BLOCK_ROW - 1) // BLOCK_ROW * BLOCK_ROW)])
  before = np.cumsum(mine, axis=0) - mine                         # rows of the same expert from earlier sources
  place = np.empty(int(recv_rows.sum()), dtype=np.int32)
  p = 0
  for s in range(n_ranks):
    for e in range(e_l):
      c = int(mine[s, e])
      place[p:p + c] = off_local[e] + before[s, e] + np.arange(c)
      p += c
  return dict(send_rows=send_rows.astype(np.int64), recv_rows=recv_rows.astype(np.int64), off_local=off_local.astype(np.int32), place=place,
              m_local=int(off_local[-1]))


def m_local_max(n_tokens_total: int, n_experts_local: int, k: int) -> int:
  """Upper bound of the grouped rows one rank can receive (all routed rows of all ranks on its experts), m_max_for of
  extra/gemm/moe_routing.py:89-90 for its shard."""
  return (-(-n_tokens_total * k // BLOCK_ROW) + n_experts_local) * BLOCK_ROW


def all_to_all_rows(dist, torch, send, send_rows, recv, recv_rows) -> None:
  """Rows of `send` (cut at send_rows) to every rank, rows from every rank into `recv` (cut at recv_rows).  torch tensors [rows, width]."""
  if dist.get_backend() == "nccl":
    dist.all_to_all_single(recv, send, output_split_sizes=[int(x) for x in recv_rows], input_split_sizes=[int(x) for x in send_rows])
    return
  rank, ops, so, ro = dist.get_rank(), [], np.concatenate([[0], np.cumsum(send_rows)]), np.concatenate([[0], np.cumsum(recv_rows)])
  for r in range(dist.get_world_size()):
    if r == rank: recv[ro[r]:ro[r + 1]] = send[so[r]:so[r + 1]]
    else:
      if send_rows[r]: ops.append(dist.P2POp(dist.isend, send[so[r]:so[r + 1]].contiguous(), r))
      if recv_rows[r]: ops.append(dist.P2POp(dist.irecv, recv[ro[r]:ro[r + 1]], r))
  if ops:
    for w in dist.batch_isend_irecv(ops): w.wait()


class ExpertParallelMoE:
  """One rank's part of an expert-parallel MXFP8 MoE FFN.  w_gate / w_up: (E_l, F, D), w_down: (E_l, D, F) fp32: THIS rank's experts
  (rank r owns experts r*E_l ..).  Call it with this rank's tokens (T_l, D) bf16 and their router logits (T_l, E) fp32."""
  def __init__(self, ranks, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray, n_experts: int, k: int, n_tokens_total: int, mode: int = 1):
    import torch
    from . import moe
    from .runtime import DeviceBuffer
    self.torch, self.dist, self.rank, self.size = torch, ranks.dist, ranks.rank, ranks.world
    self.E, self.k, self.mode = n_experts, k, mode
    self.E_l, self.F, self.D = w_gate.shape
    assert self.E_l * self.size == n_experts
    self.local = moe.MxMoE(w_gate, w_up, w_down, k, mode)          # holds the quantised expert shard; its own routing is not used
    self.m_max = m_local_max(n_tokens_total, self.E_l, k)
    dev = "cuda"
    u8 = torch.uint8
    self.recv_q, self.recv_e8 = torch.empty((self.m_max, self.D), dtype=u8, device=dev), torch.empty((self.m_max, self.D // 32), dtype=u8, device=dev)
    self.a_q, self.a_e8 = torch.zeros((self.m_max, self.D), dtype=u8, device=dev), torch.zeros((self.m_max, self.D // 32), dtype=u8, device=dev)
    self.h = torch.zeros((self.m_max, 4 * self.F), dtype=u8, device=dev)                 # bf16 values as bytes (NCCL has no 16-bit integer type)
    self.act_q, self.act_e8 = torch.empty((self.m_max, self.F), dtype=u8, device=dev), torch.empty((self.m_max, self.F // 32), dtype=u8, device=dev)
    self.y = torch.zeros((self.m_max, 2 * self.D), dtype=u8, device=dev)
    self.y_send = torch.empty((self.m_max, 2 * self.D), dtype=u8, device=dev)
    self._per_T = {}

  exchange_kind = "host-planned: counts all-gather, two all_to_all_single (NCCL) each way"

  def timed(self, x_bf16, logits, n_tokens: int, reps: int) -> float:
    """Milliseconds per call over `reps` calls, CUDA events on the stream the layer runs on (the default stream)."""
    from .runtime import Event
    e0, e1 = Event(), Event()
    e0.record(None)
    for _ in range(reps): self(x_bf16, logits, n_tokens)
    e1.record(None)
    e1.synchronize()
    return e0.elapsed_ms(e1) / reps

  def _buffers(self, T: int):
    b = self._per_T.get(T)
    if b is None:
      from . import _lib
      from .runtime import DeviceBuffer
      t, n = self.torch, T * self.k
      b = dict(topi=DeviceBuffer.empty((T, self.k), np.int32), w=DeviceBuffer.empty((T, self.k), np.float32), dest=DeviceBuffer.empty((n,), np.int32),
               off=DeviceBuffer.empty((self.E + 1,), np.int32), scratch=DeviceBuffer(_lib.load().b200q_moe_route_scratch_bytes(T, self.E, self.k)),
               counts=t.zeros(self.E, dtype=t.int32, device="cuda"), send_q=t.empty((n, self.D), dtype=t.uint8, device="cuda"),
               send_e8=t.empty((n, self.D // 32), dtype=t.uint8, device="cuda"), y_back=t.empty((n, 2 * self.D), dtype=t.uint8, device="cuda"),
               out=DeviceBuffer.empty((T, self.D), np.uint16))
      self._per_T[T] = b
    return b

  def __call__(self, x_bf16, logits, n_tokens: int):
    """-> DeviceBuffer (T_l, D) bf16.  Runs on the default stream; the host reads the routing counts (the exchange sizes) in between."""
    from . import _lib
    from ._lib import check, BF16
    from .runtime import ptr_of
    lib, t, dist, T = _lib.load(), self.torch, self.dist, n_tokens
    b = self._buffers(T)
    # 1. route over all experts, compact expert-sorted order (= sorted by destination rank); quantise every routed row into it
    check(lib.b200q_moe_route_pad(ptr_of(logits), T, self.E, self.k, self.mode, 1, b["topi"].ptr, b["w"].ptr, b["dest"].ptr, b["off"].ptr,
                                  b["counts"].data_ptr(), b["scratch"].ptr, None))
    check(lib.b200q_quantize_mxfp8(ptr_of(x_bf16), BF16, T, self.D, b["dest"].ptr, self.k, b["send_q"].data_ptr(), b["send_e8"].data_ptr(), None))
    # 2. everybody's per-expert counts -> the exchange sizes and the receiver's grouping
    t.cuda.synchronize()
    allc = [t.empty_like(b["counts"]) for _ in range(self.size)]
    dist.all_gather(allc, b["counts"])
    plan = exchange_plan(np.stack([c.cpu().numpy() for c in allc]), self.rank)
    n_recv = int(plan["recv_rows"].sum())
    assert plan["m_local"] <= self.m_max
    # 3. dispatch across ranks: the quantised rows and their scale bytes
    all_to_all_rows(dist, t, b["send_q"], plan["send_rows"], self.recv_q[:n_recv], plan["recv_rows"])
    all_to_all_rows(dist, t, b["send_e8"], plan["send_rows"], self.recv_e8[:n_recv], plan["recv_rows"])
    # 4. regroup by local expert (256-padded groups, zero rows in the padding), expert FFN on the shard
    place, off_l = t.from_numpy(plan["place"]).cuda(), t.from_numpy(plan["off_local"]).cuda()
    self.a_q.zero_(); self.a_e8.zero_()
    check(lib.b200q_permute_rows(self.recv_q.data_ptr(), place.data_ptr(), n_recv, self.D, self.a_q.data_ptr(), 0, None))
    check(lib.b200q_permute_rows(self.recv_e8.data_ptr(), place.data_ptr(), n_recv, self.D // 32, self.a_e8.data_ptr(), 0, None))
    m, loc = self.local, plan["m_local"]
    if loc:
      if m.fused:
        check(lib.b200q_grouped_mxfp8_gemm_swiglu(self.a_q.data_ptr(), self.a_e8.data_ptr(), m.gu_q.ptr, m.gu_e8.ptr, off_l.data_ptr(), self.E_l, loc,
                                                  2 * self.F, self.D, self.act_q.data_ptr(), self.act_e8.data_ptr(), None))
      else:
        check(lib.b200q_grouped_mxfp8_gemm(self.a_q.data_ptr(), self.a_e8.data_ptr(), m.gu_q.ptr, m.gu_e8.ptr, off_l.data_ptr(), self.E_l, loc, 2 * self.F,
                                           self.D, self.h.data_ptr(), None))
        check(lib.b200q_swiglu_quantize_mxfp8(self.h.data_ptr(), loc, None, self.F, self.act_q.data_ptr(), self.act_e8.data_ptr(), None))
      check(lib.b200q_grouped_mxfp8_gemm(self.act_q.data_ptr(), self.act_e8.data_ptr(), m.dn_q.ptr, m.dn_e8.ptr, off_l.data_ptr(), self.E_l, loc, self.D,
                                         self.F, self.y.data_ptr(), None))
    # 5. results back in arrival order, combine on the rank that owns the tokens
    check(lib.b200q_permute_rows(self.y.data_ptr(), place.data_ptr(), n_recv, 2 * self.D, self.y_send.data_ptr(), 1, None))
    t.cuda.synchronize()
    all_to_all_rows(dist, t, self.y_send[:n_recv], plan["recv_rows"], b["y_back"], plan["send_rows"])
    check(lib.b200q_moe_combine(b["y_back"].data_ptr(), b["dest"].ptr, b["w"].ptr, T, self.k, self.D, b["out"].ptr, None))
    t.cuda.synchronize()
    self.last_plan = plan
    return b["out"]


class PeerExpertParallelMoE:
  """One rank's part of an expert-parallel MXFP8 MoE FFN whose exchange runs over peer memory and is planned on the device
  (csrc/ep.cu): no communication library, no host read and no synchronisation inside a call -- a call enqueues kernels only.
  Weights as `ExpertParallelMoE`.  `group` gives rank / size and a host channel for the set-up (`TPGroup`, or anything with
  rank, size, exchange(blob) and barrier()); `connect()` maps every rank's buffers into this process over CUDA IPC, or takes the
  pointer tables directly (ranks that live in one process, as in the one-GPU tests)."""
  SHARED = ("counts_all", "a_q", "a_e8", "y", "flags")
  exchange_kind = "device-planned over peer memory: counts mailbox, remote dispatch-quantise stores, flags, pull-combine (no library call, no host read)"

  def __init__(self, group, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray, n_experts: int, k: int, n_tokens_total: int, mode: int = 1):
    from . import moe, _lib
    from ._lib import check
    from .runtime import DeviceBuffer, synchronize
    self.group, self.rank, self.size = group, group.rank, group.size
    self.E, self.k, self.mode = n_experts, k, mode
    self.E_l, self.F, self.D = w_gate.shape
    assert self.E_l * self.size == n_experts and self.D % 256 == 0
    self.local = moe.MxMoE(w_gate, w_up, w_down, k, mode)          # holds the quantised expert shard; its own routing is not used
    self.m_max = m_local_max(n_tokens_total, self.E_l, k)
    m = self.m_max
    self.buf = dict(counts_all=DeviceBuffer(4 * self.size * n_experts), a_q=DeviceBuffer.empty((m, self.D), np.uint8, zero=True),
                    a_e8=DeviceBuffer.empty((m, self.D // 32), np.uint8, zero=True), y=DeviceBuffer.empty((m, self.D), np.uint16, zero=True),
                    flags=DeviceBuffer.empty((2, self.size), np.uint32, zero=True))
    check(_lib.load().b200q_memset(self.buf["counts_all"].ptr, 0xFF, self.buf["counts_all"].nbytes, None))
    self.h = DeviceBuffer.empty((m, 2 * self.F), np.uint16, zero=True)
    self.act_q, self.act_e8 = DeviceBuffer.empty((m, self.F), np.uint8, zero=True), DeviceBuffer.empty((m, self.F // 32), np.uint8, zero=True)
    self.send_base, self.off_local = DeviceBuffer.empty((n_experts,), np.int32, zero=True), DeviceBuffer.empty((self.E_l + 1,), np.int32, zero=True)
    self.scratch = DeviceBuffer.empty((1,), np.uint32, zero=True)
    synchronize()
    self._per_T, self.tables = {}, None

  def connect(self, tables: dict | None = None) -> None:
    """tables: name -> list of device pointers by rank, for every name of SHARED; None = exchange CUDA IPC handles through the group."""
    import ctypes
    if tables is None:
      from .tensor_parallel import share_buffer
      tables = {name: share_buffer(self.group, self.buf[name]) for name in self.SHARED}
      self.group.barrier()                       # nobody stores into buffers that are not initialised yet
    self.tables = {name: (ctypes.c_void_p * self.size)(*tables[name]) for name in self.SHARED}

  def _args(self, T: int):
    b = self._per_T.get(T)
    if b is None:
      from . import _lib
      from .runtime import DeviceBuffer
      assert self.tables is not None, "connect() first"
      n = T * self.k
      b = dict(topi=DeviceBuffer.empty((T, self.k), np.int32), w=DeviceBuffer.empty((T, self.k), np.float32), dest=DeviceBuffer.empty((n,), np.int32),
               off=DeviceBuffer.empty((self.E + 1,), np.int32), counts=DeviceBuffer.empty((self.E,), np.int32, zero=True),
               rscratch=DeviceBuffer(_lib.load().b200q_moe_route_scratch_bytes(T, self.E, self.k)), remote_row=DeviceBuffer.empty((n,), np.int32, zero=True),
               out=DeviceBuffer.empty((T, self.D), np.uint16))
      t = self.tables
      b["args"] = _lib.EpArgs(n_ranks=self.size, rank=self.rank, n_experts=self.E, k=self.k, d_model=self.D, n_tokens=T, m_max=self.m_max,
                              topi=b["topi"].ptr, dest=b["dest"].ptr, off=b["off"].ptr, counts=b["counts"].ptr, counts_all=t["counts_all"], a_q=t["a_q"],
                              a_e8=t["a_e8"], y=t["y"], flags=t["flags"], send_base=self.send_base.ptr, off_local=self.off_local.ptr,
                              remote_row=b["remote_row"].ptr, scratch=self.scratch.ptr)
      self._per_T[T] = b
    return b

  # The four stretches of a call between which another rank's progress is needed.  A rank runs them back to back on one stream; ranks
  # that share a GPU (tests) run stretch i for every rank before stretch i + 1, so that no kernel ever waits for a launch behind it.
  def route_publish(self, logits, T: int, stream=None) -> None:
    from . import _lib
    from ._lib import check
    from .runtime import ptr_of, stream_ptr
    lib, s, b = _lib.load(), stream_ptr(stream), self._args(T)
    check(lib.b200q_moe_route_pad(ptr_of(logits), T, self.E, self.k, self.mode, 1, b["topi"].ptr, b["w"].ptr, b["dest"].ptr, b["off"].ptr, b["counts"].ptr,
                                  b["rscratch"].ptr, s))
    check(lib.b200q_ep_publish_counts(b["args"], s))

  def plan_dispatch(self, x_bf16, T: int, stream=None) -> None:
    from . import _lib
    from ._lib import check
    from .runtime import ptr_of, stream_ptr
    lib, s, b = _lib.load(), stream_ptr(stream), self._args(T)
    check(lib.b200q_ep_plan(b["args"], s))
    check(lib.b200q_ep_dispatch(b["args"], ptr_of(x_bf16), s))

  def experts_signal(self, T: int, stream=None, spin_limit: int = 0) -> None:
    from . import _lib
    from ._lib import check
    from .runtime import stream_ptr
    lib, s, b, m, loc = _lib.load(), stream_ptr(stream), self._args(T), self.local, self.m_max
    a_q, a_e8, y, off_l = self.buf["a_q"].ptr, self.buf["a_e8"].ptr, self.buf["y"].ptr, self.off_local.ptr
    check(lib.b200q_ep_wait(b["args"], 0, spin_limit, s))
    if m.fused:
      check(lib.b200q_grouped_mxfp8_gemm_swiglu(a_q, a_e8, m.gu_q.ptr, m.gu_e8.ptr, off_l, self.E_l, loc, 2 * self.F, self.D, self.act_q.ptr, self.act_e8.ptr, s))
    else:
      check(lib.b200q_grouped_mxfp8_gemm(a_q, a_e8, m.gu_q.ptr, m.gu_e8.ptr, off_l, self.E_l, loc, 2 * self.F, self.D, self.h.ptr, s))
      check(lib.b200q_swiglu_quantize_mxfp8(self.h.ptr, loc, off_l + 4 * self.E_l, self.F, self.act_q.ptr, self.act_e8.ptr, s))
    check(lib.b200q_grouped_mxfp8_gemm(self.act_q.ptr, self.act_e8.ptr, m.dn_q.ptr, m.dn_e8.ptr, off_l, self.E_l, loc, self.D, self.F, y, s))
    check(lib.b200q_ep_signal_results(b["args"], s))

  def combine(self, T: int, stream=None, spin_limit: int = 0):
    from . import _lib
    from ._lib import check
    from .runtime import stream_ptr
    lib, s, b = _lib.load(), stream_ptr(stream), self._args(T)
    check(lib.b200q_ep_wait(b["args"], 1, spin_limit, s))
    check(lib.b200q_ep_combine(b["args"], b["w"].ptr, b["out"].ptr, s))
    return b["out"]

  def __call__(self, x_bf16, logits, n_tokens: int, stream=None):
    """-> DeviceBuffer (T_l, D) bf16, enqueued on `stream`; nothing is synchronised."""
    self.route_publish(logits, n_tokens, stream)
    self.plan_dispatch(x_bf16, n_tokens, stream)
    self.experts_signal(n_tokens, stream)
    return self.combine(n_tokens, stream)

  def timed(self, x_bf16, logits, n_tokens: int, reps: int) -> float:
    """Milliseconds per call over `reps` calls, CUDA events on the stream the layer runs on (the default stream)."""
    from .runtime import Event
    e0, e1 = Event(), Event()
    e0.record(None)
    for _ in range(reps): self(x_bf16, logits, n_tokens)
    e1.record(None)
    e1.synchronize()
    return e0.elapsed_ms(e1) / reps
