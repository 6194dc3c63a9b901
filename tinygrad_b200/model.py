"""The quantized-LLM decode path on one B200: host-side mirror of tinygrad/llm/model.py.

`TransformerConfig` carries the reference's field names (model.py:52-83);
`Transformer.generate(tokens)` yields greedy tokens like the reference's
`generate` at temperature 0 (model.py:464-484).  The forward pass of one token is
five fused launches per block (norm+QKV GEMV, attention, O GEMV+residual,
norm+gate/up GEMV+SwiGLU, down GEMV+residual) plus embedding, head GEMV and
arg-max, chained with programmatic dependent launch and replayed as one CUDA graph.
"""
from __future__ import annotations
from dataclasses import dataclass
import numpy as np
from . import _lib, quant
from ._lib import check, F32, F16, EPI_LINEAR, EPI_SILU_MUL, FLAG_PDL
from .runtime import DeviceBuffer, Stream, Graph, Event, synchronize as runtime_sync
import ctypes, os

# batched decode: attention of all sequences in one launch of the one-token kernel instead of the prompt-pass kernels with one query row
# per CTA (measured 1.4 % slower at 8 sequences x 130 positions: off unless asked for)
SEQ_ATTENTION = os.environ.get("B200Q_SEQ_ATTENTION", "0") == "1"


@dataclass(frozen=True)
class TransformerConfig:           # field names of tinygrad/llm/model.py:52-83 (dense GQA subset)
  num_blocks: int
  dim: int
  hidden_dim: int
  n_heads: int
  n_kv_heads: int
  norm_eps: float
  vocab_size: int
  head_dim: int
  rope_theta: float
  rope_dim: int
  v_head_dim: int = 0
  max_context: int = 0
  qkv_bias: bool = False
  kv_dtype: str = "float16"        # the cache dtype; the reference takes it from DEFAULT_FLOAT (model.py:202-203)
  num_experts: int = 0             # > 0: every block's FFN is a routed mixture of experts (model.py:94-98,110-135) with MXFP8 expert weights
  num_experts_per_tok: int = 0
  norm_topk_prob: bool = False
  expert_gating_func: str = "softmax"   # "softmax" | "sigmoid" | "softmax_weight" | "sqrt_softplus" (ExpertGating, model.py:9-13)
  routed_scaling_factor: float = 1.0
  shared_expert_dim: int = 0            # > 0: a dense SwiGLU expert every token also goes through (model.py:99-103,131-134)
  shared_expert_gate: bool = True       # its output is scaled by sigmoid(x . ffn_gate_inp_shexp) when that tensor is present
  expert_bias: bool = False             # exp_probs_b: a bias added to the scores for the selection only (model.py:113,123)


def precompute_freqs_cis(dim: int, end: int, theta: float) -> np.ndarray:
  """cos || sin table of tinygrad/llm/model.py:15-19, fp32 [end, dim]."""
  f = (1.0 / (np.float32(theta) ** (np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim)))).astype(np.float32)
  ang = np.arange(end, dtype=np.float32)[:, None] * f[None, :]
  return np.concatenate([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


class _Block:
  pass


# hand-over edges used when the caller does not choose (see Transformer.__init__): the ones that measured faster
DEFAULT_HANDOVER = tuple(e for e in os.environ.get("B200Q_HANDOVER", "attn_o").split(",") if e)
STAGED_HANDOVER = os.environ.get("B200Q_STAGED_HANDOVER", "1") == "1"


class Transformer:
  def __init__(self, config: TransformerConfig, state_dict: dict, ggml_type: int = _lib.Q4_0, n_split: int = 0, use_pdl: bool = True,
               use_graph: bool = True, gemv_max_ctas: int = 0, handover=None, tp=None, output_type: int = None, prefill_rows: int = 64,
               prefill_chunk: int = 512, batch: int = 1, engine: str = None, linear_types: dict = None, pipelined_gemm: bool = True):
    """state_dict: the reference's tensor names -> numpy arrays; Linear weights as raw
    GGUF block bytes (uint8), embeddings / norms / biases as fp16.
    tp: a tensor_parallel.TPGroup; `config` is then the FULL model and `state_dict` this rank's shard (shard_state_dict).
    output_type: GGML type of `output.weight` when it differs from the block Linears' (F16 / BF16 / F32 heads run the dense GEMV).
    prefill_rows: prompts with at least this many uncached tokens go through the tensor-core GEMM path, `prefill_chunk` rows at a
    time (0: always one token per step, whose fp32-activation numerics are the reference's own); shorter ones take decode steps.
    engine: how a one-token step runs.  "step": one persistent kernel for the whole step (b200q_decode_step); "chain": five launches per
    block chained with programmatic dependent launch and replayed as a CUDA graph (the default: at batch 1 it measured faster, the
    grid-wide waits inside one kernel costing more than kernel boundaries do).
    linear_types: state-dict name -> GGML type of block Linear weights whose type is not `ggml_type` (files that mix block formats, e.g.
    Q4_K with Q6_K).  Unless every block Linear is of one fused type (Q4_0 / Q8_0) the blocks run on the dense-weight GEMV: every
    weight is dequantised once to fp16 on the device -- the cast the reference applies to every loaded tensor (model.py:376).
    batch: sequences decoded in lock-step (`generate_batch`): one KV cache per sequence, every Linear a tensor-core GEMM over the
    batch rows (the reference's forward on tokens [B, T], model.py:358-364; its cache is sized by the first call's batch, model.py:200-203)."""
    self.tp, self.full_config = tp, config
    if tp is not None:
      from .tensor_parallel import local_config
      config = local_config(config, tp.size)
    c = self.config = config
    vocab_full = self.full_config.vocab_size
    assert c.max_context > 0 and c.n_heads % c.n_kv_heads == 0
    self.qtype, self.flags, self.use_graph = ggml_type, (FLAG_PDL if use_pdl else 0), use_graph
    self.q_dim, self.kv_dim = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
    self.pipelined_gemm = pipelined_gemm      # prompt GEMMs on the pipelined kernel (False: the single-buffered one)
    self.gemv_max_ctas = gemv_max_ctas if isinstance(gemv_max_ctas, dict) else {"*": gemv_max_ctas}   # per Linear ("qkv", "o", "gate_up", "down", "head") or one for all
    self.n_split = n_split or _lib.load().b200q_attn_min_split(c.max_context)
    self.max_context = c.max_context
    self.stream = Stream(tp.stream_ptr()) if (tp is not None and tp.stream_ptr() is not None) else Stream()
    self.tp_peer = tp is not None and tp.kind_id == "peer"
    sd = state_dict
    qkv_rows = self.q_dim + 2 * self.kv_dim
    assert self.q_dim % 16 == 0 and self.kv_dim % 16 == 0, "q/k/v are packed back to back in whole 16-row tiles"
    self.blk = []
    self.weight_bytes = 0
    lt = dict(linear_types or {})
    names7 = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")
    self.dense_blocks = ggml_type not in (_lib.Q4_0, _lib.Q8_0) or any(lt.get(f"blk.{i}.{n}.weight", ggml_type) != ggml_type
                                                                      for i in range(c.num_blocks) for n in names7)
    if self.dense_blocks:
      assert tp is None and batch == 1 and not c.num_experts, "the dense-weight path serves single-sequence dense models on one GPU"
      def dense16(name, n_out, n_in):       # -> fp16 [n_out, n_in] on the device, whatever the tensor's type
        raw, typ = sd[name], lt.get(name, ggml_type)
        if typ in quant.GGML_QUANT: return quant.dequantize(np.ascontiguousarray(raw).view(np.uint8).reshape(-1), n_out * n_in, typ, np.float16)
        return DeviceBuffer.from_numpy(np.asarray(raw).astype(np.float16).reshape(n_out, n_in))
    for i in range(c.num_blocks if self.dense_blocks else 0):
      b = _Block()
      parts = [dense16(f"blk.{i}.attn_{n}.weight", rows, c.dim) for n, rows in (("q", self.q_dim), ("k", self.kv_dim), ("v", self.kv_dim))]
      b.qkv = DeviceBuffer(2 * qkv_rows * c.dim)
      off = 0
      for part in parts:
        check(_lib.load().b200q_memcpy_d2d(b.qkv.ptr + off, part.ptr, part.nbytes, None)); off += part.nbytes
      runtime_sync()
      b.qkv_bias = DeviceBuffer.from_numpy(np.concatenate([np.asarray(sd[f"blk.{i}.attn_{n}.bias"], dtype=np.float16) for n in "qkv"])) if c.qkv_bias else None
      b.o_w = dense16(f"blk.{i}.attn_output.weight", c.dim, self.q_dim)
      b.gate_w, b.up_w = dense16(f"blk.{i}.ffn_gate.weight", c.hidden_dim, c.dim), dense16(f"blk.{i}.ffn_up.weight", c.hidden_dim, c.dim)
      b.down_w = dense16(f"blk.{i}.ffn_down.weight", c.dim, c.hidden_dim)
      b.moe = b.router = None
      b.attn_norm = DeviceBuffer.from_numpy(np.asarray(sd[f"blk.{i}.attn_norm.weight"], dtype=np.float16))
      b.ffn_norm = DeviceBuffer.from_numpy(np.asarray(sd[f"blk.{i}.ffn_norm.weight"], dtype=np.float16))
      kvdt = np.float16 if c.kv_dtype == "float16" else np.float32
      b.k_cache = DeviceBuffer.empty((batch, c.n_kv_heads, c.max_context, c.head_dim), kvdt, zero=True)
      b.v_cache = DeviceBuffer.empty((batch, c.n_kv_heads, c.max_context, c.head_dim), kvdt, zero=True)
      self.blk.append(b)
      self.weight_bytes += 2 * (qkv_rows * c.dim + c.dim * self.q_dim + 3 * c.hidden_dim * c.dim)
    for i in range(0 if self.dense_blocks else c.num_blocks):
      b = _Block()
      b.qkv = DeviceBuffer(quant.packed_bytes(ggml_type, qkv_rows, c.dim))
      off = 0
      for name, rows in (("attn_q", self.q_dim), ("attn_k", self.kv_dim), ("attn_v", self.kv_dim)):
        quant.repack(sd[f"blk.{i}.{name}.weight"], rows, c.dim, ggml_type, out=b.qkv, out_offset=off)
        off += quant.packed_bytes(ggml_type, rows, c.dim)
      b.qkv_bias = None
      if c.qkv_bias:
        b.qkv_bias = DeviceBuffer.from_numpy(np.concatenate([np.asarray(sd[f"blk.{i}.attn_{n}.bias"], dtype=np.float16) for n in "qkv"]))
      b.attn_output = quant.repack(sd[f"blk.{i}.attn_output.weight"], c.dim, self.q_dim, ggml_type)
      b.moe = b.router = None
      if c.num_experts:
        # routed experts: fp32 (E, out, in) weights quantised to MXFP8 on the device; the router stays a dense Linear (model.py:94-98)
        from . import moe
        if c.expert_gating_func not in moe.GATING: raise ValueError(f"unknown expert gating function {c.expert_gating_func!r}")
        gating = moe.Gating(c.expert_gating_func, c.norm_topk_prob, c.routed_scaling_factor,
                            np.asarray(sd[f"blk.{i}.exp_probs_b.bias"], dtype=np.float32) if c.expert_bias else None)
        b.moe = moe.MxMoE(*(np.asarray(sd[f"blk.{i}.ffn_{n}_exps.weight"], dtype=np.float32) for n in ("gate", "up", "down")), c.num_experts_per_tok, gating)
        r = np.asarray(sd[f"blk.{i}.ffn_gate_inp.weight"])
        b.router = quant.DenseWeight(r, c.num_experts, c.dim, quant.GGML_F16 if r.dtype == np.float16 else quant.GGML_F32)
        b.sh_gate_up = b.sh_down = b.sh_inp = None
        if c.shared_expert_dim:      # the shared expert is an ordinary quantised SwiGLU FFN; its optional gate a [dim] vector
          b.sh_gate_up = quant.repack(sd[f"blk.{i}.ffn_gate_shexp.weight"], c.shared_expert_dim, c.dim, ggml_type, raw_up=sd[f"blk.{i}.ffn_up_shexp.weight"])
          b.sh_down = quant.repack(sd[f"blk.{i}.ffn_down_shexp.weight"], c.dim, c.shared_expert_dim, ggml_type)
          if c.shared_expert_gate and f"blk.{i}.ffn_gate_inp_shexp.weight" in sd:
            gw = np.asarray(sd[f"blk.{i}.ffn_gate_inp_shexp.weight"])
            b.sh_inp = quant.DenseWeight(gw.reshape(1, c.dim), 1, c.dim, quant.GGML_F16 if gw.dtype == np.float16 else quant.GGML_F32)
      else:
        b.gate_up = quant.repack(sd[f"blk.{i}.ffn_gate.weight"], c.hidden_dim, c.dim, ggml_type, raw_up=sd[f"blk.{i}.ffn_up.weight"])
        b.ffn_down = quant.repack(sd[f"blk.{i}.ffn_down.weight"], c.dim, c.hidden_dim, ggml_type)
      b.attn_norm = DeviceBuffer.from_numpy(np.asarray(sd[f"blk.{i}.attn_norm.weight"], dtype=np.float16))
      b.ffn_norm = DeviceBuffer.from_numpy(np.asarray(sd[f"blk.{i}.ffn_norm.weight"], dtype=np.float16))
      kvdt = np.float16 if c.kv_dtype == "float16" else np.float32
      b.k_cache = DeviceBuffer.empty((batch, c.n_kv_heads, c.max_context, c.head_dim), kvdt, zero=True)
      b.v_cache = DeviceBuffer.empty((batch, c.n_kv_heads, c.max_context, c.head_dim), kvdt, zero=True)
      self.blk.append(b)
      nel, nby = quant.GGML_QUANT[ggml_type]
      self.weight_bytes += (qkv_rows * c.dim + c.dim * self.q_dim + (0 if c.num_experts else 3 * c.hidden_dim * c.dim)) // nel * nby
    if self.dense_blocks: self.up_buf = DeviceBuffer.empty((c.hidden_dim,), np.float32, zero=True)
    self.output_type = ggml_type if output_type is None else output_type
    # a Q6_K head (the usual companion of K-quant blocks) runs the fused GEMV too; several sequences at once go through the dense GEMV
    if self.output_type in (_lib.Q4_0, _lib.Q8_0) or (self.output_type == _lib.Q6_K and batch == 1 and c.dim % 256 == 0):
      self.output = quant.repack(sd["output.weight"], c.vocab_size, c.dim, self.output_type)
      self.weight_bytes += c.vocab_size * c.dim // quant.GGML_QUANT[self.output_type][0] * quant.GGML_QUANT[self.output_type][1]
    else:
      self.output = quant.DenseWeight(sd["output.weight"], c.vocab_size, c.dim, self.output_type)
      self.weight_bytes += self.output.algorithmic_bytes
    self.output_norm = DeviceBuffer.from_numpy(np.asarray(sd["output_norm.weight"], dtype=np.float16))
    self.token_embd = DeviceBuffer.from_numpy(np.asarray(sd["token_embd.weight"], dtype=np.float16))
    self.rope = DeviceBuffer.from_numpy(precompute_freqs_cis(c.rope_dim, c.max_context, c.rope_theta))
    # activations of one token (fp32 residual stream, model.py:359)
    self.x = tp.empty_f32(c.dim) if tp is not None else DeviceBuffer.empty((c.dim,), np.float32, zero=True)   # NCCL reduces it in place
    self.qkv = DeviceBuffer.empty((qkv_rows,), np.float32, zero=True)
    self.attn = DeviceBuffer.empty((self.q_dim,), np.float32, zero=True)
    self.act = DeviceBuffer.empty((c.hidden_dim,), np.float32, zero=True)
    if tp is not None: self.logits_part, self.logits = tp.empty_f32(c.vocab_size), tp.empty_f32(vocab_full)
    else: self.logits = self.logits_part = DeviceBuffer.empty((c.vocab_size,), np.float32, zero=True)
    if self.tp_peer and isinstance(self.output, quant.DenseWeight): raise NotImplementedError("sharded models need a Q4_0 / Q8_0 head")
    if self.tp_peer:      # two alternating mailboxes for the row-split linears (O, down), one for the vocabulary slices of the head
      from .tensor_parallel import PeerMailbox
      self.mb_o, self.mb_down = PeerMailbox(tp, tp.size, c.dim), PeerMailbox(tp, tp.size, c.dim)
      self.mb_logits = PeerMailbox(tp, 1, vocab_full)
    self.batch = batch
    assert batch >= 1 and (batch == 1 or tp is None), "batched decode runs on one GPU"
    self.tokens = DeviceBuffer.empty((batch, c.max_context + 1), np.int32, zero=True)     # sequence 0 is the single-sequence state
    self.pos = DeviceBuffer.empty((batch,), np.int32, zero=True)
    self.seq_cache_bytes = c.n_kv_heads * c.max_context * c.head_dim * np.dtype(kvdt).itemsize
    self.attn_scratch = DeviceBuffer(_lib.load().b200q_attn_scratch_bytes(c.n_heads, c.n_kv_heads, c.head_dim, self.n_split), zero=True)
    self.argmax_scratch = DeviceBuffer(_lib.load().b200q_argmax_scratch_bytes(), zero=True)
    # Quantised activation hand-over between consecutive kernels (needs whole 128-wide groups everywhere).  Each edge of
    # the chain can be switched on its own: attn_o (attention -> output projection), o_gateup, gateup_down, down_qkv.
    can = c.head_dim == 128 and c.dim % 128 == 0 and c.hidden_dim % 128 == 0 and self.q_dim % 128 == 0 and not self.dense_blocks
    all_edges = ("attn_o", "o_gateup", "gateup_down", "down_qkv")
    if handover is None: edges = DEFAULT_HANDOVER
    elif isinstance(handover, str): edges = tuple(e for e in handover.split(",") if e)
    else: edges = all_edges if handover else ()
    assert all(e in all_edges for e in edges), f"unknown hand-over edge in {edges}"
    if tp is not None: edges = tuple(e for e in edges if e in ("attn_o", "gateup_down"))   # records of all-reduced vectors would hold partial sums
    self.edges = frozenset(edges) if can else frozenset()
    self.handover = bool(self.edges)
    xqb = _lib.load().b200q_xq_bytes
    if "down_qkv" in self.edges: self.xq_a, self.ss_a = DeviceBuffer(xqb(c.dim), zero=True), DeviceBuffer.empty((c.dim // 32,), np.float32, zero=True)
    if "o_gateup" in self.edges: self.xq_b, self.ss_b = DeviceBuffer(xqb(c.dim), zero=True), DeviceBuffer.empty((c.dim // 32,), np.float32, zero=True)
    if "attn_o" in self.edges: self.xq_attn = DeviceBuffer(xqb(self.q_dim), zero=True)
    if "gateup_down" in self.edges: self.xq_act = DeviceBuffer(xqb(c.hidden_dim), zero=True)
    # staging row of the producing GEMVs (32-bit words, all-ones = empty; the kernels leave it empty): row tiles stay dealt to CTAs
    # one by one.  Without it a producing CTA takes runs of 2 / 4 consecutive tiles, which leaves the grid unevenly loaded.
    self.ho_stage = None
    if self.edges and STAGED_HANDOVER:
      self.ho_stage = {n: DeviceBuffer.from_numpy(np.concatenate([np.full(n, 0xFFFFFFFF, np.uint32), np.zeros(n // 32, np.uint32)]))
                       for n in {c.dim, c.hidden_dim}}      # [n_out words | n_out / 32 counters] per producing width
    self._graphs = {}
    self._cached_tokens: list = []
    self.prefill_rows = prefill_rows if (tp is None and not self.dense_blocks and c.hidden_dim % 8 == 0 and c.head_dim in (16, 32, 64, 128)) else 0
    self.prefill_chunk, self._pf, self._batch_logits, self._skinny_ws, self._batch_graph = max(1, prefill_chunk), None, None, None, None
    self._seq_attn_scratch = None
    self.is_moe, self._host_pos = c.num_experts > 0, 0
    if self.is_moe:
      assert tp is None and c.head_dim in (16, 32, 64, 128), "the mixture-of-experts model runs on the row path of one GPU"
      self.prefill_rows = 1
    self.launches_per_step = (7 if self.dense_blocks else 5) * c.num_blocks + 3
    # ---- the whole-step kernel: a device table of the blocks' pointers, its workspace, and the two argument blocks (with / without head)
    self._step_args = None
    if engine not in (None, "step", "chain"): raise ValueError(f"unknown engine {engine!r}")
    if engine == "step" and tp is None and not self.is_moe and not self.dense_blocks and batch == 1 and not isinstance(self.output, quant.DenseWeight) and self.output_type == ggml_type:
      lib = _lib.load()
      table = (_lib.DecodeLayer * c.num_blocks)(*[_lib.DecodeLayer(b.qkv.ptr, b.qkv_bias.ptr if b.qkv_bias else None, b.attn_output.buf.ptr, b.gate_up.buf.ptr,
                                                                  b.ffn_down.buf.ptr, b.attn_norm.ptr, b.ffn_norm.ptr, b.k_cache.ptr, b.v_cache.ptr) for b in self.blk])
      self._layer_table = DeviceBuffer.from_numpy(np.frombuffer(bytes(table), dtype=np.uint8))
      def mk(with_head):
        return _lib.DecodeStepArgs(self._layer_table.ptr, c.num_blocks, ggml_type, c.dim, c.hidden_dim, c.n_heads, c.n_kv_heads, c.head_dim, c.rope_dim,
                                   c.max_context, c.vocab_size, c.vocab_size, F16 if c.kv_dtype == "float16" else F32, c.norm_eps, self.token_embd.ptr,
                                   self.output_norm.ptr, self.output.buf.ptr, self.rope.ptr, self.tokens.ptr, self.pos.ptr, self.x.ptr, self.qkv.ptr,
                                   self.attn.ptr, self.act.ptr, self.logits.ptr, None, 0, with_head, 0, None)
      probe = mk(1)
      rc = lib.b200q_decode_step_supported(ctypes.byref(probe))
      if rc == 0:
        self._step_ws = DeviceBuffer(lib.b200q_decode_step_workspace_bytes(ctypes.byref(probe)), zero=True)
        self._step_args = {}
        for wh in (0, 1):
          a = mk(wh)
          a.workspace, a.workspace_bytes = self._step_ws.ptr, self._step_ws.nbytes
          self._step_args[bool(wh)] = a
        self.launches_per_step = 1
      elif engine == "step":
        check(rc)
    elif engine == "step":
      raise ValueError("the whole-step kernel takes dense single-GPU models whose head has the block Linears' quant type")
    self.engine = "step" if self._step_args else "chain"

  # ---- one token through the network (launch sequence; captured into a graph) ----
  def _enqueue_step(self, with_head: bool, attention: bool = True, tail: bool = True) -> None:
    c, lib, s, fl = self.config, _lib.load(), self.stream.ptr, self.flags
    kvdt = F16 if c.kv_dtype == "float16" else F32
    grid = lambda name: self.gemv_max_ctas.get(name, self.gemv_max_ctas.get("*", 0))
    kw = dict(flags=fl, stream=s)
    tp = self.tp
    # A launch that follows an NCCL call is fully stream-ordered: the programmatic-launch attribute right behind the
    # event waits NCCL leaves in the stream was measured to let the kernel start before the reduced vector is there.
    peer = self.tp_peer
    kw_after_coll = dict(kw, flags=0) if (tp is not None and not peer) else kw
    rkw = dict(residual=self.x, residual_scale=1.0 / tp.size) if tp is not None else dict(residual=self.x)   # row-split shards add residual / n_ranks
    # peer-memory collectives: the row-split GEMV stores its partial row into every rank's mailbox; the reducer adds the residual once
    rkw_o = dict(peers=self.mb_o.targets, peer_rank=tp.rank) if peer else rkw
    rkw_d = dict(peers=self.mb_down.targets, peer_rank=tp.rank) if peer else rkw
    vocab_full = self.full_config.vocab_size
    e, nss = self.edges, c.dim // 32
    qkv_rows = self.q_dim + 2 * self.kv_dim
    # the four hand-over edges: kwargs of the consuming (xq_in...) and of the producing (xq_out...) launch
    in_a = dict(xq_in=self.xq_a, ss_in=self.ss_a, ss_count=nss) if "down_qkv" in e else {}
    in_b = dict(xq_in=self.xq_b, ss_in=self.ss_b, ss_count=nss) if "o_gateup" in e else {}
    in_attn = dict(xq_in=self.xq_attn) if "attn_o" in e else {}
    in_act = dict(xq_in=self.xq_act) if "gateup_down" in e else {}
    if attention or tail:
      ho = "down_qkv" in e
      check(lib.b200q_embed(self.token_embd.ptr, self.tokens.ptr, self.pos.ptr, self.x.ptr, c.dim, vocab_full, c.max_context,
                            self.xq_a.ptr if ho else None, self.blk[0].attn_norm.ptr if ho else None, self.ss_a.ptr if ho else None, fl, s))
    for i, b in enumerate(self.blk if self.dense_blocks else ()):
      # dense-weight blocks: the same step on fp16 matrices, one launch per Linear (norm / bias / residual fused as in the quantised GEMV)
      quant.gemv_dense(b.qkv, F16, qkv_rows, c.dim, self.x, self.qkv, norm_weight=b.attn_norm, norm_eps=c.norm_eps, bias=b.qkv_bias, flags=fl, stream=s)
      a = _lib.AttnArgs(self.qkv.ptr, b.k_cache.ptr, b.v_cache.ptr, kvdt, self.rope.ptr, self.pos.ptr, self.attn.ptr, self.attn_scratch.ptr,
                        c.n_heads, c.n_kv_heads, c.head_dim, c.rope_dim, c.max_context, self.n_split, fl, None)
      check(lib.b200q_attn_decode(ctypes.byref(a), s))
      quant.gemv_dense(b.o_w, F16, c.dim, self.q_dim, self.attn, self.x, residual=self.x, flags=fl, stream=s)
      quant.gemv_dense(b.gate_w, F16, c.hidden_dim, c.dim, self.x, self.act, norm_weight=b.ffn_norm, norm_eps=c.norm_eps, flags=fl, stream=s)
      quant.gemv_dense(b.up_w, F16, c.hidden_dim, c.dim, self.x, self.up_buf, norm_weight=b.ffn_norm, norm_eps=c.norm_eps, flags=fl, stream=s)
      check(lib.b200q_silu_mul(self.act.ptr, self.up_buf.ptr, self.act.ptr, c.hidden_dim, fl, s))
      quant.gemv_dense(b.down_w, F16, c.dim, c.hidden_dim, self.act, self.x, residual=self.x, flags=fl, stream=s)
    for i, b in enumerate(() if self.dense_blocks else self.blk):
      nxt_norm = self.blk[i + 1].attn_norm if i + 1 < len(self.blk) else self.output_norm
      st = (lambda n: dict(xq_out_stage=self.ho_stage[n])) if self.ho_stage is not None else (lambda n: {})
      out_b = dict(xq_out=self.xq_b, xq_out_norm_weight=b.ffn_norm, ss_out=self.ss_b, **st(c.dim)) if "o_gateup" in e else {}
      out_act = dict(xq_out=self.xq_act, **st(c.hidden_dim)) if "gateup_down" in e else {}
      out_a = dict(xq_out=self.xq_a, xq_out_norm_weight=nxt_norm, ss_out=self.ss_a, **st(c.dim)) if "down_qkv" in e else {}
      quant.gemv(b.qkv.ptr, self.qtype, qkv_rows, c.dim, None if in_a else self.x, self.qkv, norm_weight=b.attn_norm, norm_eps=c.norm_eps,
                 bias=b.qkv_bias, max_ctas=grid("qkv"), **in_a, **(kw_after_coll if i > 0 else kw))
      if attention:
        a = _lib.AttnArgs(self.qkv.ptr, b.k_cache.ptr, b.v_cache.ptr, kvdt, self.rope.ptr, self.pos.ptr, self.attn.ptr, self.attn_scratch.ptr,
                          c.n_heads, c.n_kv_heads, c.head_dim, c.rope_dim, c.max_context, self.n_split, fl,
                          self.xq_attn.ptr if "attn_o" in e else None)
        check(lib.b200q_attn_decode(ctypes.byref(a), s))
      quant.gemv(b.attn_output.buf.ptr, self.qtype, c.dim, self.q_dim, None if in_attn else self.attn, None if peer else self.x, **rkw_o,
                 **in_attn, **out_b, max_ctas=grid("o"), **kw)
      if peer: self.mb_o.reduce(self.x, residual=self.x, flags=fl, stream=s)
      elif tp is not None: tp.all_reduce(self.x)
      quant.gemv(b.gate_up.buf.ptr, self.qtype, c.hidden_dim, c.dim, None if in_b else self.x, None if out_act else self.act,
                 norm_weight=b.ffn_norm, norm_eps=c.norm_eps, epilogue=EPI_SILU_MUL, max_ctas=grid("gate_up"), **in_b, **out_act, **kw_after_coll)
      quant.gemv(b.ffn_down.buf.ptr, self.qtype, c.dim, c.hidden_dim, None if in_act else self.act, None if peer else self.x, **rkw_d,
                 **in_act, **out_a, max_ctas=grid("down"), **kw)
      if peer: self.mb_down.reduce(self.x, residual=self.x, flags=fl, stream=s)
      elif tp is not None: tp.all_reduce(self.x)
    if with_head:
      if isinstance(self.output, quant.DenseWeight):
        quant.gemv_dense(self.output.buf, self.output.dtype, c.vocab_size, c.dim, self.x, self.logits_part, norm_weight=self.output_norm,
                         norm_eps=c.norm_eps, flags=kw_after_coll["flags"], stream=s)
      else:
        in_h = {} if self.output_type == _lib.Q6_K else in_a       # the Q6_K kernel quantises the row itself
        quant.gemv(self.output.buf.ptr, self.output_type, c.vocab_size, c.dim, None if in_h else self.x, self.logits_part,
                   norm_weight=self.output_norm, norm_eps=c.norm_eps, max_ctas=grid("head"), **in_h, **kw_after_coll,
                   **(dict(peers=self.mb_logits.targets, peer_rank=tp.rank) if peer else {}))
      if peer: self.mb_logits.reduce(self.logits, flags=fl, stream=s)          # every rank's vocabulary slice, handed over
      elif tp is not None: tp.all_gather(self.logits, self.logits_part)
      if tail: check(lib.b200q_argmax_advance(self.logits.ptr, vocab_full, self.tokens.ptr, self.pos.ptr, c.max_context, self.argmax_scratch.ptr,
                                              0 if (tp is not None and not peer) else fl, s))
    elif tail:
      check(lib.b200q_advance(self.pos.ptr, c.max_context, 0 if (tp is not None and not peer) else fl, s))

  # ---- several prompt tokens at once: tcgen05 dequant GEMMs + batched causal attention ----
  def _prefill_buffers(self):
    if self._pf is None:
      c, T = self.config, self.prefill_chunk
      self._pf = dict(x=DeviceBuffer.empty((T, c.dim), np.float32), xn=DeviceBuffer.empty((T, c.dim), np.float32),
                      qkv=DeviceBuffer.empty((T, self.q_dim + 2 * self.kv_dim), np.float32), q16=DeviceBuffer.empty((T, self.q_dim), np.float32),
                      att=DeviceBuffer.empty((T, self.q_dim), np.float32),
                      act=DeviceBuffer.empty((T, max(c.hidden_dim, c.shared_expert_dim, 1)), np.float32),
                      # activation tiles of the pipelined GEMM (split once per GEMM, read by every column tile's CTA)
                      ws=DeviceBuffer(quant.qgemm_workspace_bytes(T, max(c.dim, self.q_dim, c.hidden_dim, c.shared_expert_dim, 1))) if self.pipelined_gemm else None)
      if self.is_moe:
        self._pf.update(xb=DeviceBuffer.empty((T, c.dim), np.uint16), logits=DeviceBuffer.empty((T, c.num_experts), np.float32))
        if c.shared_expert_dim: self._pf.update(sh=DeviceBuffer.empty((T, c.dim), np.float32), shg=DeviceBuffer.empty((T,), np.float32))
    return self._pf

  def prefill(self, start_pos: int, n: int, sync: bool = True, seq: int = 0) -> None:
    """Run tokens[start_pos : start_pos + n] (already on the device) through every block and fill the KV cache; no logits.
    The forward of tinygrad/llm/model.py:358-362 for T = n, in chunks: per block rmsnorm -> QKV GEMM -> RoPE + cache append +
    causal attention -> O GEMM (+residual) -> rmsnorm -> gate/up GEMM with SwiGLU epilogue -> down GEMM (+residual).
    Activations stay fp32 between the kernels; the GEMMs split them into fp16 hi + lo halves for the tensor core."""
    c, lib, s, f = self.config, _lib.load(), self.stream.ptr, self._prefill_buffers()
    kvdt = F16 if c.kv_dtype == "float16" else F32
    qkv_rows = self.q_dim + 2 * self.kv_dim
    for p0 in range(start_pos, start_pos + n, self.prefill_chunk):
      T = min(self.prefill_chunk, start_pos + n - p0)
      check(lib.b200q_embed_rows(self.token_embd.ptr, self.tokens.ptr + 4 * (seq * (c.max_context + 1) + p0), 1, None, T, c.dim,
                                 self.full_config.vocab_size, f["x"].ptr, s))
      for b in self.blk:
        check(lib.b200q_rmsnorm_rows(f["x"].ptr, b.attn_norm.ptr, c.norm_eps, T, c.dim, f["xn"].ptr, F32, s))
        quant.qgemm(b.qkv.ptr, self.qtype, qkv_rows, c.dim, f["xn"], f["qkv"], T, x_dtype=F32, y_dtype=F32, bias=b.qkv_bias, stream=s, workspace=f["ws"])
        check(lib.b200q_attn_prefill(f["qkv"].ptr, b.k_cache.ptr + seq * self.seq_cache_bytes, b.v_cache.ptr + seq * self.seq_cache_bytes, kvdt,
                                     self.rope.ptr, p0, T, c.n_heads, c.n_kv_heads, c.head_dim,
                                     c.rope_dim, c.max_context, f["q16"].ptr, f["att"].ptr, F32, s))
        quant.qgemm(b.attn_output.buf.ptr, self.qtype, c.dim, self.q_dim, f["att"], f["x"], T, x_dtype=F32, y_dtype=F32, residual=f["x"], stream=s, workspace=f["ws"])
        check(lib.b200q_rmsnorm_rows(f["x"].ptr, b.ffn_norm.ptr, c.norm_eps, T, c.dim, f["xn"].ptr, F32, s))
        if b.moe is not None:
          # router on the fp32 normed rows, experts on their bf16 rounding (the activation dtype of the MXFP8 path); bf16 result + residual
          quant.gemv_dense(b.router.buf, b.router.dtype, c.num_experts, c.dim, f["xn"], f["logits"], m=T, stream=s)
          check(lib.b200q_rmsnorm_rows(f["x"].ptr, b.ffn_norm.ptr, c.norm_eps, T, c.dim, f["xb"].ptr, _lib.BF16, s))
          y = b.moe(f["xb"], f["logits"], T, stream=s)
          if b.sh_gate_up is not None:      # shared expert on the fp32 normed rows (model.py:131-134), added before x moves
            quant.qgemm(b.sh_gate_up.buf.ptr, self.qtype, 2 * c.shared_expert_dim, c.dim, f["xn"], f["act"], T, x_dtype=F32, y_dtype=F32,
                        epilogue=EPI_SILU_MUL, stream=s, workspace=f["ws"])
            quant.qgemm(b.sh_down.buf.ptr, self.qtype, c.dim, c.shared_expert_dim, f["act"], f["sh"], T, x_dtype=F32, y_dtype=F32, stream=s, workspace=f["ws"])
            if b.sh_inp is not None: quant.gemv_dense(b.sh_inp.buf, b.sh_inp.dtype, 1, c.dim, f["xn"], f["shg"], m=T, stream=s)
            check(lib.b200q_add_rows_gated(f["x"].ptr, f["sh"].ptr, f["shg"].ptr if b.sh_inp is not None else None, T, c.dim, s))
          check(lib.b200q_add_rows_bf16(f["x"].ptr, y.ptr, T * c.dim, s))
          continue
        quant.qgemm(b.gate_up.buf.ptr, self.qtype, 2 * c.hidden_dim, c.dim, f["xn"], f["act"], T, x_dtype=F32, y_dtype=F32, epilogue=EPI_SILU_MUL,
                    stream=s, workspace=f["ws"])
        quant.qgemm(b.ffn_down.buf.ptr, self.qtype, c.dim, c.hidden_dim, f["act"], f["x"], T, x_dtype=F32, y_dtype=F32, residual=f["x"], stream=s, workspace=f["ws"])
    if sync:
      self.stream.synchronize()
      self.pos.copy_from(np.array([start_pos + n], dtype=np.int32), offset=4 * seq)
      self._host_pos = start_pos + n

  # ---- several sequences in lock-step ----
  def decode_batch_step(self) -> None:
    """One new token for each of the `batch` sequences, all at the same position: every Linear is one GEMM over the batch rows
    (weights streamed once per step), attention runs per sequence on its own cache, the arg-max per sequence.  Captured once into a
    CUDA graph (positions and tokens live on the device) and replayed."""
    self._check_room()
    if not self.use_graph: return self._enqueue_batch_step()
    if self._batch_graph is None:
      self._enqueue_batch_step()                       # allocates the buffers outside the capture (and is a real step)
      self._batch_graph = Graph(self.stream)
      with self._batch_graph: self._enqueue_batch_step(count=False)
      return
    self._batch_graph.launch()
    self._host_pos += 1

  def _enqueue_batch_step(self, count: bool = True) -> None:
    c, lib, s, f, B = self.config, _lib.load(), self.stream.ptr, self._prefill_buffers(), self.batch
    assert B <= self.prefill_chunk and not self.is_moe
    kvdt = F16 if c.kv_dtype == "float16" else F32
    qkv_rows = self.q_dim + 2 * self.kv_dim
    head_q = not isinstance(self.output, quant.DenseWeight)
    if B <= quant.FEW_ROW_MAX and quant.FEW_ROW_FUSED:       # 8 rows per pass on the int8 tensor cores at the one-row GEMV's arithmetic (weights streamed once per pass)
      if self._skinny_ws is None:
        shapes = [(qkv_rows, c.dim), (c.dim, self.q_dim), (2 * c.hidden_dim, c.dim), (c.dim, c.hidden_dim)] + ([(c.vocab_size, c.dim)] if head_q else [])
        self._skinny_ws = DeviceBuffer(max(quant.qgemv_rows_workspace_bytes(B, o, i) for o, i in shapes))
      def gemm(w, qt, n_out, n_in, x, y, **kw): quant.qgemv_rows(w, qt, n_out, n_in, x, y, B, self._skinny_ws, x_dtype=F32, y_dtype=F32, stream=s, **kw)
    elif B <= 32:    # the weight-streaming GEMM shape (swapped operands, split K); its partial sums go through one workspace
      if self._skinny_ws is None:
        shapes = [(qkv_rows, c.dim), (c.dim, self.q_dim), (2 * c.hidden_dim, c.dim), (c.dim, c.hidden_dim)] + ([(c.vocab_size, c.dim)] if head_q else [])
        self._skinny_ws = DeviceBuffer(max(quant.qgemm_skinny_workspace_bytes(B, o, i) for o, i in shapes))
      def gemm(w, qt, n_out, n_in, x, y, **kw): quant.qgemm_skinny(w, qt, n_out, n_in, x, y, B, self._skinny_ws, x_dtype=F32, y_dtype=F32, stream=s, **kw)
    else:
      def gemm(w, qt, n_out, n_in, x, y, **kw): quant.qgemm(w, qt, n_out, n_in, x, y, B, x_dtype=F32, y_dtype=F32, stream=s, **kw)
    # the position comes from the device (sequence 0's counter; all sequences move together), so the launch sequence can be replayed as a graph
    check(lib.b200q_embed_rows(self.token_embd.ptr, self.tokens.ptr, c.max_context + 1, self.pos.ptr, B, c.dim, c.vocab_size, f["x"].ptr, s))
    fold = B <= quant.FEW_ROW_MAX and quant.FEW_ROW_FUSED     # the few-row kernel's pre-pass applies the RMSNorm itself: no norm launches
    seq_attn = SEQ_ATTENTION and c.n_heads // c.n_kv_heads <= 8 and c.head_dim % 8 == 0 and c.head_dim <= 128
    if seq_attn and self._seq_attn_scratch is None:
      stride = lib.b200q_attn_seq_scratch_stride(c.n_heads, c.n_kv_heads, c.head_dim, self.n_split)
      self._seq_attn_scratch = DeviceBuffer(B * stride, zero=True)
    def normed(norm):
      if fold: return f["x"], {"norm_weight": norm, "norm_eps": c.norm_eps}
      check(lib.b200q_rmsnorm_rows(f["x"].ptr, norm.ptr, c.norm_eps, B, c.dim, f["xn"].ptr, F32, s))
      return f["xn"], {}
    for b in self.blk:
      xin, kw = normed(b.attn_norm)
      gemm(b.qkv.ptr, self.qtype, qkv_rows, c.dim, xin, f["qkv"], bias=b.qkv_bias, **kw)
      if seq_attn:     # the one-token kernel over (KV head, slice, sequence): RoPE, cache append and attention in one launch
        a = _lib.AttnArgs(f["qkv"].ptr, b.k_cache.ptr, b.v_cache.ptr, kvdt, self.rope.ptr, self.pos.ptr, f["att"].ptr, self._seq_attn_scratch.ptr,
                          c.n_heads, c.n_kv_heads, c.head_dim, c.rope_dim, c.max_context, self.n_split, _lib.FLAG_PDL, None)
        check(lib.b200q_attn_decode_seqs(ctypes.byref(a), B, s))
      else:
        check(lib.b200q_attn_decode_batch(f["qkv"].ptr, b.k_cache.ptr, b.v_cache.ptr, kvdt, self.rope.ptr, 0, self.pos.ptr, B, c.n_heads, c.n_kv_heads,
                                          c.head_dim, c.rope_dim, c.max_context, f["q16"].ptr, f["att"].ptr, F32, s))
      gemm(b.attn_output.buf.ptr, self.qtype, c.dim, self.q_dim, f["att"], f["x"], residual=f["x"])
      xin, kw = normed(b.ffn_norm)
      gemm(b.gate_up.buf.ptr, self.qtype, 2 * c.hidden_dim, c.dim, xin, f["act"], epilogue=EPI_SILU_MUL, **kw)
      gemm(b.ffn_down.buf.ptr, self.qtype, c.dim, c.hidden_dim, f["act"], f["x"], residual=f["x"])
    if self._batch_logits is None: self._batch_logits = DeviceBuffer.empty((B, c.vocab_size), np.float32)
    if head_q and fold:
      gemm(self.output.buf.ptr, self.output_type, c.vocab_size, c.dim, f["x"], self._batch_logits, norm_weight=self.output_norm, norm_eps=c.norm_eps)
    else:
      check(lib.b200q_rmsnorm_rows(f["x"].ptr, self.output_norm.ptr, c.norm_eps, B, c.dim, f["xn"].ptr, F32, s))
      if head_q: gemm(self.output.buf.ptr, self.output_type, c.vocab_size, c.dim, f["xn"], self._batch_logits)
      else: quant.gemv_dense(self.output.buf, self.output.dtype, c.vocab_size, c.dim, f["xn"], self._batch_logits, m=B, stream=s)
    for i in range(B):
      check(lib.b200q_argmax_advance(self._batch_logits.ptr + 4 * i * c.vocab_size, c.vocab_size, self.tokens.ptr + 4 * i * (c.max_context + 1),
                                     self.pos.ptr + 4 * i, c.max_context, self.argmax_scratch.ptr, 0, s))
    if count: self._host_pos += 1

  def generate_batch(self, prompts: list):
    """Greedy generation for `batch` prompts of equal length; yields the list of the sequences' next tokens per step."""
    c, B = self.config, self.batch
    assert len(prompts) == B and len({len(p) for p in prompts}) == 1 and len(prompts[0]) >= 1
    L = len(prompts[0])
    self.stream.synchronize()
    tok = np.zeros((B, c.max_context + 1), np.int32)
    for i, p in enumerate(prompts): tok[i, :L] = p
    self.tokens.copy_from(tok)
    for i in range(B):
      if L > 1: self.prefill(0, L - 1, seq=i)
    self.pos.copy_from(np.full((B,), L - 1, dtype=np.int32))
    self._host_pos, n = L - 1, L
    while n < c.max_context:
      self.decode_batch_step()
      self.stream.synchronize()
      yield [int(t) for t in self.tokens.numpy((B, c.max_context + 1), np.int32)[:, n]]
      n += 1

  def _step_rows(self, with_head: bool) -> None:
    """One token through the row path (mixture-of-experts models: their FFN is not part of the fused one-token chain)."""
    c, lib, s = self.config, _lib.load(), self.stream.ptr
    self.prefill(self._host_pos, 1, sync=False)
    if with_head:
      x_last = self._pf["x"]
      if isinstance(self.output, quant.DenseWeight):
        quant.gemv_dense(self.output.buf, self.output.dtype, c.vocab_size, c.dim, x_last, self.logits, norm_weight=self.output_norm, norm_eps=c.norm_eps,
                         stream=s)
      else:
        quant.gemv(self.output.buf.ptr, self.output_type, c.vocab_size, c.dim, x_last, self.logits, norm_weight=self.output_norm, norm_eps=c.norm_eps,
                   stream=s)
      check(lib.b200q_argmax_advance(self.logits.ptr, c.vocab_size, self.tokens.ptr, self.pos.ptr, c.max_context, self.argmax_scratch.ptr, 0, s))
    else:
      check(lib.b200q_advance(self.pos.ptr, c.max_context, 0, s))
    self._host_pos += 1

  def _check_room(self) -> None:
    if self._host_pos >= self.max_context:
      raise RuntimeError(f"context full: position {self._host_pos} has no KV-cache row (max_context {self.max_context})")

  def gemv_launches(self) -> list:
    """(n_out rows streamed, n_in) of every GEMV launch of one step with the head, in launch order."""
    c = self.config
    per_block = [(self.q_dim + 2 * self.kv_dim, c.dim), (c.dim, self.q_dim), (2 * c.hidden_dim, c.dim), (c.dim, c.hidden_dim)]
    return per_block * c.num_blocks + [(c.vocab_size, c.dim)]

  def gemv_only_graph(self) -> Graph:
    """The GEMV launches of one step alone, in order, for timing the weight stream by itself
    (it overwrites the activation buffers: use it after the real steps)."""
    g = Graph(self.stream)
    with g: self._enqueue_step(with_head=True, attention=False, tail=False)
    return g

  def step(self, with_head: bool = True) -> None:
    """Advance by one token on the device: reads tokens[pos]; with the head, writes tokens[pos+1].
    The host mirrors the device position and refuses a step that has no KV-cache row left (nothing is launched then)."""
    self._check_room()
    if self.is_moe: return self._step_rows(with_head)
    self._host_pos += 1
    if self._step_args: return check(_lib.load().b200q_decode_step(ctypes.byref(self._step_args[bool(with_head)]), self.stream.ptr))
    if not self.use_graph: return self._enqueue_step(with_head)
    g = self._graphs.get(with_head)
    if g is None:
      g = Graph(self.stream)
      with g: self._enqueue_step(with_head)
      self._graphs[with_head] = g
    g.launch()

  # ---- host-visible state ----
  def set_state(self, tokens: list, pos: int) -> None:
    self.stream.synchronize()
    if tokens: self.tokens.copy_from(np.asarray(tokens, dtype=np.int32))
    self.pos.copy_from(np.array([pos], dtype=np.int32))
    self._host_pos = pos

  def read_token(self, index: int) -> int:
    self.stream.synchronize()
    return int(self.tokens.numpy((1,), np.int32, offset=4 * index)[0])

  def read_logits(self) -> np.ndarray:
    self.stream.synchronize()
    return self.logits.numpy()

  def get_start_pos(self, tokens: list) -> int:
    """How much of the KV cache the new prompt can reuse (model.py:456-462)."""
    n = 0
    for a, b in zip(tokens[:-1], self._cached_tokens):
      if a != b: break
      n += 1
    return n

  def generate(self, tokens: list, temperature: float = 0.0):
    """Greedy generation (model.py:464-484 at temperature 0).  Yields one token id at a time;
    the prompt is consumed one position per step through the same kernels."""
    if temperature != 0.0: raise NotImplementedError("only greedy decoding (temperature 0) is implemented")
    tokens = list(tokens)
    start_pos = self.get_start_pos(tokens)
    self.set_state(tokens, start_pos)
    n_pre = len(tokens) - 1 - start_pos
    if self.prefill_rows and n_pre >= self.prefill_rows: self.prefill(start_pos, n_pre)
    else:
      for _ in range(n_pre): self.step(with_head=False)
    while len(tokens) < self.max_context:
      self.step(with_head=True)
      tok = self.read_token(len(tokens))
      tokens.append(tok)
      self._cached_tokens = tokens[:-1]
      yield tok
