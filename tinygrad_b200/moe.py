"""MXFP8 mixture-of-experts feed-forward on the device: host-side mirror of the reference's grouped path.

`quantize_mxfp8` is extra/gemm/cdna_asm_gemm.py:149-159; `route` / `combine` are extra/gemm/moe_routing.py:109-131;
`MxMoE.__call__` chains them like examples/mlperf/models/gpt_oss.py:215-226 (route -> dispatch -> grouped_mx_gemm ->
activation -> grouped_mx_gemm -> combine), with the SwiGLU of tinygrad/llm/model.py:129.  bf16 tensors travel as
uint16 arrays on the host (numpy has no bfloat16).  All compute is in libb200q.so.
"""
from dataclasses import dataclass
import numpy as np
from . import _lib
from ._lib import check, F32, BF16
from .runtime import DeviceBuffer, stream_ptr

ROUTE_TOPK_SOFTMAX, ROUTE_SOFTMAX_TOPK = 0, 1   # weights = softmax over the k best logits | softmax over all experts, not renormalised
GATING = {"softmax": 1, "sigmoid": 2, "softmax_weight": 3, "sqrt_softplus": 4}     # ExpertGating, tinygrad/llm/model.py:9-13


@dataclass(frozen=True)
class Gating:
  """The gating of tinygrad's MoE block (tinygrad/llm/model.py:110-128): scoring function, renormalisation over the selected k,
  scaling factor and optional selection bias (fp32 [n_experts], added to the scores for the selection only)."""
  func: str = "softmax"
  norm_topk_prob: bool = False
  routed_scaling_factor: float = 1.0
  sel_bias: object = None

  def resolved(self):
    """(gating id, normalize) after the reference's shortcut: softmax + normalize + no bias is softmax over the k selected logits."""
    g, n = GATING[self.func], bool(self.norm_topk_prob)
    if g == 1 and n and self.sel_bias is None: g, n = 3, False
    return g, n


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
  """fp32 -> bf16 bit patterns, round-to-nearest-even (tinygrad/dtype.py:222-226)."""
  u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
  return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
  return (b.astype(np.uint32) << 16).view(np.float32)


def quantize_mxfp8(x: DeviceBuffer, rows: int, k: int, dtype: int, dest_row: DeviceBuffer = None, fan: int = 1, out_rows: int = None, stream=None):
  """-> (q codes uint8 [out_rows, k], e8 uint8 [out_rows, k/32]).  With dest_row the rows are scattered (dispatch) into zeroed outputs."""
  out_rows = rows if out_rows is None else out_rows
  q, e8 = DeviceBuffer.empty((out_rows, k), np.uint8, zero=dest_row is not None), DeviceBuffer.empty((out_rows, k // 32), np.uint8, zero=dest_row is not None)
  check(_lib.load().b200q_quantize_mxfp8(x.ptr, dtype, rows, k, dest_row.ptr if dest_row else None, fan, q.ptr, e8.ptr, stream_ptr(stream)))
  return q, e8


class Routing:
  """Device tables of `route` (extra/gemm/moe_routing.py:92-122).  Buffers are allocated once and reused by `run`."""
  def __init__(self, n_tokens: int, n_experts: int, k: int, mode=ROUTE_TOPK_SOFTMAX):
    """mode: ROUTE_TOPK_SOFTMAX (`route` of extra/gemm/moe_routing.py), ROUTE_SOFTMAX_TOPK (the OLMoE defaults of tinygrad/llm), or a `Gating`."""
    lib = _lib.load()
    self.n_tokens, self.n_experts, self.k, self.mode = n_tokens, n_experts, k, mode
    self._bias = None
    if isinstance(mode, Gating) and mode.sel_bias is not None:
      self._bias = DeviceBuffer.from_numpy(np.asarray(mode.sel_bias, dtype=np.float32).reshape(n_experts))
    self.m_l = lib.b200q_moe_rows_max(n_tokens, n_experts, k)
    self.topi, self.weights = DeviceBuffer.empty((n_tokens, k), np.int32), DeviceBuffer.empty((n_tokens, k), np.float32)
    self.dest_row, self.off = DeviceBuffer.empty((n_tokens * k,), np.int32), DeviceBuffer.empty((n_experts + 1,), np.int32)
    self._scratch = DeviceBuffer(lib.b200q_moe_route_scratch_bytes(n_tokens, n_experts, k))

  def run(self, logits: DeviceBuffer, stream=None) -> "Routing":
    if isinstance(self.mode, Gating):
      g, norm = self.mode.resolved()
      check(_lib.load().b200q_moe_route_gating(logits.ptr, self._bias.ptr if self._bias else None, self.n_tokens, self.n_experts, self.k, g, int(norm),
                                               float(self.mode.routed_scaling_factor), 256, self.topi.ptr, self.weights.ptr, self.dest_row.ptr,
                                               self.off.ptr, None, self._scratch.ptr, stream_ptr(stream)))
      return self
    check(_lib.load().b200q_moe_route(logits.ptr, self.n_tokens, self.n_experts, self.k, self.mode, self.topi.ptr, self.weights.ptr,
                                      self.dest_row.ptr, self.off.ptr, self._scratch.ptr, stream_ptr(stream)))
    return self


class MxMoE:
  """Expert SwiGLU FFN with MXFP8 operands.  w_gate / w_up: (E, F, D), w_down: (E, D, F), fp32 numpy; quantised once along K.
  The workspace for `n_tokens` tokens is allocated on the first call and reused: a call launches kernels only."""
  def __init__(self, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray, k: int, mode: int = ROUTE_SOFTMAX_TOPK):
    self.E, self.F, self.D = w_gate.shape
    self.k, self.mode = k, mode
    # one GEMM yields gate and up.  F % 128 == 0: rows interleaved 128 gate / 128 up per 256-row tile, so that the GEMM's epilogue
    # can apply silu(gate) * up and requantise (b200q_grouped_mxfp8_gemm_swiglu); else [gate | up] halves and a separate kernel
    self.fused = self.F % 128 == 0
    if self.fused:
      gu = np.stack([w_gate.reshape(self.E, self.F // 128, 128, self.D), w_up.reshape(self.E, self.F // 128, 128, self.D)], axis=2)
      gu = np.ascontiguousarray(gu.reshape(self.E, 2 * self.F, self.D), dtype=np.float32)
    else:
      gu = np.concatenate([w_gate, w_up], axis=1).astype(np.float32)
    self.gu_q, self.gu_e8 = quantize_mxfp8(DeviceBuffer.from_numpy(gu), self.E * 2 * self.F, self.D, F32)
    self.dn_q, self.dn_e8 = quantize_mxfp8(DeviceBuffer.from_numpy(w_down.astype(np.float32)), self.E * self.D, self.F, F32)
    self._wss, self._ws = {}, None

  def _workspace(self, n_tokens: int):
    self._ws = self._wss.get(n_tokens)
    if self._ws is None:
      r = Routing(n_tokens, self.E, self.k, self.mode)
      m = r.m_l
      # a_q / a_e8 are zeroed once, here: the rows between the groups (padding to 256) feed only output rows that nobody reads, and what a
      # later call leaves there is an earlier call's quantised row (finite codes, valid exponents), never an uninitialised pattern
      self._ws = self._wss[n_tokens] = dict(T=n_tokens, r=r, a_q=DeviceBuffer.empty((m, self.D), np.uint8, zero=True),
                      a_e8=DeviceBuffer.empty((m, self.D // 32), np.uint8, zero=True),
                      h=DeviceBuffer.empty((m, 2 * self.F), np.uint16, zero=True), act_q=DeviceBuffer.empty((m, self.F), np.uint8),
                      act_e8=DeviceBuffer.empty((m, self.F // 32), np.uint8), y=DeviceBuffer.empty((m, self.D), np.uint16, zero=True),
                      out=DeviceBuffer.empty((n_tokens, self.D), np.uint16))
    return self._ws

  def __call__(self, x_bf16: DeviceBuffer, logits: DeviceBuffer, n_tokens: int, stream=None) -> DeviceBuffer:
    """x (T, D) bf16, router logits (T, E) fp32 -> (T, D) bf16."""
    lib, s, w = _lib.load(), stream_ptr(stream), self._workspace(n_tokens)
    r = w["r"].run(logits, stream)
    check(lib.b200q_quantize_mxfp8(x_bf16.ptr, BF16, n_tokens, self.D, r.dest_row.ptr, self.k, w["a_q"].ptr, w["a_e8"].ptr, s))
    if self.fused:
      check(lib.b200q_grouped_mxfp8_gemm_swiglu(w["a_q"].ptr, w["a_e8"].ptr, self.gu_q.ptr, self.gu_e8.ptr, r.off.ptr, self.E, r.m_l, 2 * self.F, self.D,
                                                w["act_q"].ptr, w["act_e8"].ptr, s))
    else:
      check(lib.b200q_grouped_mxfp8_gemm(w["a_q"].ptr, w["a_e8"].ptr, self.gu_q.ptr, self.gu_e8.ptr, r.off.ptr, self.E, r.m_l, 2 * self.F, self.D,
                                         w["h"].ptr, s))
      check(lib.b200q_swiglu_quantize_mxfp8(w["h"].ptr, r.m_l, r.off.ptr + 4 * self.E, self.F, w["act_q"].ptr, w["act_e8"].ptr, s))
    check(lib.b200q_grouped_mxfp8_gemm(w["act_q"].ptr, w["act_e8"].ptr, self.dn_q.ptr, self.dn_e8.ptr, r.off.ptr, self.E, r.m_l, self.D, self.F,
                                       w["y"].ptr, s))
    check(lib.b200q_moe_combine(w["y"].ptr, r.dest_row.ptr, r.weights.ptr, n_tokens, self.k, self.D, w["out"].ptr, s))
    self.last_routing = r
    return w["out"]

  def phases(self, x_bf16: DeviceBuffer, logits: DeviceBuffer, n_tokens: int, stream=None) -> dict:
    """name -> a callable that enqueues that phase of `__call__` alone on `stream` (for timing them one by one; call the layer once first)."""
    lib, s, w, T = _lib.load(), stream_ptr(stream), self._workspace(n_tokens), n_tokens
    r = w["r"]
    ph = {"route": lambda: r.run(logits, stream),
          "dispatch_quantize": lambda: lib.b200q_quantize_mxfp8(x_bf16.ptr, BF16, T, self.D, r.dest_row.ptr, self.k, w["a_q"].ptr, w["a_e8"].ptr, s)}
    if self.fused:
      ph["gate_up_gemm_swiglu"] = lambda: lib.b200q_grouped_mxfp8_gemm_swiglu(w["a_q"].ptr, w["a_e8"].ptr, self.gu_q.ptr, self.gu_e8.ptr, r.off.ptr, self.E,
                                                                             r.m_l, 2 * self.F, self.D, w["act_q"].ptr, w["act_e8"].ptr, s)
    else:
      ph["gate_up_gemm"] = lambda: lib.b200q_grouped_mxfp8_gemm(w["a_q"].ptr, w["a_e8"].ptr, self.gu_q.ptr, self.gu_e8.ptr, r.off.ptr, self.E, r.m_l,
                                                               2 * self.F, self.D, w["h"].ptr, s)
      ph["swiglu_quantize"] = lambda: lib.b200q_swiglu_quantize_mxfp8(w["h"].ptr, r.m_l, r.off.ptr + 4 * self.E, self.F, w["act_q"].ptr, w["act_e8"].ptr, s)
    ph["down_gemm"] = lambda: lib.b200q_grouped_mxfp8_gemm(w["act_q"].ptr, w["act_e8"].ptr, self.dn_q.ptr, self.dn_e8.ptr, r.off.ptr, self.E, r.m_l, self.D,
                                                          self.F, w["y"].ptr, s)
    ph["combine"] = lambda: lib.b200q_moe_combine(w["y"].ptr, r.dest_row.ptr, r.weights.ptr, T, self.k, self.D, w["out"].ptr, s)
    return ph


class ExpertWeights:
  """`ExpertWeights` of tinygrad/llm/model.py:21-27 on MXFP8 operands: weight (num_experts, out_features, in_features), and
  `__call__(sel, x)` with sel (T, k) int32 and x (T, 1, in) or (T, k, in) bf16 -> (T, k, out) bf16, row (t, j) = x[t, j or 0] @ weight[sel[t, j]].T.
  The rows are grouped by expert (b200q_moe_route_tables), quantised into the groups, multiplied by one grouped GEMM and gathered back
  into (t, j) order.  out_features must be a multiple of 256 and in_features of 128 (the grouped GEMM's tile sizes)."""
  def __init__(self, weight: np.ndarray):
    self.num_experts, self.out_features, self.in_features = weight.shape
    if self.out_features % 256 or self.in_features % 128: raise ValueError("out_features % 256 == in_features % 128 == 0 is required")
    self.w_q, self.w_e8 = quantize_mxfp8(DeviceBuffer.from_numpy(np.ascontiguousarray(weight, dtype=np.float32)), self.num_experts * self.out_features,
                                         self.in_features, F32)
    self._ws = {}

  def __call__(self, sel: DeviceBuffer, x: DeviceBuffer, stream=None) -> DeviceBuffer:
    T, k = sel.shape
    fan_in = x.shape[-2] if len(x.shape) == 3 else 1
    if x.shape[0] != T or x.shape[-1] != self.in_features or fan_in not in (1, k): raise ValueError(f"x {x.shape} does not match sel {sel.shape}")
    lib, s, E = _lib.load(), stream_ptr(stream), self.num_experts
    w = self._ws.get((T, k))
    if w is None:
      m = lib.b200q_moe_rows_max(T, E, k)
      w = self._ws[(T, k)] = dict(m=m, dest=DeviceBuffer.empty((T * k,), np.int32), off=DeviceBuffer.empty((E + 1,), np.int32),
                                  scratch=DeviceBuffer(lib.b200q_moe_route_scratch_bytes(T, E, k)),
                                  a_q=DeviceBuffer.empty((m, self.in_features), np.uint8, zero=True), a_e8=DeviceBuffer.empty((m, self.in_features // 32), np.uint8, zero=True),
                                  y=DeviceBuffer.empty((m, self.out_features), np.uint16, zero=True), out=DeviceBuffer.empty((T, k, self.out_features), np.uint16))
    check(lib.b200q_moe_route_tables(sel.ptr, T, E, k, 256, w["dest"].ptr, w["off"].ptr, None, w["scratch"].ptr, s))
    # x (T, 1, in): one row fans out to its k destinations; x (T, k, in): row (t, j) goes to its own destination
    rows, fan = (T, k) if fan_in == 1 else (T * k, 1)
    check(lib.b200q_quantize_mxfp8(x.ptr, BF16, rows, self.in_features, w["dest"].ptr, fan, w["a_q"].ptr, w["a_e8"].ptr, s))
    check(lib.b200q_grouped_mxfp8_gemm(w["a_q"].ptr, w["a_e8"].ptr, self.w_q.ptr, self.w_e8.ptr, w["off"].ptr, E, w["m"], self.out_features, self.in_features,
                                       w["y"].ptr, s))
    check(lib.b200q_permute_rows(w["y"].ptr, w["dest"].ptr, T * k, 2 * self.out_features, w["out"].ptr, 1, s))
    return w["out"]
