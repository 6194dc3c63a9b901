"""numpy restatement of tinygrad's LLM forward pass (test infrastructure).

Follows tinygrad/llm/model.py: ``apply_rope`` :29-33, ``pairwise_topk`` :35-41,
``FFNBlock._feed_forward`` :109-137, ``TransformerBlock._attention`` :167-198,
``Transformer.forward`` :358-364 and ``generate`` :464-484; RMSNorm from
tinygrad/nn/__init__.py:300-304; attention from tinygrad/mixin/rand.py:298-326;
linear numerics from tinygrad/mixin/op.py:367-392 (fp32 accumulation).

Weights are a dict name -> ndarray with the reference's state-dict names.
Quantised linears are given as their exact fp32 dequantised matrices: with the
fp32 residual stream of the model the reference's fused kernels use the
unrounded fp32 dequant value (the lazy fp16 cast is removed by
tinygrad/codegen/late/coalesce.py:100).
"""
from dataclasses import dataclass
import numpy as np

SOFTMAX, SIGMOID, SOFTMAX_WEIGHT, SQRT_SOFTPLUS = 1, 2, 3, 4   # model.py:9-13


@dataclass
class Config:                      # the fields of model.py:52-83 this path uses
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
  max_context: int
  num_experts: int = 0
  num_experts_per_tok: int = 0
  norm_topk_prob: bool = False
  expert_gating_func: int = SOFTMAX
  routed_scaling_factor: float = 1.0
  qkv_bias: bool = False
  kv_dtype: str = "float16"


def freqs_cis(dim: int, end: int, theta: float) -> np.ndarray:
  """model.py:15-19: cos || sin of pos * theta^(-2i/dim), fp32."""
  f = (1.0 / (np.float32(theta) ** (np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim)))).astype(np.float32)
  ang = np.arange(end, dtype=np.float32)[:, None] * f[None, :]
  return np.concatenate([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
  """nn/__init__.py:300-304: fp32 norm, cast back, then times weight."""
  xf = x.astype(np.float32)
  n = xf * (1.0 / np.sqrt((xf * xf).mean(-1, keepdims=True, dtype=np.float32) + np.float32(eps))).astype(np.float32)
  return (n.astype(x.dtype) * w.astype(np.float32)).astype(np.float32)


def linear(x: np.ndarray, w: np.ndarray, b=None) -> np.ndarray:
  """x (..., in) @ w(out, in)^T (+ b); fp32 products, fp32 accumulation."""
  y = x.astype(np.float32) @ w.astype(np.float32).T
  return y if b is None else y + b.astype(np.float32)


def linear_f16(x16: np.ndarray, w32: np.ndarray) -> np.ndarray:
  """The fp16-activation case (a single Linear called on an fp16 tensor): the
  weight is rounded to fp16, each product is an fp16 multiply, and the sum is
  accumulated in fp32 and cast back to fp16 (tinygrad/mixin/op.py:367-392,
  tinygrad/dtype.py:212-216)."""
  w16 = w32.astype(np.float16)
  prod = (x16[..., None, :].astype(np.float16) * w16[None, ...]).astype(np.float16)
  return prod.astype(np.float32).sum(-1, dtype=np.float32).astype(np.float16)


def apply_rope(x: np.ndarray, fc: np.ndarray) -> np.ndarray:
  """model.py:29-33, half-split layout.  x (B,H,T,R), fc (T,R)."""
  cos, sin = np.split(fc.reshape(1, 1, x.shape[2], -1), 2, axis=-1)
  x1, x2 = np.split(x, 2, axis=-1)
  return np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], axis=-1)


def softmax(x: np.ndarray, axis=-1) -> np.ndarray:
  m = x.max(axis, keepdims=True)
  e = np.exp((x - m).astype(np.float32))
  return (e / e.sum(axis, keepdims=True, dtype=np.float32)).astype(np.float32)


def silu(x): return x / (1.0 + np.exp(-x.astype(np.float32)))


def pairwise_topk(x: np.ndarray, k: int):
  """model.py:35-41: rank by compare-count (ties: the lower index ranks
  higher), keep the k top ranks in ascending-rank order."""
  n = x.shape[-1]
  idx = np.arange(n)
  cmp = (x[..., :, None] > x[..., None, :]) | ((x[..., :, None] == x[..., None, :]) & (idx[:, None] < idx[None, :]))
  rank = cmp.sum(-1)                                   # n-1 for the largest
  order = np.zeros(x.shape, dtype=np.int64)
  np.put_along_axis(order, rank, np.broadcast_to(idx, x.shape), axis=-1)
  sel = order[..., n - k:].astype(np.int32)
  return np.take_along_axis(x, sel, axis=-1), sel


def moe_gate(logits: np.ndarray, gating: int, normalize: bool, k: int, scale: float = 1.0, bias=None):
  """Router logits (..., E) -> (sel (..., k) int32 in ascending rank order, probs (..., k)): tinygrad/llm/model.py:112-128."""
  if gating == SOFTMAX and normalize and bias is None: gating, normalize = SOFTMAX_WEIGHT, False      # model.py:116-117
  if gating == SOFTMAX_WEIGHT: scores = logits
  elif gating == SOFTMAX: scores = softmax(logits)
  elif gating == SIGMOID: scores = (1.0 / (1.0 + np.exp(-logits))).astype(np.float32)
  else: scores = np.sqrt(np.log1p(np.exp(logits))).astype(np.float32)
  _, sel = pairwise_topk(scores if bias is None else scores + bias.astype(np.float32), k)           # the bias only steers the selection
  probs = np.take_along_axis(scores, sel.astype(np.int64), axis=-1)
  if gating == SOFTMAX_WEIGHT: probs = softmax(probs)
  if normalize: probs = probs / probs.sum(-1, keepdims=True)
  return sel, (probs * np.float32(scale)).astype(np.float32)


class Transformer:
  def __init__(self, cfg: Config, weights: dict):
    self.cfg, self.w = cfg, weights
    kvdt = np.float16 if cfg.kv_dtype == "float16" else np.float32
    self.cache = [np.zeros((2, 1, cfg.n_kv_heads, cfg.max_context, cfg.head_dim), dtype=kvdt) for _ in range(cfg.num_blocks)]
    self.fc = freqs_cis(cfg.rope_dim, cfg.max_context, cfg.rope_theta)

  def _lin(self, name, x):
    return linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

  def _attention(self, i, x, start_pos):                       # model.py:167-198
    c, (B, T, _) = self.cfg, x.shape
    q, k, v = (self._lin(f"blk.{i}.attn_{n}", x) for n in "qkv")
    q = q.reshape(B, T, c.n_heads, c.head_dim).transpose(0, 2, 1, 3)
    k = k.reshape(B, T, c.n_kv_heads, c.head_dim).transpose(0, 2, 1, 3)
    v = v.reshape(B, T, c.n_kv_heads, c.head_dim).transpose(0, 2, 1, 3)
    fc = self.fc[start_pos:start_pos + T]
    q = np.concatenate([apply_rope(q[..., :c.rope_dim], fc), q[..., c.rope_dim:]], axis=-1)
    k = np.concatenate([apply_rope(k[..., :c.rope_dim], fc), k[..., c.rope_dim:]], axis=-1)
    cache = self.cache[i]
    cache[0, :, :, start_pos:start_pos + T] = k.astype(cache.dtype)
    cache[1, :, :, start_pos:start_pos + T] = v.astype(cache.dtype)
    kk = cache[0, :, :, :start_pos + T].astype(np.float32)
    vv = cache[1, :, :, :start_pos + T].astype(np.float32)
    rep = c.n_heads // c.n_kv_heads                              # rand.py:314-316
    kk, vv = np.repeat(kk, rep, axis=1), np.repeat(vv, rep, axis=1)
    qk = (q.astype(np.float32) @ kk.transpose(0, 1, 3, 2)) / np.float32(np.sqrt(c.head_dim))
    if T != 1:                                                   # model.py:194-195, lower-right causal
      mask = np.triu(np.full((T, start_pos + T), -np.inf, dtype=np.float32), start_pos + 1)
      qk = qk + mask
    attn = softmax(qk) @ vv
    attn = attn.transpose(0, 2, 1, 3).reshape(B, T, -1)
    return self._lin(f"blk.{i}.attn_output", attn)

  def _feed_forward(self, i, x):                                 # model.py:109-137
    c = self.cfg
    if c.num_experts == 0:
      return self._lin(f"blk.{i}.ffn_down", silu(self._lin(f"blk.{i}.ffn_gate", x)) * self._lin(f"blk.{i}.ffn_up", x))
    logits = self._lin(f"blk.{i}.ffn_gate_inp", x)
    sel, probs = moe_gate(logits, c.expert_gating_func, c.norm_topk_prob, c.num_experts_per_tok, c.routed_scaling_factor,
                          self.w.get(f"blk.{i}.exp_probs_b.bias"))
    wg, wu, wd = (self.w[f"blk.{i}.ffn_{n}_exps.weight"] for n in ("gate", "up", "down"))
    h = x[:, :, None, :]                                         # (B,T,1,D)
    g = np.einsum("btid,btkod->btko", h, wg[sel])                 # model.py:25-27
    u = np.einsum("btid,btkod->btko", h, wu[sel])
    d = np.einsum("btkh,btkoh->btko", (silu(g) * u).astype(np.float32), wd[sel])
    out = (d * probs[..., None]).sum(2).astype(np.float32)
    return out + self._shared_expert(i, x)

  def _shared_expert(self, i, x):                                # model.py:131-134
    if f"blk.{i}.ffn_gate_shexp.weight" not in self.w: return np.float32(0.0)
    sh = self._lin(f"blk.{i}.ffn_down_shexp", silu(self._lin(f"blk.{i}.ffn_gate_shexp", x)) * self._lin(f"blk.{i}.ffn_up_shexp", x))
    gate = self.w.get(f"blk.{i}.ffn_gate_inp_shexp.weight")
    if gate is not None: sh = sh * (1.0 / (1.0 + np.exp(-(x * gate.astype(np.float32)).sum(-1, keepdims=True, dtype=np.float32))))
    return sh.astype(np.float32)

  def forward_logits(self, tokens: np.ndarray, start_pos: int) -> np.ndarray:
    """model.py:358-362 up to the logits of the last token.  tokens (1,T)."""
    c = self.cfg
    x = self.w["token_embd.weight"][tokens].astype(np.float32)
    for i in range(c.num_blocks):
      h = x + self._attention(i, rmsnorm(x, self.w[f"blk.{i}.attn_norm.weight"], c.norm_eps), start_pos)
      x = h + self._feed_forward(i, rmsnorm(h, self.w[f"blk.{i}.ffn_norm.weight"], c.norm_eps))
    return linear(rmsnorm(x[:, -1:], self.w["output_norm.weight"], c.norm_eps), self.w["output.weight"])[:, -1, :]

  def generate(self, tokens: list, n_new: int, chunk_size: int = 32, keep_logits: bool = False):
    """model.py:464-484 with temperature 0: chunked prefill, then greedy
    decode (the Gumbel term of model.py:364 is negligible against
    logits * 1e12, so the sample is the arg-max, lowest index on ties)."""
    tokens, out, logs, start_pos = list(tokens), [], [], 0
    while len(out) < n_new:
      n = min(chunk_size, len(tokens) - start_pos)
      lg = self.forward_logits(np.array([tokens[start_pos:start_pos + n]]), start_pos)
      start_pos += n
      if start_pos < len(tokens): continue
      tok = int(np.argmax(lg[0]))
      tokens.append(tok); out.append(tok)
      if keep_logits: logs.append(lg[0].copy())
    return (out, logs) if keep_logits else out
