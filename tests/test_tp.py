"""Tensor-parallel decode: the sharding arithmetic on CPU, and a 2-GPU run against the oracle where two GPUs exist."""
import os, subprocess, sys, pathlib
import numpy as np
import pytest
from oracle import ggml_quant as gq
from tinygrad_b200 import synth

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("typ,blk", [(2, 18), (8, 34)])
def test_shards_recompose_the_full_linears(typ, blk):
  """Column-split outputs concatenate, row-split partial products sum: the identities the all-reduce relies on."""
  from tinygrad_b200.model import TransformerConfig
  from tinygrad_b200 import tensor_parallel as tpar
  cfg = TransformerConfig(num_blocks=1, dim=256, hidden_dim=512, n_heads=4, n_kv_heads=2, norm_eps=1e-5, vocab_size=64, head_dim=64, rope_theta=1e4,
                          rope_dim=64, max_context=16, qkv_bias=True)
  sd = synth.dense_model_raw(cfg, typ, seed=1)
  tp = 2
  lc = tpar.local_config(cfg, tp)
  assert (lc.n_heads, lc.n_kv_heads, lc.hidden_dim, lc.vocab_size, lc.dim) == (2, 1, 256, 32, 256)
  shards = [tpar.shard_state_dict(sd, cfg, r, tp, blk) for r in range(tp)]
  full = {n: gq.weight_matrix(sd[n + ".weight"], o, i, typ) for n, o, i in synth.linear_names(cfg)}
  loc = [{n: gq.weight_matrix(s[n + ".weight"], o, i, typ) for n, o, i in synth.linear_names(lc)} for s in shards]
  rng = np.random.default_rng(0)
  x = rng.standard_normal(cfg.dim).astype(np.float32)
  for n in ("blk.0.attn_q", "blk.0.attn_k", "blk.0.attn_v", "blk.0.ffn_gate", "blk.0.ffn_up", "output"):
    np.testing.assert_array_equal(np.concatenate([l[n] @ x for l in loc]), full[n] @ x)
  a = rng.standard_normal(cfg.n_heads * cfg.head_dim).astype(np.float32)
  np.testing.assert_allclose(sum(l["blk.0.attn_output"] @ a[r * 128:(r + 1) * 128] for r, l in enumerate(loc)), full["blk.0.attn_output"] @ a, rtol=1e-5, atol=1e-5)
  h = rng.standard_normal(cfg.hidden_dim).astype(np.float32)
  np.testing.assert_allclose(sum(l["blk.0.ffn_down"] @ h[r * 256:(r + 1) * 256] for r, l in enumerate(loc)), full["blk.0.ffn_down"] @ h, rtol=1e-5, atol=1e-5)
  np.testing.assert_array_equal(np.concatenate([s["blk.0.attn_q.bias"] for s in shards]), sd["blk.0.attn_q.bias"])
  assert shards[0]["token_embd.weight"] is sd["token_embd.weight"]          # replicated


@pytest.mark.gpu
def test_two_gpu_tensor_parallel_stream_matches_oracle():
  from tinygrad_b200 import build, runtime
  build.build_lib()
  if runtime.device_count() < 2: pytest.skip("needs two GPUs")
  env = dict(os.environ, NCCL_NVLS_ENABLE="0")
  r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                      "--master-port", "29533", str(ROOT / "tests" / "tp_worker.py")], capture_output=True, text=True, timeout=300, env=env)
  assert r.returncode == 0 and "tp ok 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
