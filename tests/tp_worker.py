"""Run under torch.distributed.run with >= 2 ranks (one per GPU): tensor-parallel greedy decode of a mid-size model, with the
library's own peer-memory collectives and with NCCL, checked on every rank against the numpy oracle of the unsharded model.
Exit code 0 = identical token stream."""
import os, sys, pathlib
sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent))
import numpy as np


def main():
  from tinygrad_b200 import build, runtime, synth, tensor_parallel as tpar
  from tinygrad_b200.replicas import Ranks
  from tinygrad_b200.model import Transformer, TransformerConfig
  from oracle import llm, ggml_quant as gq
  build.build_lib()
  ranks = Ranks(backend="nccl")
  runtime.set_device(ranks.local)
  kinds = [k for k in ("peer", "nccl") if f"--only-{k}" in sys.argv] or ["peer", "nccl"]
  for kind, typ, blk_bytes, use_graph in [(k, *cfg3) for k in kinds for cfg3 in ((2, 18, False), (2, 18, True), (8, 34, True))]:
    tp = tpar.TPGroup(ranks, kind)
    kw = dict(num_blocks=3, dim=512, hidden_dim=1536, n_heads=8, n_kv_heads=4, norm_eps=1e-5, vocab_size=2048, head_dim=64, rope_theta=500000.0,
              rope_dim=64, max_context=128, qkv_bias=(typ == 8), kv_dtype="float16")
    cfg = TransformerConfig(**kw)
    sd = synth.dense_model_raw(cfg, typ, seed=21, embd_std=0.3, scale_std=0.02 if typ == 2 else 0.0015)
    shapes = {n: (o, i) for n, o, i in synth.linear_names(cfg)}
    w = {k: (gq.weight_matrix(v, *shapes[k[:-7]], typ) if v.dtype == np.uint8 else v) for k, v in sd.items()}
    prompt = [int(t) for t in np.random.default_rng(3).integers(0, 2048, 20)]
    want, want_logits = llm.Transformer(llm.Config(**kw), w).generate(prompt, 12, keep_logits=True)
    m = Transformer(cfg, tpar.shard_state_dict(sd, cfg, ranks.rank, ranks.world, blk_bytes), ggml_type=typ, tp=tp, use_graph=use_graph)
    got = []
    for i, tok in enumerate(m.generate(list(prompt))):
      lg = m.read_logits()
      err = np.abs(lg - want_logits[i])
      assert (err <= 3e-2 + 3e-2 * np.abs(want_logits[i])).all(), f"rank {ranks.rank}: logits off at step {i}: {err.max()}"
      got.append(tok)
      if len(got) == 12: break
    assert got == want, f"rank {ranks.rank} type {typ}: {got} != {want}"
    assert runtime.device_status() == 0
    if ranks.rank == 0: print("config ok", kind, typ, use_graph, flush=True)
  ranks.barrier()
  if ranks.rank == 0: print("tp ok", ranks.world, flush=True)
  os._exit(0)     # captured graphs hold NCCL work: leave without tearing the process group down


if __name__ == "__main__":
  main()
