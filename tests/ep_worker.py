"""Run under torch.distributed.run with >= 2 ranks (one per GPU): the expert-parallel MXFP8 MoE FFN on token shards, checked on
every rank against the single-GPU MxMoE run on all tokens (which the same rank computes for itself).  Exit code 0 = bit-identical."""
import os, sys, pathlib, time
sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent))
import numpy as np


def main():
  from tinygrad_b200 import build, runtime, moe, expert_parallel as ep
  from tinygrad_b200.replicas import Ranks
  from tinygrad_b200.runtime import DeviceBuffer
  build.build_lib()
  ranks = Ranks(backend="nccl")
  runtime.set_device(ranks.local)
  G, r = ranks.world, ranks.rank
  big = "--bench" in sys.argv
  T, D, F, E, k = (4096, 2048, 1024, 64, 8) if big else (64 * G + 8 * G, 256, 128, 4 * G, 2)
  rng = np.random.default_rng(7)                                   # every rank draws the same full problem
  wg, wu, wd = ((rng.standard_normal(s, dtype=np.float32) * 0.05) for s in ((E, F, D), (E, F, D), (E, D, F)))
  x = moe.to_bf16_bits(rng.standard_normal((T, D), dtype=np.float32))
  logits = rng.standard_normal((T, E), dtype=np.float32)
  T_l, E_l = T // G, E // G
  from tinygrad_b200 import tensor_parallel as tpar
  sl = slice(r * E_l, (r + 1) * E_l)
  for mode, kind in ([(1, "peer"), (1, "nccl")] if big else [(0, "peer"), (1, "peer"), (0, "nccl"), (1, "nccl")]):
    if kind == "peer":
      shard = ep.PeerExpertParallelMoE(tpar.TPGroup(ranks, "peer"), wg[sl], wu[sl], wd[sl], E, k, T, mode)
      shard.connect()
    else: shard = ep.ExpertParallelMoE(ranks, wg[sl], wu[sl], wd[sl], E, k, T, mode)
    ranks.barrier()
    dx, dl = DeviceBuffer.from_numpy(x[r * T_l:(r + 1) * T_l]), DeviceBuffer.from_numpy(logits[r * T_l:(r + 1) * T_l])
    out = shard(dx, dl, T_l).numpy()
    if big:
      import torch
      for _ in range(3): shard(dx, dl, T_l)
      ranks.barrier(); torch.cuda.synchronize()
      t0 = time.perf_counter()
      for _ in range(10): shard(dx, dl, T_l)
      torch.cuda.synchronize(); ranks.barrier()
      ms = ranks.max((time.perf_counter() - t0) * 1e3 / 10)
      if r == 0: print(f"ep bench [{kind}]: {G} ranks, {T} tokens, {ms:.3f} ms per layer, {T * k * 3 * 2 * D * F / ms / 1e9:.1f} TFLOP/s useful", flush=True)
    full = moe.MxMoE(wg, wu, wd, k, mode)
    ref = full(DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(logits), T).numpy()[r * T_l:(r + 1) * T_l]
    if not np.array_equal(out, ref):
      bad = int((out != ref).sum())
      print(f"rank {r} mode {mode} kind {kind}: status {runtime.mx_status()}, {bad} of {out.size} bf16 values differ from the single-GPU result", flush=True)
      os._exit(1)
    if runtime.mx_status() != 0:
      print(f"rank {r} mode {mode} kind {kind}: a bounded wait ran out", flush=True)
      os._exit(1)
  ranks.barrier()
  if r == 0: print(f"ep ok {G}", flush=True)
  os._exit(0)


if __name__ == "__main__":
  main()
