"""One process per GPU: rank bookkeeping for the replicated (weak-scaling) decode benchmark.

The decode path of a model that fits one GPU does not shard: every rank decodes its own sequence and no data-path
collective exists.  torch.distributed is plumbing only: a barrier around the timed region and the max / sum of per-rank
scalars.  Backend "nccl" on GPUs, "gloo" on CPU (tests)."""
import os


class Ranks:
  def __init__(self, backend: str = "nccl"):
    self.rank, self.world, self.local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    self.backend, self.dist, self.torch = backend, None, None
    if self.world > 1:
      import torch, torch.distributed as dist
      self.torch, self.dist = torch, dist
      if backend == "nccl":
        torch.cuda.set_device(self.local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
      else:
        dist.init_process_group(backend)

  def _reduce(self, value: float, op) -> float:
    if self.dist is None: return float(value)
    t = self.torch.tensor([value], dtype=self.torch.float64, device="cuda" if self.backend == "nccl" else "cpu")
    self.dist.all_reduce(t, op=op)
    return float(t.item())

  def max(self, value: float) -> float: return self._reduce(value, self.dist.ReduceOp.MAX if self.dist else None)
  def sum(self, value: float) -> float: return self._reduce(value, self.dist.ReduceOp.SUM if self.dist else None)

  def barrier(self) -> None:
    if self.dist is not None: self.dist.barrier()

  def close(self) -> None:
    if self.dist is not None: self.dist.destroy_process_group()


def whole_job_rate(units_per_rank: int, ms_per_rank: float, ranks: Ranks) -> float:
  """Units all ranks processed divided by the slowest rank's time (units per second)."""
  return ranks.sum(units_per_rank) / (ranks.max(ms_per_rank) * 1e-3)
