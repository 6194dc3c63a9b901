"""The N > 1 plumbing of the benchmark on CPU: two gloo ranks, max-over-ranks timing, whole-job rate."""
import os, socket
import pytest


def _worker(rank, world, port, out):
  os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
  from tinygrad_b200.replicas import Ranks, whole_job_rate
  r = Ranks(backend="gloo")
  r.barrier()
  ms = 10.0 if rank == 0 else 25.0                       # rank 1 is the slow one
  out.put((rank, r.max(ms), r.sum(100), whole_job_rate(100, ms, r)))
  r.barrier()
  r.close()


def test_two_gloo_ranks_report_the_slowest_time_and_the_summed_work():
  mp = pytest.importorskip("torch.multiprocessing")
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  procs = [ctx.Process(target=_worker, args=(i, 2, port, q)) for i in range(2)]
  for p in procs: p.start()
  res = sorted(q.get(timeout=120) for _ in range(2))
  for p in procs: p.join(timeout=60)
  for rank, mx, sm, rate in res:
    assert mx == 25.0 and sm == 200.0 and abs(rate - 200 / 0.025) < 1e-6


def test_single_rank_needs_no_process_group(monkeypatch):
  for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"): monkeypatch.delenv(k, raising=False)
  from tinygrad_b200.replicas import Ranks, whole_job_rate
  r = Ranks()
  assert r.world == 1 and r.max(3.5) == 3.5 and whole_job_rate(10, 5.0, r) == 2000.0
