"""Expert-parallel exchange on CPU: the index plan (pure numpy) and the two all-to-alls over two gloo ranks."""
import os, socket
import numpy as np
import pytest
from tinygrad_b200 import expert_parallel as ep


def test_exchange_plan_groups_every_row_once():
  rng = np.random.default_rng(0)
  counts = rng.integers(0, 600, (4, 16))
  counts[2, 5] = 0; counts[:, 9] = 0                                  # an empty pair and an expert nobody routes to
  for rank in range(4):
    p = ep.exchange_plan(counts, rank)
    e_l = 4
    mine = counts[:, rank * e_l:(rank + 1) * e_l]
    assert p["send_rows"].tolist() == counts[rank].reshape(4, e_l).sum(1).tolist()
    assert p["recv_rows"].tolist() == mine.sum(1).tolist()
    assert (p["off_local"] % 256 == 0).all() and p["m_local"] == p["off_local"][-1]
    assert (np.diff(p["off_local"]) >= mine.sum(0)).all() and (np.diff(p["off_local"]) - mine.sum(0) < 256).all()
    assert len(set(p["place"].tolist())) == len(p["place"]) == mine.sum()          # a permutation into distinct rows
    # arrival order is (source, expert); every row of expert e lands inside group e, sources in order
    i = 0
    for s in range(4):
      for e in range(e_l):
        rows = p["place"][i:i + mine[s, e]]; i += mine[s, e]
        assert ((rows >= p["off_local"][e]) & (rows < p["off_local"][e] + mine.sum(0)[e])).all()
        assert (np.diff(rows) == 1).all()
  assert ep.m_local_max(4096, 16, 8) == (128 + 16) * 256


def _worker(rank, world, port, out):
  os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
  import torch
  from tinygrad_b200.replicas import Ranks
  r = Ranks(backend="gloo")
  n_experts, e_l, width = 8, 4, 5
  rng = np.random.default_rng(10 + rank)
  mine_counts = rng.integers(0, 40, n_experts)
  allc = [torch.zeros(n_experts, dtype=torch.int64) for _ in range(world)]
  r.dist.all_gather(allc, torch.from_numpy(mine_counts))
  counts = np.stack([c.numpy() for c in allc])
  plan = ep.exchange_plan(counts, rank)
  # a row carries (source, expert, index within (source, expert)); the send buffer is expert-sorted
  rows = np.array([(rank, e, i, 0, 0) for e in range(n_experts) for i in range(mine_counts[e])], dtype=np.int32).reshape(-1, width)
  send, recv = torch.from_numpy(rows), torch.zeros((int(plan["recv_rows"].sum()), width), dtype=torch.int32)
  ep.all_to_all_rows(r.dist, torch, send, plan["send_rows"], recv, plan["recv_rows"])
  grouped = np.full((plan["m_local"], width), -1, np.int32)
  grouped[plan["place"]] = recv.numpy()
  ok = True
  for e in range(e_l):
    g = grouped[plan["off_local"][e]:plan["off_local"][e + 1]]
    real = g[g[:, 0] >= 0]
    ok &= bool((real[:, 1] == rank * e_l + e).all()) and len(real) == counts[:, rank * e_l + e].sum()
    ok &= bool((g[len(real):, 0] == -1).all())                                      # padding rows stay untouched
    ok &= real[:, 0].tolist() == sorted(real[:, 0].tolist())                         # sources in order inside a group
  # results go back in arrival order and arrive in the sender's own order
  back = torch.zeros_like(send)
  ep.all_to_all_rows(r.dist, torch, torch.from_numpy(grouped[plan["place"]]), plan["recv_rows"], back, plan["send_rows"])
  ok &= bool((back.numpy() == rows).all())
  out.put((rank, ok))
  r.barrier()
  r.close()


def test_two_gloo_ranks_exchange_and_regroup():
  mp = pytest.importorskip("torch.multiprocessing")
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
  ctx = mp.get_context("spawn")
  q = ctx.Queue()
  procs = [ctx.Process(target=_worker, args=(i, 2, port, q)) for i in range(2)]
  for p in procs: p.start()
  res = sorted(q.get(timeout=120) for _ in range(2))
  for p in procs: p.join(timeout=60)
  assert res == [(0, True), (1, True)]


@pytest.mark.gpu
def test_two_gpu_expert_parallel_matches_single_gpu():
  import subprocess, sys, pathlib
  from tinygrad_b200 import build, runtime
  build.build_lib()
  if runtime.device_count() < 2: pytest.skip("needs two GPUs")
  root = pathlib.Path(__file__).resolve().parent.parent
  env = dict(os.environ, NCCL_NVLS_ENABLE="0")
  r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                      "--master-port", "29541", str(root / "tests" / "ep_worker.py")], capture_output=True, text=True, timeout=300, env=env)
  assert r.returncode == 0 and "ep ok 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
