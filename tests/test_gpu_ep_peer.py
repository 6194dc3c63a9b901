"""The device-planned expert-parallel exchange (csrc/ep.cu) on ONE GPU: R ranks live in this process, each with its own buffers and
pointer tables to everybody's, and run the four stretches of a call in lock step (stretch i for all ranks before stretch i + 1, so that
no kernel waits for a launch behind it).  The result of every rank must equal the single-device MxMoE on all tokens bit for bit --
the placement the device plan derives is the one `route` gives the concatenated tokens (extra/gemm/moe_routing.py:109-131)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class _Rank:
  def __init__(self, rank, size): self.rank, self.size = rank, size
  def exchange(self, blob): raise AssertionError("ranks in one process share pointers directly")
  def barrier(self): pass


def _layers(R, T, D, F, E, k, mode, seed=11):
  from tinygrad_b200 import moe, expert_parallel as ep
  rng = np.random.default_rng(seed)
  wg, wu, wd = ((rng.standard_normal(s, dtype=np.float32) * 0.05) for s in ((E, F, D), (E, F, D), (E, D, F)))
  E_l = E // R
  shards = [ep.PeerExpertParallelMoE(_Rank(r, R), wg[r * E_l:(r + 1) * E_l], wu[r * E_l:(r + 1) * E_l], wd[r * E_l:(r + 1) * E_l], E, k, T, mode)
            for r in range(R)]
  tables = {name: [s.buf[name].ptr for s in shards] for name in ep.PeerExpertParallelMoE.SHARED}
  for s in shards: s.connect(tables)
  return shards, moe.MxMoE(wg, wu, wd, k, mode), rng


def _run(shards, xs, ls, T_l):
  for s, l in zip(shards, ls): s.route_publish(l, T_l)
  for s, x in zip(shards, xs): s.plan_dispatch(x, T_l)
  for s in shards: s.experts_signal(T_l)
  return [s.combine(T_l).numpy().copy() for s in shards]


@pytest.mark.parametrize("R,T,D,F,E,k,mode", [(2, 144, 256, 128, 8, 2, 1), (4, 288, 256, 128, 8, 2, 0), (2, 96, 512, 256, 4, 3, 1), (8, 512, 256, 128, 32, 4, 1)])
def test_virtual_ranks_match_the_single_device_layer(R, T, D, F, E, k, mode):
  from tinygrad_b200 import moe, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  shards, full, rng = _layers(R, T, D, F, E, k, mode)
  T_l = T // R
  for call in range(3):                                           # the mailboxes and flags re-arm themselves: several layers in a row
    x = moe.to_bf16_bits(rng.standard_normal((T, D), dtype=np.float32))
    logits = rng.standard_normal((T, E), dtype=np.float32)
    if call == 2: logits[:, : E // 2] -= 30.0                     # half of the experts (whole ranks) get no rows at all
    xs = [DeviceBuffer.from_numpy(x[r * T_l:(r + 1) * T_l]) for r in range(R)]
    ls = [DeviceBuffer.from_numpy(logits[r * T_l:(r + 1) * T_l]) for r in range(R)]
    outs = _run(shards, xs, ls, T_l)
    ref = full(DeviceBuffer.from_numpy(x), DeviceBuffer.from_numpy(logits), T).numpy()
    for r in range(R): np.testing.assert_array_equal(outs[r], ref[r * T_l:(r + 1) * T_l], err_msg=f"rank {r}, call {call}")
    assert runtime.mx_status() == 0
  # the plan itself against the host-side index arithmetic
  from tinygrad_b200 import expert_parallel as ep
  counts = np.stack([s._per_T[T_l]["counts"].numpy() for s in shards])
  for r, s in enumerate(shards):
    np.testing.assert_array_equal(s.off_local.numpy(), ep.exchange_plan(counts, r)["off_local"])


def test_a_wait_that_nobody_answers_runs_out_and_reports():
  """Rank 1 never dispatches: rank 0's wait for "rows landed" gives up after its limit, the call completes and the status word says so."""
  from tinygrad_b200 import moe, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  R, T, D, F, E, k = 2, 64, 256, 128, 4, 2
  shards, _, rng = _layers(R, T, D, F, E, k, 1)
  T_l = T // R
  x = DeviceBuffer.from_numpy(moe.to_bf16_bits(rng.standard_normal((T_l, D), dtype=np.float32)))
  lg = DeviceBuffer.from_numpy(rng.standard_normal((T_l, E), dtype=np.float32))
  for s in shards: s.route_publish(lg, T_l)
  shards[0].plan_dispatch(x, T_l)
  shards[0].experts_signal(T_l, spin_limit=2000)
  runtime.synchronize()
  assert runtime.mx_status() == 1
  assert runtime.mx_status() == 0


def test_bad_arguments_are_refused():
  import ctypes
  from tinygrad_b200 import _lib
  lib = _lib.load()
  a = _lib.EpArgs(n_ranks=2, rank=2, n_experts=4, k=2, d_model=256, n_tokens=8, m_max=512)
  assert lib.b200q_ep_plan(ctypes.byref(a), None) != 0
  assert lib.b200q_ep_plan(None, None) != 0
