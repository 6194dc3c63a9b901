"""The peer-memory collectives on one GPU: several "ranks" live in one process, each with its own mailbox, the sharded GEMVs of
all ranks are launched first and the reducers afterwards (a reducer waits for words, so what fills them must not sit behind it in
the stream).  The arithmetic and the mailbox protocol are exactly the multi-GPU ones; only the pointers are local."""
import ctypes
import numpy as np
import pytest
from oracle import ggml_quant as gq, llm
from tinygrad_b200 import synth
from gpu_util import need_gpu, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _gpu(): need_gpu()


def _mailboxes(n_ranks, n_slots, n):
  from tinygrad_b200 import _lib
  from tinygrad_b200.runtime import DeviceBuffer, synchronize
  boxes = [DeviceBuffer(4 * n_slots * n) for _ in range(n_ranks)]
  for b in boxes: _lib.check(_lib.load().b200q_memset(b.ptr, 0xFF, b.nbytes, None))
  synchronize()
  return boxes, (ctypes.c_void_p * n_ranks)(*[b.ptr for b in boxes])


@pytest.mark.parametrize("typ,n_ranks,n_out,n_in", [(2, 2, 512, 1024), (8, 4, 200, 2048), (2, 8, 4096, 8192)])
def test_row_split_linear_all_reduce(typ, n_ranks, n_out, n_in):
  """y = W x + residual with W split by input columns over the ranks (tinygrad shards wo / w2 on that axis, examples/llama3.py:236-241):
  every rank ends with the same bits, equal to the unsharded product within the path's tolerance."""
  from tinygrad_b200 import _lib, quant, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  from tinygrad_b200.tensor_parallel import _cols
  rng = np.random.default_rng(n_out + n_ranks)
  raw = synth.BLOCK_MAKERS[typ](n_out, n_in, rng)
  x, res = rng.standard_normal(n_in).astype(np.float32), rng.standard_normal(n_out).astype(np.float32)
  kl = n_in // n_ranks
  shards = [quant.repack(_cols(raw, n_out, n_in, 18 if typ == 2 else 34, r * kl, (r + 1) * kl), n_out, kl, typ) for r in range(n_ranks)]
  boxes, targets = _mailboxes(n_ranks, n_ranks, n_out)
  for step in range(2):                       # the second step finds the mailboxes as the first one left them
    for r in range(n_ranks):
      quant.gemv(shards[r].buf.ptr, typ, n_out, kl, DeviceBuffer.from_numpy(x[r * kl:(r + 1) * kl]), None, peers=targets, peer_rank=r)
    outs = []
    for r in range(n_ranks):
      out = DeviceBuffer.from_numpy(res.copy())
      _lib.check(_lib.load().b200q_mailbox_reduce(boxes[r].ptr, n_ranks, n_out, out.ptr, out.ptr, 0, 0, None))
      outs.append(out.numpy())
    ref = llm.linear(x[None], gq.weight_matrix(raw, n_out, n_in, typ))[0] + res
    assert_close(outs[0], ref, tol=1e-2)
    assert np.abs(outs[0] - ref).max() <= 5e-4 * np.abs(ref).max()
    for o in outs[1:]: np.testing.assert_array_equal(o.view(np.uint32), outs[0].view(np.uint32))
    for b in boxes: assert (b.numpy((n_ranks * n_out,), np.uint32) == 0xFFFFFFFF).all()          # every word handed back empty
  assert runtime.device_status() == 0


def test_column_split_all_gather():
  """A vocabulary head split by output rows: every rank's slice lands in its part of the one-slot mailbox of every rank."""
  from tinygrad_b200 import _lib, quant, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  n_ranks, vocab, dim = 4, 1024, 512
  rng = np.random.default_rng(3)
  raw, x = synth.q4_0_blocks(vocab, dim, rng), rng.standard_normal(dim).astype(np.float32)
  vl = vocab // n_ranks
  rows = raw.reshape(vocab, -1)
  shards = [quant.repack(np.ascontiguousarray(rows[r * vl:(r + 1) * vl]).reshape(-1), vl, dim, 2) for r in range(n_ranks)]
  boxes, targets = _mailboxes(n_ranks, 1, vocab)
  dx = DeviceBuffer.from_numpy(x)
  for r in range(n_ranks): quant.gemv(shards[r].buf.ptr, 2, vl, dim, dx, None, peers=targets, peer_rank=r)
  ref = llm.linear(x[None], gq.weight_matrix(raw, vocab, dim, 2))[0]
  for r in range(n_ranks):
    out = DeviceBuffer.empty((vocab,), np.float32)
    _lib.check(_lib.load().b200q_mailbox_reduce(boxes[r].ptr, 1, vocab, None, out.ptr, 0, 0, None))
    assert_close(out.numpy(), ref, tol=1e-2)
  assert runtime.device_status() == 0


def test_a_word_that_never_arrives_ends_the_wait_with_a_status():
  """Failure detection without a fault: one rank's slot stays empty; the reducer gives up after its (short) limit, counts the word as
  zero, raises the status word, and the mailbox and the device stay usable."""
  from tinygrad_b200 import _lib, runtime
  from tinygrad_b200.runtime import DeviceBuffer
  lib = _lib.load()
  n = 300
  boxes, _ = _mailboxes(1, 2, n)
  got = np.arange(n, dtype=np.float32)
  _lib.check(lib.b200q_memcpy_h2d(boxes[0].ptr, got.ctypes.data, 4 * n, None))              # slot 0 arrived, slot 1 never does
  res = np.full(n, 0.5, np.float32)
  out = DeviceBuffer.empty((n,), np.float32)
  assert runtime.device_status() == 0
  _lib.check(lib.b200q_mailbox_reduce(boxes[0].ptr, 2, n, DeviceBuffer.from_numpy(res).ptr, out.ptr, 50, 0, None))
  np.testing.assert_array_equal(out.numpy(), got + 0.5)
  assert runtime.device_status() == 1 and runtime.device_status() == 0                       # raised once, cleared by the read
  full = np.stack([got, 2 * got]).astype(np.float32)
  _lib.check(lib.b200q_memcpy_h2d(boxes[0].ptr, full.ctypes.data, full.nbytes, None))        # the same mailbox, a complete delivery
  _lib.check(lib.b200q_mailbox_reduce(boxes[0].ptr, 2, n, None, out.ptr, 0, 0, None))
  np.testing.assert_array_equal(out.numpy(), 3 * got)
  assert runtime.device_status() == 0
