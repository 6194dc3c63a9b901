"""The in-graph seam on CPU: our prebuilt cubin as an `Ops.PROGRAM` inside tinygrad's scheduler and JIT.

Runs the reference itself (imported from a checkout on disk; skipped where there is none) on its compile-only device
`DEV=NULL:CUDA:sm_100`, which schedules, lowers and "launches" without a GPU.  What is checked is everything that happens
before a launch: the op is accepted by `Tensor.custom_kernel`, is not re-compiled, survives `TinyJit` capture, and carries the
write / read slots from which the JIT's graph runner derives the edge to the kernel that consumes its output."""
import os, pathlib, subprocess, sys, textwrap
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
REF = pathlib.Path(os.environ.get("TINYGRAD_REF", "/root/reference"))

SCRIPT = textwrap.dedent('''
  import os, sys
  os.environ["DEV"] = "NULL:CUDA:sm_100"
  sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
  import numpy as np
  from tinygrad import Tensor, TinyJit
  from tinygrad.uop.ops import Ops, ProgramInfo
  from tinygrad_b200 import tg_op

  n_out, n_in = 4096, 4096
  lin = tg_op.B200QLinear(n_in, n_out, 2, np.zeros(n_out * n_in // 32 * 18, np.uint8))
  y = lin(Tensor.empty(1, 1, n_in))
  assert y.shape == (1, 1, n_out), y.shape
  y.realize()                                                  # eager: scheduled and handed to the (null) runtime

  @TinyJit
  def step(x): return (lin(x) * 2.0).realize()                 # a consumer kernel right behind ours
  for _ in range(4): out = step(Tensor.empty(1, 1, n_in).realize())
  assert out.shape == (1, 1, n_out)
  calls = []
  for c in step.captured._linear.src:                          # graph batches wrap their calls in CUSTOM_FUNCTION("graph")
    a0 = c.src[0]
    calls += list(a0.src[0].src) if a0.op is Ops.CUSTOM_FUNCTION else [c]
  ours = [c for c in calls if c.src[0].op is Ops.PROGRAM and c.src[0].arg.name == "b200q_tg_gemv_q4_0"]
  assert len(ours) == 1, [getattr(c.src[0].arg, "name", None) for c in calls]
  prg = ours[0].src[0]
  assert isinstance(prg.arg, ProgramInfo) and prg.src[-1].op is Ops.BINARY and prg.src[-1].arg[:4] == b"\\x7fELF"
  assert prg.arg.outs == (0,) and prg.arg.ins == (1, 2, 3) and prg.arg.globals == (0, 1, 2, 3) and prg.arg.vars == ()
  assert prg.arg.global_size == (32, 1, 1) and prg.arg.local_size == (256, 1, 1), (prg.arg.global_size, prg.arg.local_size)
  # the consumer reads the buffer our kernel writes (slot 0): with outs = (0,) the graph runner orders it behind us
  out_buf = ours[0].src[1]
  after = calls[calls.index(ours[0]) + 1:]
  assert any(any(b is out_buf for b in c.src[1:]) for c in after), "no captured kernel consumes the op's output buffer"
  # Q8_0 and several activation rows take the same route
  lin8 = tg_op.B200QLinear(512, 96, 8, np.zeros(96 * 512 // 32 * 34, np.uint8))
  assert lin8(Tensor.empty(2, 3, 512)).realize().shape == (2, 3, 96)
  assert tg_op.launch_dims(96, 6) == ((1, 6, 1), (256, 1, 1))
  print("TG_OP_OK")
''')


def test_quant_linear_is_a_tinygrad_op_on_the_null_cuda_device(tmp_path):
  if not (REF / "tinygrad" / "tensor.py").exists(): pytest.skip("no tinygrad checkout to run the op inside")
  from tinygrad_b200 import build
  build.build_cubin()
  script = tmp_path / "tg_op_check.py"
  script.write_text(SCRIPT)
  env = {k: v for k, v in os.environ.items() if k not in ("DEV", "CUDA", "NV")}
  r = subprocess.run([sys.executable, str(script), str(REF), str(ROOT)], capture_output=True, text=True, env=env, timeout=600)
  assert r.returncode == 0 and "TG_OP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_unsupported_type_is_refused_before_tinygrad_is_touched():
  from tinygrad_b200 import tg_op
  assert tg_op.launch_dims(4096, 1) == ((32, 1, 1), (256, 1, 1))
  with pytest.raises(ValueError): tg_op.B200QLinear(256, 16, 14, b"")
