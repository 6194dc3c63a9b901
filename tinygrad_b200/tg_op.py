"""The quantised Linear as an op INSIDE tinygrad's graph: takes and returns tinygrad Tensors.

`Tensor.custom_kernel(out, x, w_packed, meta, fxn=...)` (tinygrad/tensor.py:390-396 -> UOp.custom_kernel,
tinygrad/uop/ops.py:1189-1192) accepts a function that returns a ready-made `Ops.PROGRAM` whose sources are
(SINK, LINEAR, SOURCE, BINARY); a PROGRAM that carries a `ProgramInfo` and a BINARY is treated as compiled
(tinygrad/engine/realize.py:256-261), so the scheduler, `TinyJit` and the CUDA graph runner launch OUR cubin like any kernel
of their own.  Precedent in the reference: extra/gemm/moe_gemm.py:30-48 (a HIP kernel wrapped the same way).

Two things differ from that precedent, both on purpose:
  * the PROGRAM gets an explicit `ProgramInfo` (tinygrad/uop/ops.py:1213-1221).  The one `ProgramInfo.from_sink` would infer from a
    bare sink has no `outs` / `ins` (it looks for STORE / LOAD uops, :1248-1251), and the JIT's graph builder takes its node
    dependencies from `outs` (tinygrad/runtime/graph/cuda.py:22): without them a consumer captured in the same graph would not
    wait for this kernel;
  * sizes travel in a small int32 tensor (`meta`), because the launcher passes tensors and bound variables only
    (tinygrad/runtime/ops_cuda.py:18-24) and `custom_kernel` wants concrete shapes.

tinygrad is imported lazily and only here: the rest of the package does not depend on it.  `B200QLinear` mirrors
`nn.Linear.__call__(x)` (tinygrad/nn/__init__.py:177) for a GGUF Q4_0 / Q8_0 weight: x (..., in_features) float32 ->
(..., out_features) float32.  The weight is re-tiled once, by the library, into a uint8 Tensor the object keeps.
"""
from __future__ import annotations
import functools, pathlib
import numpy as np

CUBIN_PATH = pathlib.Path(__file__).resolve().parent / "tg_kernels.cubin"
KERNEL_NAMES = {2: "b200q_tg_gemv_q4_0", 8: "b200q_tg_gemv_q8_0"}
TG_THREADS, TG_WARPS = 256, 8
BLOCK_BYTES = {2: 18, 8: 34}


@functools.cache
def _cubin() -> bytes:
  if not CUBIN_PATH.exists(): raise RuntimeError(f"{CUBIN_PATH} is missing: run `python -m tinygrad_b200.build` (there is no fallback kernel)")
  return CUBIN_PATH.read_bytes()


def launch_dims(n_out: int, m: int) -> tuple:
  """(global_size, local_size) of b200q_tg_gemv_*: one warp per 16-row tile, 8 warps per block, one grid row per activation row."""
  row_tiles = -(-n_out // 16)
  return (-(-row_tiles // TG_WARPS), m, 1), (TG_THREADS, 1, 1)


def gemv_program(out, x, w, meta, *, qtype: int, n_out: int, n_in: int, m: int, target):
  """The `fxn` of Tensor.custom_kernel: placeholders of (out, x, w_packed, meta) -> a compiled Ops.PROGRAM."""
  from tinygrad.uop.ops import UOp, Ops, KernelInfo, ProgramInfo
  from tinygrad.renderer import Estimates
  name = KERNEL_NAMES[qtype]
  gsz, lsz = launch_dims(n_out, m)
  wbytes = n_out * n_in // 32 * BLOCK_BYTES[qtype]
  sink = UOp.sink(out.base, x.base, w.base, meta.base, UOp.special(lsz[0], "lidx0"), UOp.special(gsz[0], "gidx0"), UOp.special(gsz[1], "gidx1"),
                  arg=KernelInfo(name, estimates=Estimates(ops=2 * m * n_out * n_in, mem=wbytes + 4 * m * (n_in + n_out))))
  info = ProgramInfo(name, gsz, lsz, (), (0, 1, 2, 3), (0,), (1, 2, 3), target)      # slot 0 is written, slots 1-3 are read
  return UOp(Ops.PROGRAM, src=(sink, UOp(Ops.LINEAR, src=(*sink.src, sink)), UOp(Ops.SOURCE, arg=f"// prebuilt sm_100a cubin: {name}"),
                               UOp(Ops.BINARY, arg=_cubin())), arg=info)


def _target_of(device: str):
  from tinygrad import Device
  return Device[device.split(",")[0] if isinstance(device, str) else device[0]].renderer.target


def quant_linear(x, w_packed, meta, qtype: int, n_out: int, n_in: int):
  """x: Tensor (..., n_in) float32 on a CUDA / NV device; w_packed: uint8 Tensor of packed tiles; meta: int32 Tensor {n_out, n_in, m}.
  Returns a Tensor (..., n_out) float32 that depends on the kernel (so the scheduler orders and the JIT captures it)."""
  from tinygrad import Tensor, dtypes
  lead = tuple(x.shape[:-1])
  m = int(np.prod(lead, dtype=np.int64)) if lead else 1
  x2 = x.reshape(m, n_in).cast(dtypes.float32).contiguous()
  out = Tensor.empty(m, n_out, dtype=dtypes.float32, device=x.device)
  fxn = functools.partial(gemv_program, qtype=qtype, n_out=n_out, n_in=n_in, m=m, target=_target_of(x.device))
  out = Tensor.custom_kernel(out, x2, w_packed, meta, fxn=fxn)[0]
  return out.reshape(*lead, n_out)


def pack_weight_host(raw: np.ndarray, n_out: int, n_in: int, qtype: int) -> np.ndarray:
  """Raw GGUF blocks -> the packed tile layout, through the library's repack kernel (needs a GPU); returns the bytes on the host."""
  from . import quant
  return quant.repack(raw, n_out, n_in, qtype).buf.numpy((quant.packed_bytes(qtype, n_out, n_in),), np.uint8)


class B200QLinear:
  """Drop-in for `nn.Linear` on a GGUF Q4_0 / Q8_0 weight inside a tinygrad model (swap it in place of the Linear object, as
  extra/fp8/fp8_linear.py:65-101 swaps its FP8Linear).  `packed`: the packed tiles as a numpy uint8 array (pack_weight_host) or
  a uint8 Tensor already on the device."""
  def __init__(self, in_features: int, out_features: int, ggml_type: int, packed, bias=None, device=None):
    if ggml_type not in KERNEL_NAMES: raise ValueError(f"GGML type '{ggml_type}' has no in-graph kernel (Q4_0 and Q8_0 do)")
    from tinygrad import Tensor
    self.in_features, self.out_features, self.ggml_type = in_features, out_features, ggml_type
    self.weight_packed = packed if isinstance(packed, Tensor) else Tensor(np.ascontiguousarray(packed, dtype=np.uint8), device=device)
    self.bias = bias
    self._meta = {}

  def _meta_for(self, m: int, device):
    from tinygrad import Tensor, dtypes
    if (m, device) not in self._meta:
      self._meta[(m, device)] = Tensor(np.array([self.out_features, self.in_features, m], dtype=np.int32), device=device).realize()
    return self._meta[(m, device)]

  def __call__(self, x):
    lead = tuple(x.shape[:-1])
    m = int(np.prod(lead, dtype=np.int64)) if lead else 1
    y = quant_linear(x, self.weight_packed, self._meta_for(m, x.device), self.ggml_type, self.out_features, self.in_features)
    return y if self.bias is None else y + self.bias
