"""Device memory, streams, events and CUDA graphs over the C ABI (numpy on the host side).

This is the only CUDA binding the package uses: no other framework sits between
the Python host code and libb200q.so.  A caller that already owns device memory
(a tinygrad Tensor's `Buffer._buf`, any object with `data_ptr()`) can pass raw
addresses to the ops instead; see `ptr_of`.
"""
import ctypes
import numpy as np
from . import _lib
from ._lib import check


def ptr_of(obj) -> int:
  """Raw device address of a DeviceBuffer, an int, None, or a foreign tensor."""
  if obj is None: return 0
  if isinstance(obj, int): return obj
  if isinstance(obj, DeviceBuffer): return obj.ptr
  if hasattr(obj, "ptr"): return int(obj.ptr)
  if hasattr(obj, "data_ptr"): return int(obj.data_ptr())
  if hasattr(obj, "__cuda_array_interface__"): return int(obj.__cuda_array_interface__["data"][0])
  raise TypeError(f"cannot take a device pointer from {type(obj)}")


class DeviceBuffer:
  """Owning device allocation with an optional (shape, dtype) view for copies to numpy."""
  def __init__(self, nbytes: int, shape=None, dtype=None, zero: bool = False):
    p = ctypes.c_void_p()
    check(_lib.load().b200q_malloc(ctypes.byref(p), nbytes))
    self.ptr, self.nbytes, self.shape, self.dtype = int(p.value), int(nbytes), shape, np.dtype(dtype) if dtype is not None else None
    if zero: self.zero_()

  @staticmethod
  def empty(shape, dtype, zero: bool = False) -> "DeviceBuffer":
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    return DeviceBuffer(int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize, shape, dtype, zero)

  @staticmethod
  def from_numpy(a: np.ndarray) -> "DeviceBuffer":
    a = np.ascontiguousarray(a)
    b = DeviceBuffer(max(a.nbytes, 1), a.shape, a.dtype)
    b.copy_from(a)
    return b

  def copy_from(self, a: np.ndarray, stream=None, offset: int = 0) -> None:
    a = np.ascontiguousarray(a)
    assert offset + a.nbytes <= self.nbytes, "host array larger than the device buffer"
    check(_lib.load().b200q_memcpy_h2d(self.ptr + offset, a.ctypes.data, a.nbytes, stream_ptr(stream)))
    if stream is None: check(_lib.load().b200q_device_synchronize())

  def numpy(self, shape=None, dtype=None, offset: int = 0) -> np.ndarray:
    shape = self.shape if shape is None else ((shape,) if isinstance(shape, int) else tuple(shape))
    dtype = self.dtype if dtype is None else np.dtype(dtype)
    out = np.empty(shape, dtype=dtype)
    assert offset + out.nbytes <= self.nbytes
    check(_lib.load().b200q_device_synchronize())
    check(_lib.load().b200q_memcpy_d2h(out.ctypes.data, self.ptr + offset, out.nbytes, None))
    check(_lib.load().b200q_device_synchronize())
    return out

  def zero_(self, stream=None) -> None:
    check(_lib.load().b200q_memset(self.ptr, 0, self.nbytes, stream_ptr(stream)))

  def free(self) -> None:
    if self.ptr:
      _lib.load().b200q_free(self.ptr)
      self.ptr = 0

  def __del__(self):
    try: self.free()
    except Exception: pass


class PinnedBuffer:
  """Page-locked host memory viewed as a numpy array (source/target of async copies)."""
  def __init__(self, shape, dtype):
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    self.nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
    p = ctypes.c_void_p()
    check(_lib.load().b200q_host_alloc(ctypes.byref(p), self.nbytes))
    self.ptr = int(p.value)
    self.array = np.frombuffer((ctypes.c_char * self.nbytes).from_address(self.ptr), dtype=dtype).reshape(shape)

  def free(self) -> None:
    if self.ptr:
      self.array = None
      _lib.load().b200q_host_free(self.ptr)
      self.ptr = 0


def stream_ptr(stream) -> int:
  return 0 if stream is None else (stream.ptr if isinstance(stream, Stream) else int(stream))


class Stream:
  def __init__(self, ptr: int = None):
    """A new non-blocking stream, or a view of an existing `cudaStream_t` (e.g. the stream NCCL calls are issued on)."""
    if ptr is not None:
      self.ptr = int(ptr)
      return
    p = ctypes.c_void_p()
    check(_lib.load().b200q_stream_create(ctypes.byref(p)))
    self.ptr = int(p.value)
  def synchronize(self) -> None: check(_lib.load().b200q_stream_synchronize(self.ptr))


class Event:
  def __init__(self):
    p = ctypes.c_void_p()
    check(_lib.load().b200q_event_create(ctypes.byref(p)))
    self.ptr = int(p.value)
  def record(self, stream=None) -> None: check(_lib.load().b200q_event_record(self.ptr, stream_ptr(stream)))
  def synchronize(self) -> None: check(_lib.load().b200q_event_synchronize(self.ptr))
  def elapsed_ms(self, stop: "Event") -> float:
    ms = ctypes.c_float()
    check(_lib.load().b200q_event_elapsed_ms(self.ptr, stop.ptr, ctypes.byref(ms)))
    return float(ms.value)


class Graph:
  """Stream capture of a fixed launch sequence, replayed with one call: the role
  TinyJit + CUDAGraph play for the reference's decode loop (tinygrad/engine/jit.py:241-291)."""
  def __init__(self, stream: Stream):
    self.stream, self.exec = stream, 0
  def __enter__(self):
    check(_lib.load().b200q_graph_begin(self.stream.ptr))
    return self
  def __exit__(self, et, ev, tb):
    p = ctypes.c_void_p()
    rc = _lib.load().b200q_graph_end(self.stream.ptr, ctypes.byref(p))
    if et is None: check(rc)
    self.exec = int(p.value or 0)
    return False
  def launch(self, stream=None) -> None:
    check(_lib.load().b200q_graph_launch(self.exec, stream_ptr(stream if stream is not None else self.stream)))


def synchronize() -> None: check(_lib.load().b200q_device_synchronize())


def set_device(i: int) -> None: check(_lib.load().b200q_set_device(i))


def device_count() -> int:
  n = ctypes.c_int()
  check(_lib.load().b200q_device_count(ctypes.byref(n)))
  return n.value


def device_props(i: int = 0) -> dict:
  sm, ma, mi, mem = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_size_t()
  check(_lib.load().b200q_device_props(i, ctypes.byref(sm), ctypes.byref(ma), ctypes.byref(mi), ctypes.byref(mem)))
  return {"sm_count": sm.value, "cc": (ma.value, mi.value), "total_mem": mem.value}


def device_status() -> int:
  """0 = fine; 1 = a bounded wait inside a kernel ran out since the last call (reads and clears the word)."""
  st = ctypes.c_int()
  check(_lib.load().b200q_status_read_clear(ctypes.byref(st)))
  return st.value


def mx_status() -> int:
  """The same word for the tcgen05 MXFP8 kernels (reads and clears it)."""
  st = ctypes.c_int()
  check(_lib.load().b200q_mx_status_read_clear(ctypes.byref(st)))
  return st.value
