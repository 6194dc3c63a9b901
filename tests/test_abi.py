"""CPU-side checks of the C-ABI library: it loads, exports every symbol the header
declares, and rejects bad arguments before touching a device."""
import ctypes, re, pathlib
import numpy as np
import pytest
from tinygrad_b200 import _lib, build

ROOT = pathlib.Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
  build.build_lib()
  return _lib.load()


def test_exports_every_declared_symbol(lib):
  header = (ROOT / "include" / "b200q.h").read_text()
  declared = set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", header))
  assert declared, "no declarations found in include/b200q.h"
  for name in sorted(declared):
    assert hasattr(lib, name), f"{name} is declared in b200q.h but not exported by libb200q.so"
  assert declared == set(_lib.SIGNATURES), "ctypes signatures and header disagree"


def test_header_is_plain_c_and_structs_match_ctypes(tmp_path):
  """include/b200q.h must be accepted by a C compiler (not only by nvcc reading it as C++), and the two argument structs
  must have the layout the ctypes mirrors in tinygrad_b200/_lib.py assume."""
  import shutil, subprocess
  cc, cxx = shutil.which("gcc") or shutil.which("cc"), shutil.which("g++") or shutil.which("c++")
  if not cc or not cxx: pytest.skip("no host C/C++ compiler")
  hdr = ROOT / "include" / "b200q.h"
  subprocess.run([cc, "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", str(hdr)], check=True)
  subprocess.run([cxx, "-std=c++17", "-fsyntax-only", "-x", "c++", str(hdr)], check=True)
  structs = {"b200q_gemv_args": _lib.GemvArgs, "b200q_attn_args": _lib.AttnArgs, "b200q_decode_layer": _lib.DecodeLayer,
             "b200q_decode_step_args": _lib.DecodeStepArgs, "b200q_ep_args": _lib.EpArgs}
  lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{hdr}"', 'int main(void) {']
  for cname, ct in structs.items():
    lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
    for fname, _ in ct._fields_: lines.append(f'  printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
  lines += ['  return 0;', '}']
  src = tmp_path / "layout.c"
  src.write_text("\n".join(lines))
  subprocess.run([cc, "-std=c11", "-o", str(tmp_path / "layout"), str(src)], check=True)
  got = dict(l.split() for l in subprocess.run([str(tmp_path / "layout")], check=True, capture_output=True, text=True).stdout.splitlines())
  for cname, ct in structs.items():
    assert int(got[cname]) == ctypes.sizeof(ct), cname
    for fname, _ in ct._fields_: assert int(got[f"{cname}.{fname}"]) == getattr(ct, fname).offset, f"{cname}.{fname}"


def test_strerror_and_version(lib):
  assert lib.b200q_version() >= 1
  assert lib.b200q_strerror(0) == b"ok"
  for code in range(-6, 0): assert b"unknown b200q" not in lib.b200q_strerror(code)
  assert b"unknown b200q" in lib.b200q_strerror(-99)


def test_packed_bytes(lib):
  assert lib.b200q_packed_bytes(_lib.Q4_0, 4096, 4096) == 4096 * 4096 // 32 * 18   # exactly the GGUF bytes
  assert lib.b200q_packed_bytes(_lib.Q8_0, 4096, 4096) == 4096 * 4096 // 32 * 34
  assert lib.b200q_packed_bytes(_lib.Q4_0, 17, 96) == 2 * 1 * 1152                 # padded to 32 rows x 128 columns
  assert lib.b200q_packed_bytes(_lib.Q6_K, 16, 256) == 2 * 1696                     # 106 bytes per row and half super-block
  assert lib.b200q_packed_bytes(_lib.Q6_K, 16, 128) == 0 and lib.b200q_packed_bytes(12, 16, 256) == 0   # not whole super-blocks; no fused Q4_K
  assert lib.b200q_packed_bytes(_lib.Q4_0, 0, 128) == 0


def test_workspace_sizes(lib):
  assert lib.b200q_qgemm_workspace_bytes(511, 4096) == 4 * 32 * 2 * 32768      # 4 row tiles x 32 column groups x (hi, lo) x 32 KB
  assert lib.b200q_qgemm_workspace_bytes(1, 96) == 2 * 32768 and lib.b200q_qgemm_workspace_bytes(0, 4096) == 0
  assert lib.b200q_qgemm_ws(_lib.Q4_0, 16, 16, _lib.F32, None, None, 0, 16, _lib.F32, 4, 16, 128, 16, 100, None) == -6     # workspace too small
  assert lib.b200q_qgemm_ws(_lib.Q4_0, 16, 16, _lib.F32, None, None, 0, 16, _lib.F32, 4, 16, 128, None, 1 << 20, None) == -1
  assert lib.b200q_fp8_absmax(None, _lib.F32, 8, 16, None) == -1 and lib.b200q_fp8_scale_bias(16, 0, 8, 16, 16, None, 16, _lib.F32, None) == -1


def test_bad_arguments_are_rejected_without_a_device(lib):
  assert lib.b200q_dequant_raw(5, 16, 16, 32, _lib.F32, None) == -1          # unknown type
  assert lib.b200q_dequant_raw(_lib.Q4_0, 16, 16, 33, _lib.F32, None) == -2  # not whole blocks
  assert lib.b200q_dequant_raw(_lib.Q6_K, 16, 16, 128, _lib.F32, None) == -2
  assert lib.b200q_dequant_raw(_lib.Q4_0, None, None, 0, _lib.F32, None) == 0  # empty input is fine
  assert lib.b200q_repack(_lib.Q4_0, None, None, 16, 16, 32, None) == -1
  assert lib.b200q_repack(_lib.Q4_0, 16, None, 16, 16, 48, None) == -2
  assert lib.b200q_repack(_lib.Q4_0, 16, None, 8, 16, 32, None) == -3        # packed buffer must be 16-byte aligned
  assert lib.b200q_repack(_lib.Q6_K, 16, 16, 16, 16, 256, None) == -4        # no interleaved gate / up tiles for Q6_K
  assert lib.b200q_repack(_lib.Q6_K, 16, None, 16, 16, 128, None) == -2
  a = _lib.GemvArgs(_lib.Q4_0, 16, 128, 1, 16, 16, _lib.F32, _lib.F32, None, 0.0, 0, None, None, 16, 0, 0, None, None, 0, None, None, None, 0.0)
  a.n_in = 100
  assert lib.b200q_gemv(ctypes.byref(a), None) == -2
  a.n_in, a.w_packed = 128, 8
  assert lib.b200q_gemv(ctypes.byref(a), None) == -3
  a.w_packed, a.y = 16, None
  assert lib.b200q_gemv(ctypes.byref(a), None) == -1
  at = _lib.AttnArgs(16, 16, 16, _lib.F16, 16, 16, 16, 16, 6, 4, 128, 128, 64, 4, 0, None)
  assert lib.b200q_attn_min_split(2048) == 32 and lib.b200q_attn_min_split(65) == 2
  assert lib.b200q_attn_decode(ctypes.byref(at), None) == -1                 # heads not a multiple of kv heads
  at.n_heads, at.head_dim = 8, 100
  assert lib.b200q_attn_decode(ctypes.byref(at), None) == -2
  at.head_dim, at.max_context = 128, 1000                                    # 4 slices of 64 do not cover 1000 positions
  assert lib.b200q_attn_decode(ctypes.byref(at), None) == -2
  a.y, a.xq_out, a.n_out = 16, 32, 200                                       # a record needs whole groups of 128 outputs
  assert lib.b200q_gemv(ctypes.byref(a), None) == -2
  assert lib.b200q_xq_bytes(4096) == 32 * 320 and lib.b200q_xq_bytes(100) == 320 and lib.b200q_xq_bytes(0) == 0
  assert lib.b200q_graph_begin(None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
  monkeypatch.setattr(_lib, "_lib", None)
  monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
  with pytest.raises(_lib.B200QError): _lib.load()


def test_step_past_the_context_end_raises_before_any_launch():
  """The host mirrors the device position: a step with no KV-cache row left raises and launches nothing
  (the object below has no device state at all, so any launch attempt would fail differently)."""
  from tinygrad_b200.model import Transformer
  m = Transformer.__new__(Transformer)
  m.max_context, m._host_pos, m.is_moe, m.use_graph = 64, 64, False, True
  with pytest.raises(RuntimeError, match="context full"): m.step()
  with pytest.raises(RuntimeError, match="context full"): m.decode_batch_step()
  assert m._host_pos == 64
