"""Build libb200q.so (the sm_100a kernels + C ABI) in-tree with nvcc."""
import os, pathlib, shutil, subprocess, sys

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libb200q.so"
SOURCES = ["api.cu", "quant_pack.cu", "gemv.cu", "decode.cu", "decode_step.cu", "mxfp8.cu", "mxfp8_gemm.cu", "tc_gemm.cu", "dense.cu", "prefill.cu", "tg_kernels.cu", "peer.cu", "ep.cu", "fp8.cu", "gemv_rows.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC", "-cudart", "shared"]


def nvcc_path() -> str:
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand): return cand
  raise RuntimeError("nvcc not found: set NVCC or put the CUDA toolkit on PATH")


def build_lib(force: bool = False, verbose: bool = False) -> pathlib.Path:
  srcs = [CSRC / s for s in SOURCES]
  deps = srcs + [CSRC / "common.cuh", CSRC / "actquant.cuh", CSRC / "mxq.cuh", CSRC / "qgemv_core.cuh", PKG.parent / "include" / "b200q.h"]
  if not force and LIB.exists() and all(LIB.stat().st_mtime >= d.stat().st_mtime for d in deps): return LIB
  cmd = [nvcc_path(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB), *map(str, srcs)]
  r = subprocess.run(cmd, capture_output=True, text=True)
  if verbose: print(r.stderr)
  if r.returncode != 0: raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
  return LIB


CUBIN = PKG / "tg_kernels.cubin"


def build_cubin(force: bool = False) -> pathlib.Path:
  """The entry kernels tinygrad's own runtime launches (tinygrad_b200/tg_op.py), as a cubin for sm_100a."""
  src = CSRC / "tg_kernels.cu"
  deps = [src, CSRC / "common.cuh", CSRC / "actquant.cuh", CSRC / "qgemv_core.cuh"]
  if not force and CUBIN.exists() and all(CUBIN.stat().st_mtime >= d.stat().st_mtime for d in deps): return CUBIN
  cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-cubin", "-o", str(CUBIN), str(src)]
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0: raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
  return CUBIN


if __name__ == "__main__":
  print(build_lib(force=True, verbose="-v" in sys.argv))
  print(build_cubin(force=True))
