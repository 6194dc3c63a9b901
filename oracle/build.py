"""Compile the C restatement (oracle/qgemv_cpu.c) into oracle/liboracle.so.
Test infrastructure: building the checker is not using it."""
import os, pathlib, shutil, subprocess

HERE = pathlib.Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"


def build_oracle(force: bool = False) -> pathlib.Path:
  src = HERE / "qgemv_cpu.c"
  if not force and LIB.exists() and LIB.stat().st_mtime >= src.stat().st_mtime: return LIB
  errs = []
  # a compiler without its OpenMP runtime is tried last, single-threaded
  for cc in dict.fromkeys(["/usr/bin/gcc", shutil.which("gcc"), os.environ.get("CC"), "cc"]):
    if not cc: continue
    for omp in (["-fopenmp"], []):
      cmd = [cc, "-O3", "-march=x86-64-v3", *omp, "-shared", "-fPIC", "-o", str(LIB), str(src), "-lm"]
      r = subprocess.run(cmd, capture_output=True, text=True)
      if r.returncode == 0: return LIB
      errs.append(" ".join(cmd) + "\n" + r.stderr[-400:])
  raise RuntimeError("could not build the C oracle:\n" + "\n".join(errs))


if __name__ == "__main__":
  print(build_oracle(force=True))
