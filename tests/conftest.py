import pathlib, sys
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path: sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (runs the sm_100a kernels through the C-ABI)")


@pytest.fixture(scope="session")
def golden():
  import numpy as np
  def load(name):
    p = GOLDEN / f"{name}.npz"
    if not p.exists(): pytest.skip(f"golden fixture {name}.npz not generated")
    return np.load(p)
  return load
