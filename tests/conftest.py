import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_oracle(path_name: str, env: dict | None = None):
    """Import oracle/<path_name>/model.py as a fresh module (env vars applied first)."""
    import importlib.util
    for key, val in (env or {}).items():
        os.environ[key] = str(val)
    file = ROOT / "oracle" / path_name / "model.py"
    spec = importlib.util.spec_from_file_location(f"oracle_{path_name}_model_{len(sys.modules)}", file)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def built_libs():
    """Build (or reuse) both shared objects; CPU-only boxes can do this too."""
    from cuda_agent_b200 import build
    build.build_all()
    return build


@pytest.fixture(scope="session")
def cuda_device(built_libs):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda:0")
