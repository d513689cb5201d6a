"""Shared pytest configuration: the `gpu` marker and common fixtures."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    """Reference outputs stored by tests/golden/make_golden.py: name -> (out bf16, state f32, meta)."""
    directory = ROOT / "tests" / "golden"
    arrays = np.load(directory / "golden_cases.npz")
    index = json.loads((directory / "golden_cases.json").read_text())["cases"]
    result = {}
    for name, meta in index.items():
        out = torch.from_numpy(arrays[f"{name}.out_bf16"].copy()).view(torch.bfloat16)
        state = torch.from_numpy(arrays[f"{name}.state_f32"].copy())
        result[name] = (out, state, meta)
    return result


@pytest.fixture(scope="session")
def native_library():
    """The built native library (builds it in-tree if the shared object is absent)."""
    from actlizela_b200 import _library
    path = _library.NATIVE_DIRECTORY / _library.LIBRARY_NAME
    if not path.is_file():
        from actlizela_b200.build_sm100 import build
        build(quiet=True)
    return _library.load_library()
