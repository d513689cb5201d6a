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
    """The built native library; rebuilt in-tree when it is absent or older than the sources it records."""
    from actlizela_b200 import _library
    from actlizela_b200.build_sm100 import build, sha
    path = _library.NATIVE_DIRECTORY / _library.LIBRARY_NAME
    receipt = _library.NATIVE_DIRECTORY / "build.json"
    stale = not path.is_file() or not receipt.is_file()
    if not stale:
        # a binary older than the sources must not be what the tests exercise: compare the receipt's source hashes
        recorded = json.loads(receipt.read_text()).get("source_sha256", {})
        stale = not recorded or any(not (ROOT / name).is_file() or sha(ROOT / name) != digest
                                    for name, digest in recorded.items())
        sources = (ROOT / "actlizela_b200" / "csrc" / "backends" / "sm100").iterdir()
        stale = stale or any(str(p.relative_to(ROOT)) not in recorded for p in sources if p.suffix in (".cu", ".cuh", ".h"))
    if stale:
        build(quiet=True)
    return _library.load_library()
