#!/usr/bin/env python3
"""Place the reference project's own CPU implementation of the path under ``oracle/_ref/``.

    python oracle/make_ref.py /path/to/reference/checkout

The reference's FP32 path is one pure-Python (PyTorch CPU) module,
``actlize_la/reference/gdn_chunk_ref.py``; there is nothing to compile.  This recipe takes that
file, unmodified, from the checkout where it lies into ``oracle/_ref/`` (git-ignored: reference
sources never enter this repository's history) and records its SHA-256 in ``oracle/_ref/ref.json``.
``bench.py --impl reference`` then times the reference's own code (``cpu_baseline.kind =
"reference"``); without the file it times the restatement in ``oracle/gdn_oracle.py`` (``"port"``).
Test infrastructure only: nothing in the product package reads ``oracle/``.
"""
from __future__ import annotations

import hashlib
import json
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
MODULE = Path("actlize_la") / "reference" / "gdn_chunk_ref.py"


def make_ref(checkout, quiet=False):
    source = Path(checkout) / MODULE
    if not source.is_file():
        raise FileNotFoundError(f"{source} not found: pass the root of the reference checkout")
    out = HERE / "_ref"
    out.mkdir(exist_ok=True)
    target = out / "gdn_chunk_ref.py"
    shutil.copyfile(source, target)
    digest = hashlib.sha256(target.read_bytes()).hexdigest()
    (out / "ref.json").write_text(json.dumps(dict(module=str(MODULE), sha256=digest), indent=2) + "\n")
    if not quiet:
        print(f"placed {target} sha256={digest[:16]}")
    return target


def load_ref():
    """The placed module, or None when the recipe has not run (or the file does not match its record)."""
    import importlib.util
    target, record = HERE / "_ref" / "gdn_chunk_ref.py", HERE / "_ref" / "ref.json"
    if not (target.is_file() and record.is_file()):
        return None
    if json.loads(record.read_text()).get("sha256") != hashlib.sha256(target.read_bytes()).hexdigest():
        return None
    spec = importlib.util.spec_from_file_location("actlize_la_reference_gdn_chunk_ref", target)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def reference_forward(module, q, k, v, g, beta, initial_state=None, output_final_state=True):
    """Call the reference's ``torch_chunk_gated_delta_rule`` the way its own callers do
    (tests/test_gdn_chunk.py:28-30 expand q and k to the value heads first)."""
    ratio = v.shape[2] // q.shape[2]
    if ratio > 1:
        q, k = q.repeat_interleave(ratio, dim=2), k.repeat_interleave(ratio, dim=2)
    return module.torch_chunk_gated_delta_rule(q, k, v, g, beta, initial_state=initial_state,
                                               output_final_state=output_final_state)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    make_ref(sys.argv[1])
