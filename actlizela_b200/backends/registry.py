"""Catalog access with the reference's semantics (actlize_la/backends/registry.py:13-44):
``ValueError`` for an unknown name, ``RuntimeError`` for a known name without an
implementation on the requested target, and never a fallback.  Importing this module does
not import torch or load a native library.
"""
from copy import deepcopy
from functools import lru_cache
import json
from pathlib import Path


@lru_cache(maxsize=1)
def _catalog():
    data = json.loads(Path(__file__).with_name("targets.json").read_text())
    if data.get("schema") != 1:
        raise RuntimeError("unsupported GDN backend catalog schema")
    return data


def backend_inventory():
    """Independent copy of the catalog; implemented != built, admitted or fastest."""
    return deepcopy(_catalog())


def require_backend(name):
    targets = _catalog()["targets"]
    if name not in targets:
        raise ValueError(f"unknown GDN backend {name!r}; choose {tuple(targets)}")
    backend = targets[name]
    if not backend["implemented"]:
        raise RuntimeError(f"GDN backend {name}: {backend.get('reason', 'not implemented')}")
    return backend


def require_implementation(algorithm, backend):
    require_backend(backend)
    algorithms = _catalog()["algorithms"]
    if algorithm not in algorithms:
        raise ValueError(f"unknown GDN algorithm {algorithm!r}; choose {tuple(algorithms)}")
    implementation = algorithms[algorithm]
    if backend not in implementation["targets"]:
        raise RuntimeError(f"GDN algorithm {algorithm} has no {backend} implementation; no fallback")
    return {**implementation, **implementation.get("target_entries", {}).get(backend, {})}
