"""Target / algorithm catalog of this package (targets.json beside this file).

Behaviour matches what callers of the reference's catalog accessor rely on
(actlize_la/backends/registry.py:13-44): an unknown name is a ``ValueError``, a known name that
cannot run on the requested target is a ``RuntimeError``, and no lookup ever substitutes another
target or algorithm.  Nothing here imports torch or opens a native library.
"""
from __future__ import annotations

import copy
import json
from pathlib import Path

_CATALOG_FILE = Path(__file__).with_name("targets.json")
_SUPPORTED_SCHEMA = 1


class Catalog:
    """The parsed catalog with the three lookups the package needs."""

    def __init__(self, path=_CATALOG_FILE):
        document = json.loads(Path(path).read_text())
        if document.get("schema") != _SUPPORTED_SCHEMA:
            raise RuntimeError(f"catalog {path} has schema {document.get('schema')!r}, expected {_SUPPORTED_SCHEMA}")
        self._document = document
        self._targets = document["targets"]
        self._algorithms = document["algorithms"]

    def snapshot(self):
        """A private deep copy: edits by the caller never reach the catalog."""
        return copy.deepcopy(self._document)

    def target(self, name):
        entry = self._targets.get(name)
        if entry is None:
            raise ValueError(f"no backend named {name!r} in the catalog (known: {', '.join(self._targets)})")
        if not entry["implemented"]:
            why = entry.get("reason") or "this package ships no kernels for it"
            raise RuntimeError(f"backend {name} cannot be used: {why}")
        return entry

    def implementation(self, algorithm, target_name):
        self.target(target_name)
        entry = self._algorithms.get(algorithm)
        if entry is None:
            raise ValueError(f"no algorithm named {algorithm!r} in the catalog (known: {', '.join(self._algorithms)})")
        if target_name not in entry["targets"]:
            raise RuntimeError(f"algorithm {algorithm} is not built for {target_name}, and nothing is substituted")
        merged = dict(entry)
        merged.update(entry.get("target_entries", {}).get(target_name, {}))
        return merged


_catalog = None


def _shared():
    global _catalog
    if _catalog is None:
        _catalog = Catalog()
    return _catalog


def backend_inventory():
    """What the catalog lists.  Being listed as implemented says nothing about being built or fastest."""
    return _shared().snapshot()


def require_backend(name):
    return _shared().target(name)


def require_implementation(algorithm, backend):
    return _shared().implementation(algorithm, backend)
