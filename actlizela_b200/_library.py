"""File-only discovery and verified loading of the native cuda_sm100 library.

Follows the reference's conventions for packaged native code
(actlize_la/_library.py:74-165 discovery sealed by a manifest hash;
actlize_la/sm90.py:23-67 receipt check before load; actlize_la/serving/_native.py:47-71
ctypes binding): the shared object sits beside a ``build.json`` receipt that records its
SHA-256; discovery reads files only; the library is dlopen'ed lazily, once, and its ABI
version, target architecture and numerical-contract string are checked against the catalog.
A missing or mismatched binary is a ``RuntimeError``; there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
from functools import lru_cache
import hashlib
import json
import os
from pathlib import Path

from .backends.registry import require_implementation

ABI_VERSION = 1
LIBRARY_NAME = "libactlize_la_sm100.so"
NATIVE_DIRECTORY = Path(__file__).resolve().parent / "_native"
ENVIRONMENT_OVERRIDE = "ACTLIZE_LA_SM100_LIBRARY"

# name -> (restype, argtypes); must list every symbol include/actlize_la_sm100.h declares
_P, _I, _LL = C.c_void_p, C.c_int, C.c_longlong
EXPORTS = {
    "actlize_la_sm100_abi_version": (_I, []),
    "actlize_la_sm100_target_arch": (_I, []),
    "actlize_la_sm100_numerical_contract": (C.c_char_p, []),
    "actlize_la_sm100_configure": (_I, []),
    "actlize_la_sm100_select": (_I, [_I] * 5),
    "actlize_la_sm100_workspace_bytes": (_LL, [_I] * 5),
    "actlize_la_sm100_forward_prepared": (_I, [_P] * 9 + [_LL] + [_I] * 6 + [_P]),
    "actlize_la_sm100_host_arena_bytes": (_LL, [_I] * 8),
    "actlize_la_sm100_forward_host": (_I, [_P] * 9 + [_LL] + [_I] * 6 + [_P]),
    "actlize_la_sm100_apply_transition": (_I, [_P] * 4 + [_I, _P]),
    "actlize_la_sm100_fold_transitions": (_I, [_P, _I] + [_P] * 4 + [_I, _P]),
    "actlize_la_sm100_launches_per_forward": (_I, [_I]),
    "actlize_la_sm100_device_status": (_I, [_P, _I]),
    "actlize_la_sm100_walk_plan_counts": (_I, [_P, _I]),
    "actlize_la_sm100_last_failure": (_I, [_P]),
    "actlize_la_sm100_selftest_walk_stall": (_I, [_P] * 7 + [_LL] + [_I] * 5 + [_P]),
    "actlize_la_sm100_selftest_wait_timeout": (_I, [_I, _P]),
    "actlize_la_sm100_prepare_inputs": (_I, [_P, _LL] + [_P] * 9 + [_LL, _I, _I, _P]),
    "actlize_la_sm100_decode_step": (_I, [_P] * 7 + [_I] * 4 + [_P]),
    "actlize_la_sm100_rmsnorm_gated": (_I, [_P] * 4 + [_LL, _P]),
    "actlize_la_sm100_out_proj": (_I, [_P] * 3 + [_I] * 3 + [_P]),
    "actlize_la_sm100_verify_step": (_I, [_P] * 8 + [_I] * 5 + [_P]),
    "actlize_la_sm100_commit_step": (_I, [_P] * 5 + [_I] * 5 + [_P]),
    "actlize_la_sm100_forward_static_scratch": (_I, [_P] * 8 + [_I] * 6 + [_P]),
    "actlize_la_sm100_projections_workspace_bytes": (_LL, [_I] * 5),
    "actlize_la_sm100_forward_projections": (_I, [_P, _LL] + [_P] * 8 + [_LL] + [_I] * 5 + [_P]),
    "actlize_la_sm100_varlen_workspace_bytes": (_LL, [_LL, _I, _I, _I]),
    "actlize_la_sm100_forward_varlen": (_I, [_P] * 9 + [_LL, _P] + [_I] * 4 + [_P]),
    "actlize_la_sm100_forward_varlen_device": (_I, [_P] * 9 + [_LL, _P, _I, _LL] + [_I] * 3 + [_P]),
}


class LibraryError(RuntimeError):
    """The native cuda_sm100 library is absent, incomplete or does not match its receipt."""


def _sha(path):
    h = hashlib.sha256()
    with Path(path).open("rb") as stream:
        for chunk in iter(lambda: stream.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def _resolve(override):
    if override is not None:
        if not override.strip():
            raise LibraryError(f"{ENVIRONMENT_OVERRIDE} must not be empty")
        path = Path(override)
        if not path.is_absolute():
            raise LibraryError(f"{ENVIRONMENT_OVERRIDE} requires an absolute file path")
    else:
        path = NATIVE_DIRECTORY / LIBRARY_NAME
    if not path.is_file():
        raise LibraryError(
            f"native cuda_sm100 library not built: {path}; run python -m actlizela_b200.build_sm100 "
            "(there is no CPU or PyTorch fallback)")
    return path.resolve()


def get_library_info(override=None):
    """Validated, JSON-serialisable identity of the native library; no dlopen, no device access."""
    path = _resolve(os.environ.get(ENVIRONMENT_OVERRIDE) if override is None else override)
    receipt_path = path.with_name("build.json")
    if not receipt_path.is_file():
        raise LibraryError(f"native library has no build receipt: {receipt_path}")
    receipt = json.loads(receipt_path.read_text())
    digest = _sha(path)
    if receipt.get("complete") is not True or receipt.get("target") != "cuda_sm100":
        raise LibraryError("build receipt is incomplete or for another target")
    if receipt.get("library_sha256") != digest:
        raise LibraryError("native library hash differs from its build receipt; rebuild")
    return dict(library_path=str(path), library_sha256=digest, receipt_path=str(receipt_path),
                target=receipt["target"], arch=receipt.get("arch"), flags=receipt.get("flags"),
                compiler=receipt.get("compiler_version"), source_sha256=receipt.get("source_sha256"),
                policy_sha256=receipt.get("policy_sha256"), abi_version=receipt.get("abi_version"))


def get_library_path(override=None):
    return Path(get_library_info(override)["library_path"])


class NativeLibrary:
    """ctypes view of one verified shared object. Construction checks identity once."""

    def __init__(self, info):
        self.info = dict(info)
        self.lib = C.CDLL(info["library_path"])
        for name, (restype, argtypes) in EXPORTS.items():
            try:
                fn = getattr(self.lib, name)
            except AttributeError:
                raise LibraryError(f"native library lacks export {name}; no fallback") from None
            fn.restype, fn.argtypes = restype, argtypes
        expected = require_implementation("wy_sm100", "cuda_sm100")["numerical_contract"]
        contract = self.lib.actlize_la_sm100_numerical_contract().decode()
        if (self.lib.actlize_la_sm100_abi_version() != ABI_VERSION
                or self.lib.actlize_la_sm100_target_arch() != 100 or contract != expected):
            raise LibraryError("native library ABI/target/numerical-contract identity mismatch")
        self.numerical_contract = contract
        self._configured = set()

    def configure(self, device):
        """Per-device function attributes; once per device, before any capture."""
        import torch
        key = str(device)
        if key not in self._configured:
            with torch.cuda.device(device):
                if torch.cuda.is_current_stream_capturing():
                    raise RuntimeError("configure the cuda_sm100 library before stream capture")
                self.check(self.lib.actlize_la_sm100_configure())
            self._configured.add(key)

    @staticmethod
    def current_stream_handle(device_index):
        """The raw cudaStream_t of torch's current stream on a device, without building a Stream object (this sits
        in front of every launch of the sequence-parallel path, whose host time shows at eight ranks)."""
        import torch
        raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
        return raw(device_index) if raw is not None else torch.cuda.current_stream(device_index).cuda_stream

    @staticmethod
    def check(code):
        if code:
            raise RuntimeError(f"cuda_sm100 native call failed with CUDA error code {code}")

    def last_failure(self, device):
        """(code, block, wait site, chunk) of a kernel on ``device`` that gave up a bounded wait, or None.
        Reads the host-visible record only: no synchronisation, so it reports launches that have already run."""
        import torch
        record = (C.c_int * 4)()
        index = torch.device(device).index
        if index is None or index == torch.cuda.current_device():
            self.check(self.lib.actlize_la_sm100_last_failure(record))
        else:
            with torch.cuda.device(device):
                self.check(self.lib.actlize_la_sm100_last_failure(record))
        return tuple(record) if record[0] else None

    def raise_on_failure(self, device, synchronize=False):
        """Raise if a kernel on ``device`` gave up waiting (its outputs are incomplete); clears the record.
        With ``synchronize`` the device is drained first, so every launch issued so far is covered."""
        import torch
        if synchronize:
            torch.cuda.synchronize(device)
        failure = self.last_failure(device)
        if failure:
            record = (C.c_int * 4)()
            with torch.cuda.device(device):
                self.check(self.lib.actlize_la_sm100_device_status(record, 1))
            raise RuntimeError(
                "a cuda_sm100 kernel gave up a bounded wait (code %d, block %d, wait site %d, chunk %d): the outputs "
                "of that launch are incomplete and must be discarded" % failure)


@lru_cache(maxsize=None)
def _load(path, digest):
    info = get_library_info(path)
    if info["library_sha256"] != digest:
        raise LibraryError("native library changed between discovery and load")
    return NativeLibrary(info)


@lru_cache(maxsize=None)
def _load_selected(override):
    info = get_library_info(override)
    return _load(info["library_path"], info["library_sha256"])


def load_library():
    """The verified native library.  Discovery, hashing and dlopen happen once per selection (the value of
    the environment override); later calls are a dictionary look-up: no file I/O or hashing per call."""
    return _load_selected(os.environ.get(ENVIRONMENT_OVERRIDE))
