"""Where the selector's device facts come from: a hardware query, or numbers the caller states.

Two modes, as in the reference (actlize_la/device.py:36-77).  ``mode="device"`` reads name, SM
count and compute capability of a CUDA device once per index and remembers them.
``mode="perfmodel"`` touches no device at all: the caller names the backend and the SM count,
and the profile is marked as configured so that the selector answers with its unmeasured default.
Nothing is guessed in either mode.
"""
from __future__ import annotations

from dataclasses import dataclass

from .backends.registry import require_backend

_BACKEND_CAPABILITY = {"cuda_sm100": (10, 0)}
_MODES = ("device", "perfmodel")
_measured = {}


@dataclass(frozen=True)
class DeviceProfile:
    name: str
    sm_count: int
    capability: tuple | None
    source: str = "measured"      # "measured": read from hardware; "configured": stated by the caller


def validate_profile_options(mode, backend, sm_count):
    """Reject combinations that would need a guess: an SM count next to a hardware query, or a model without
    an explicit backend and a positive integer SM count."""
    if mode not in _MODES:
        raise ValueError(f"mode is {mode!r}; it must be one of {_MODES}")
    if mode == "device":
        if sm_count is not None:
            raise ValueError("an sm_count is only meaningful with mode='perfmodel' (a hardware query reads its own)")
        return
    if backend is None:
        raise ValueError("mode='perfmodel' needs the backend spelled out: no device is looked at")
    require_backend(backend)
    if isinstance(sm_count, bool) or not isinstance(sm_count, int) or sm_count < 1:
        raise ValueError("mode='perfmodel' needs sm_count as a positive integer")


def device_profile(index):
    """Facts of CUDA device ``index``, queried on first use."""
    profile = _measured.get(index)
    if profile is None:
        import torch
        props = torch.cuda.get_device_properties(index)
        profile = DeviceProfile(props.name, props.multi_processor_count, (props.major, props.minor))
        _measured[index] = profile
    return profile


def get_device_profile(index=None, *, mode="device", backend=None, sm_count=None):
    validate_profile_options(mode, backend, sm_count)
    if mode == "device":
        return device_profile(index)
    return DeviceProfile(backend, sm_count, _BACKEND_CAPABILITY.get(backend), source="configured")
