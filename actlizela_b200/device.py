"""Measured device metadata or explicit model inputs, never an implicit fallback.

Same contract as the reference's actlize_la/device.py:36-77: ``mode='device'`` queries the
hardware once per index (cached); ``mode='perfmodel'`` takes an explicit backend and SM
count and never touches a device.
"""
from dataclasses import dataclass
from functools import lru_cache

from .backends.registry import require_backend

_CAPABILITY = {"cuda_sm100": (10, 0)}


@dataclass(frozen=True)
class DeviceProfile:
    name: str
    sm_count: int
    capability: tuple | None
    source: str = "measured"


def validate_profile_options(mode, backend, sm_count):
    if mode not in ("device", "perfmodel"):
        raise ValueError("mode must be 'device' or 'perfmodel'")
    if mode == "device":
        if sm_count is not None:
            raise ValueError("sm_count is a model input; it requires mode='perfmodel'")
        return
    if backend is None:
        raise ValueError("perfmodel requires an explicit backend; no hardware discovery")
    require_backend(backend)
    if type(sm_count) is not int or sm_count <= 0:
        raise ValueError("perfmodel requires an explicit positive integer sm_count")


@lru_cache(maxsize=None)
def device_profile(index):
    """Hardware query, cached per device index."""
    import torch
    props = torch.cuda.get_device_properties(index)
    return DeviceProfile(props.name, props.multi_processor_count, (props.major, props.minor))


def get_device_profile(index=None, *, mode="device", backend=None, sm_count=None):
    validate_profile_options(mode, backend, sm_count)
    if mode == "perfmodel":
        return DeviceProfile(backend, sm_count, _CAPABILITY.get(backend), source="configured")
    return device_profile(index)
