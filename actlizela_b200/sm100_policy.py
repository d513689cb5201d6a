"""Metadata-only configuration selection for the B200 backend.

Static table in the style of the reference's actlize_la/sm90_policy.py:13-81 and
sm90_policy.json: exact (B,T,Hk,Hv) rows, a labelled default for everything else, duplicate
or unknown rows rejected at load.  Selection reads shapes and the device profile only:
no gate values, no tensor copies, no launches, no runtime compilation, no autotuning.
The same table is compiled into the native library (actlize_la_sm100_select).
"""
from dataclasses import dataclass
from functools import lru_cache
import hashlib
import json
from pathlib import Path

from .device import device_profile, get_device_profile, validate_profile_options

POLICY_FILE = Path(__file__).with_suffix(".json")


@lru_cache(maxsize=1)
def policy():
    data = json.loads(POLICY_FILE.read_text())
    if data.get("schema") != 1 or data.get("default") not in data.get("configurations", ()):
        raise ValueError("invalid SM100 policy")
    if set(data.get("configuration_ids", ())) != set(data["configurations"]):
        raise ValueError("SM100 policy configuration ids do not cover the configurations")
    rows = data["rows"]
    keys = [tuple(r["shape"]) for r in rows]
    if len(set(keys)) != len(keys) or any(r["configuration"] not in data["configurations"] for r in rows):
        raise ValueError("duplicate or unknown SM100 policy row")
    if any(not 1 <= int(r.get("segments", 1)) <= 16 for r in rows):
        raise ValueError("SM100 policy row with an unsupported segment count")
    if any(not 1 <= int(r.get("parallel", 1)) <= 8 for r in rows):
        raise ValueError("SM100 policy row with an unsupported parallel sub-segment count")
    return data


def policy_digest():
    return hashlib.sha256(POLICY_FILE.read_bytes()).hexdigest()


@dataclass(frozen=True)
class Selection:
    configuration: str
    basis: str
    policy_id: str
    segments: int = 1     # sequence segments whose prepare overlaps the previous segment's walk
    parallel: int = 1     # sub-segments of every (batch, value head) walk that are walked at the same time

    @property
    def configuration_id(self):
        """Native configuration word: kernel family in the low bits, segment count in bits 8..15, parallel
        sub-segments of the walk in bits 16..19."""
        family = policy()["configuration_ids"][self.configuration]
        return family | (self.segments << 8) | ((self.parallel << 16) if family == 1 else 0)


def default_parallel(batch, length, value_heads):
    """Parallel sub-segments of the walk for a shape without a measured row: as many as give every one of the 148
    SMs one walk CTA, at least 8 chunks per sub-segment, at most 8.  The native selector computes the same."""
    heads, chunks = batch * value_heads, (length + 63) // 64
    return max(1, min(8, 148 // heads, chunks // 8))


def default_segments(batch, length, value_heads):
    """Segment count for a shape without a measured row.  Overlapping the prepare of a later segment with the walk
    of an earlier one only pays while the walk leaves SMs idle, i.e. when it is not split into parallel
    sub-segments: then up to 64 heads -> isqrt(chunks/8) clamped to 1..8, more -> 1.  The native selector computes
    the same."""
    from math import isqrt
    heads, chunks = batch * value_heads, (length + 63) // 64
    if heads > 64 or default_parallel(batch, length, value_heads) > 1:
        return 1
    return max(1, min(8, isqrt(chunks // 8)))


def tensor_backend(q):
    """Device tensor -> backend name; only capability (10,0) is admitted, nothing is guessed."""
    device = getattr(q, "device", None)
    if device is None or device.type != "cuda":
        raise ValueError("automatic GDN requires a CUDA device tensor")
    profile = device_profile(device.index)
    if profile.capability == (10, 0):
        return "cuda_sm100"
    raise ValueError("automatic GDN target unsupported; this build admits sm_100 devices only")


def select(shape, profile):
    """shape=(B,T,Hk,Hv,K,V); metadata only."""
    data = policy()
    if len(shape) != 6 or any(not isinstance(x, int) or x <= 0 for x in shape):
        raise ValueError("SM100 selector requires positive B,T,Hk,Hv,K,V")
    if shape[3] % shape[2] or tuple(shape[4:]) != tuple(data["head_dimensions"]):
        raise ValueError("SM100 requires integral grouped value heads and K=V=128")
    expected = data["device"]
    if profile.capability != tuple(expected["capability"]):
        raise ValueError("SM100 shape policy cannot be applied to another execution target")
    if profile.source == "configured":
        return Selection(data["default"], "perfmodel-unmeasured-default", data["id"])
    if profile.source != "measured":
        raise ValueError("unknown device profile source")
    if expected["name_contains"] not in profile.name or profile.sm_count != expected["sm_count"]:
        return Selection(data["default"], "unmeasured-device-default", data["id"])
    for row in data["rows"]:
        if tuple(row["shape"]) == tuple(shape[:4]):
            return Selection(row["configuration"], "b200-measured-shape", data["id"],
                             int(row.get("segments", 1)), int(row.get("parallel", 1)))
    return Selection(data["default"], "unmeasured-shape-default", data["id"],
                     default_segments(shape[0], shape[1], shape[3]), default_parallel(shape[0], shape[1], shape[3]))


_SELECTIONS = {}


def selection_for(q, v, *, mode="device", sm_count=None):
    """Selection for a pair of device tensors; remembered per (shapes, device, mode) after the first call, as the
    reference remembers its route (actlize_la/sm90_auto.py:68-89): table and device profile are both static."""
    key = (tuple(q.shape), tuple(v.shape), q.device, v.device, mode, sm_count)
    held = _SELECTIONS.get(key)
    if held is not None:
        return held
    validate_profile_options(mode, "cuda_sm100", sm_count)
    if q.ndim != 4 or v.ndim != 4 or tuple(q.shape[:2]) != tuple(v.shape[:2]):
        raise ValueError("SM100 requires q/v [B,T,H,D] with matching batch and sequence")
    if q.device.type != "cuda" or q.device != v.device:
        raise ValueError("SM100 q/v must be on the same CUDA device")
    shape = tuple(int(x) for x in (*q.shape[:3], v.shape[2], q.shape[3], v.shape[3]))
    profile = (get_device_profile(mode=mode, backend="cuda_sm100", sm_count=sm_count)
               if mode == "perfmodel" else device_profile(q.device.index))
    held = select(shape, profile)
    if len(_SELECTIONS) > 256:
        _SELECTIONS.clear()
    _SELECTIONS[key] = held
    return held
