"""actlizela_b200: the gated-delta-rule forward of actlizeLA, rebuilt for NVIDIA B200 (sm_100a).

Public names mirror the reference package (actlize_la/__init__.py:9-40) for the one path this
build covers; everything is imported lazily so that importing the package never loads a
native library or initialises CUDA.
"""
from importlib import import_module

__version__ = "0.1.0"

_MODULES = {
    "gdn_forward": "gdn_interface",
    "get_gdn_route_info": "gdn_route",
    "backend_inventory": "backends",
    "get_device_profile": "device",
    "get_library_info": "_library",
    "get_library_path": "_library",
    "load_sm100": "sm100",
    "gdn_chunk_sm100": "sm100",
    "gdn_forward_sharded": "sharding",
    "shard_plan": "sharding",
    "gdn_forward_sequence_parallel": "sequence_parallel",
    "capture_sequence_parallel": "sequence_parallel",
    "gdn_forward_varlen": "varlen",
    "gdn_prepare_inputs": "aux_ops",
    "gdn_decode_step": "aux_ops",
    "gdn_forward_projections": "aux_ops",
    "gdn_verify_step": "aux_ops",
    "gdn_commit_step": "aux_ops",
    "rmsnorm_gated": "aux_ops",
    "out_proj_gemm": "aux_ops",
}


def __getattr__(name):
    if name not in _MODULES:
        raise AttributeError(name)
    value = getattr(import_module(f".{_MODULES[name]}", __name__), name)
    globals()[name] = value
    return value


__all__ = sorted(_MODULES)
