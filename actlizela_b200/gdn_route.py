"""Preparation-time route inspection; never called from forward or replay.

Extends the reference's inspector (actlize_la/gdn_route.py:16-77, which covers PPU1.0 only)
to the cuda_sm100 route: it reports the backend, algorithm, selected configuration, native
entry symbol and the identity of the loaded shared object, and marks device execution as
NOT_RUN.  It reads tensor metadata only (shape, stride, dtype, device), never tensor data,
and launches nothing.
"""
from pathlib import Path

from .gdn_interface import _resolve_forward

NATIVE_ENTRY = "actlize_la_sm100_forward_prepared"


def _metadata(tensor):
    if tensor is None:
        return None
    return dict(shape=list(tensor.shape), stride=list(tensor.stride()),
                dtype=str(tensor.dtype), device=str(tensor.device))


def get_gdn_route_info(q, k, v, g, beta, initial_state=None, output_final_state=True,
                       *, load_binary=True, **forward_options):
    """Describe the same route as gdn_forward without executing a device kernel.

    ``load_binary=False`` reports policy only.  The default verifies the native library
    against its build receipt, loads it and records its path and SHA-256.
    """
    route = _resolve_forward(q, initial_state, **forward_options)
    mode = forward_options.get("mode", "device")
    sm_count = forward_options.get("sm_count")
    from .sm100_policy import policy_digest, selection_for
    if route["configuration"] is None:
        selection = selection_for(q, v, mode=mode, sm_count=sm_count)
        configuration, basis = selection.configuration, selection.basis
    else:
        from .sm100 import configuration_id
        configuration_id(route["configuration"])
        configuration, basis = route["configuration"], "explicit-diagnostic"
    result = dict(
        schema=1, api="gdn_forward", backend=route["backend"], algorithm=route["algorithm"],
        selected=route["selected"], delivery=None, configuration=configuration,
        configuration_basis=basis, policy_sha256=policy_digest(),
        python_entry=f"actlizela_b200.{route['module']}.{route['entry']}",
        python_sources_on_disk=[str(Path(__file__).with_name(name)) for name in
                                ("gdn_interface.py", f"{route['module']}.py", "sm100_policy.json")],
        native_entry=NATIVE_ENTRY, numerical_contract=route["numerical_contract"],
        state_layout="B,Hv,K,V", final_state_dtype=route["final_state_dtype"],
        output_final_state=bool(output_final_state),
        inputs={name: _metadata(value) for name, value in
                zip(("q", "k", "v", "g", "beta", "initial_state"),
                    (q, k, v, g, beta, initial_state))},
        native_status="NOT_LOADED", device_execution="NOT_RUN",
    )
    if load_binary:
        from ._library import load_library
        library = load_library()
        if not callable(getattr(library.lib, NATIVE_ENTRY, None)):
            raise RuntimeError(f"selected native entry is missing: {NATIVE_ENTRY}; no fallback")
        result["native_images"] = [dict(path=library.info["library_path"],
                                        sha256=library.info["library_sha256"])]
        result["native_build"] = dict(flags=library.info["flags"], compiler=library.info["compiler"])
        result["native_status"] = "LOADED_FILES_VERIFIED_NOT_DEVICE_ADMITTED"
    return result
