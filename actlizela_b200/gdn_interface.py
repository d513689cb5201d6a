"""Common forward contract: the reference's public ``gdn_forward`` with a cuda_sm100 route.

Argument meaning and error behaviour follow actlize_la/gdn_interface.py:14-84:
``algorithm="auto"`` picks the backend from the device of ``q`` and the kernel configuration
from the static shape table; an explicit ``algorithm="wy_sm100", backend="cuda_sm100"`` call
may name a configuration for diagnostics.  ``delivery`` belongs to other targets and is
rejected.  Selection never examines gate values or compiles anything during a call, and an
unsupported device or a missing binary is an error, never a fallback.
"""
from importlib import import_module

from .backends.registry import require_implementation
from .device import validate_profile_options


def _resolve_forward(q, initial_state=None, *, algorithm="auto", backend=None,
                     delivery=None, configuration=None, mode="device", sm_count=None):
    """Single policy authority for execution and preparation-time inspection."""
    validate_profile_options(mode, backend, sm_count)
    if delivery is not None:
        raise ValueError("cuda_sm100 owns its pipeline; delivery selectors do not apply")
    if algorithm == "auto":
        if configuration is not None:
            raise ValueError("auto selects its configuration; use explicit wy_sm100 for diagnostics")
        if backend is None:
            from .sm100_policy import tensor_backend
            backend = tensor_backend(q)
        algorithm = "wy_sm100"
        selected = "auto"
    else:
        selected = algorithm
        if backend is None:
            raise ValueError(f"{algorithm} requires an explicit backend")
    implementation = require_implementation(algorithm, backend)
    if initial_state is not None and not implementation["initial_state"]:
        raise ValueError(f"{algorithm} does not accept initial_state; it must not be dropped")
    return dict(implementation, backend=backend, algorithm=algorithm, selected=selected,
                delivery=None, configuration=configuration)


def gdn_forward(q, k, v, g, beta, initial_state=None, output_final_state=True,
                *, algorithm="auto", backend=None, delivery=None, configuration=None,
                mode="device", sm_count=None):
    """Complete chunked gated-delta-rule forward.

    q,k [B,T,Hk,128] BF16; v [B,T,Hv,128] BF16 (Hv % Hk == 0); g [B,T,Hv] natural-log decay
    (BF16 or FP32); beta [B,T,Hv] BF16; optional FP32 initial_state [B,Hv,128,128] (K by V).
    Returns (output BF16 [B,T,Hv,128], final FP32 state or None).  Chunk size 64 and the
    1/sqrt(128) query scale are built in; no hidden Q/K normalisation, gate activation,
    rescaling or state conversion takes place.
    """
    route = _resolve_forward(q, initial_state, algorithm=algorithm, backend=backend,
                             delivery=delivery, configuration=configuration,
                             mode=mode, sm_count=sm_count)
    call = getattr(import_module(f".{route['module']}", __package__), route["entry"])
    return call(q, k, v, g, beta, initial_state=initial_state,
                output_final_state=output_final_state, backend=route["backend"],
                configuration=route["configuration"], mode=mode, sm_count=sm_count)
