"""The steps either side of the chunked forward, on the same native library.

* ``gdn_prepare_inputs``: Q/K L2 normalisation, gate activation and beta from a fused projection
  (reference: csrc/serving/prefill.cu:45-70, csrc/serving/runtime.cuh:48-52).
* ``gdn_decode_step``: one token on the FP32 ``[B,Hv,128,128]`` K-by-V state, in place
  (reference: actlize_la/reference/gdn_chunk_ref.py:135-143; csrc/serving/gdn.cu:152).
* ``rmsnorm_gated``: ``y * rsqrt(mean y^2 + 1e-6) * weight * silu(z)`` per 128-wide row
  (reference: actlize_la.rmsnorm_gated, docs/OUTPUT_GATE.md:7-15).
All three are single memory-bound kernels launched on the caller's current stream.
"""
from __future__ import annotations

from ._library import load_library


def _bf16_cuda(x, name, last=None):
    import torch
    if x.dtype != torch.bfloat16 or x.device.type != "cuda" or not x.is_contiguous():
        raise ValueError(f"{name} must be a contiguous BF16 CUDA tensor")
    if last is not None and x.shape[-1] != last:
        raise ValueError(f"{name} must have a last dimension of {last}")


def gdn_prepare_inputs(mixed, a, b, a_log, dt_bias, key_heads, value_heads):
    """mixed [N, (2Hk+Hv)*128] BF16, a,b [N,Hv] BF16, a_log, dt_bias [Hv] FP32 ->
    (q [N,Hk,128], k [N,Hk,128], v [N,Hv,128] BF16, g [N,Hv] FP32, beta [N,Hv] BF16)."""
    import torch
    _bf16_cuda(a, "a", value_heads)
    _bf16_cuda(b, "b", value_heads)
    if mixed.dtype != torch.bfloat16 or mixed.device.type != "cuda" or mixed.ndim != 2 or mixed.stride(1) != 1:
        raise ValueError("mixed must be a 2-D BF16 CUDA tensor with unit inner stride")
    n, width = mixed.shape
    if width != (2 * key_heads + value_heads) * 128 or value_heads % key_heads:
        raise ValueError("mixed must hold [q heads | k heads | v heads] x 128 and Hv % Hk == 0")
    if a_log.dtype != torch.float32 or dt_bias.dtype != torch.float32 or a_log.numel() != value_heads:
        raise ValueError("a_log and dt_bias must be FP32 [Hv]")
    lib = load_library()
    q = torch.empty(n, key_heads, 128, dtype=torch.bfloat16, device=mixed.device)
    k = torch.empty_like(q)
    v = torch.empty(n, value_heads, 128, dtype=torch.bfloat16, device=mixed.device)
    g = torch.empty(n, value_heads, dtype=torch.float32, device=mixed.device)
    beta = torch.empty(n, value_heads, dtype=torch.bfloat16, device=mixed.device)
    with torch.cuda.device(mixed.device):
        lib.check(lib.lib.actlize_la_sm100_prepare_inputs(
            mixed.data_ptr(), mixed.stride(0), a.data_ptr(), b.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(),
            q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), n, key_heads, value_heads,
            torch.cuda.current_stream().cuda_stream))
    return q, k, v, g, beta


def gdn_decode_step(q, k, v, g, beta, state):
    """q,k [B,Hk,128], v [B,Hv,128] BF16, g [B,Hv] (BF16/FP32 natural-log decay), beta [B,Hv] BF16,
    state FP32 [B,Hv,128,128] updated IN PLACE.  Returns the BF16 output [B,Hv,128]."""
    import torch
    for name, x in (("q", q), ("k", k), ("v", v), ("beta", beta)):
        _bf16_cuda(x, name)
    b_, hk = q.shape[0], q.shape[1]
    hv = v.shape[1]
    if tuple(state.shape) != (b_, hv, 128, 128) or state.dtype != torch.float32 or not state.is_contiguous():
        raise ValueError("state must be contiguous FP32 [B,Hv,128,128] in K-by-V order")
    if g.dtype not in (torch.bfloat16, torch.float32) or tuple(g.shape) != (b_, hv) or hv % hk:
        raise ValueError("g must be BF16/FP32 [B,Hv] and Hv % Hk == 0")
    lib = load_library()
    out = torch.empty_like(v)
    with torch.cuda.device(q.device):
        lib.check(lib.lib.actlize_la_sm100_decode_step(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), state.data_ptr(),
            out.data_ptr(), b_, hk, hv, int(g.dtype == torch.float32), torch.cuda.current_stream().cuda_stream))
    return out


def gdn_forward_projections(mixed, a, b, a_log, dt_bias, key_heads, value_heads, initial_state=None,
                            output_final_state=True):
    """The forward straight from the layer's projection outputs: ``mixed`` BF16 [B,T,(2Hk+Hv)*128] laid out
    [q heads | k heads | v heads], ``a``, ``b`` BF16 [B,T,Hv], ``a_log``, ``dt_bias`` FP32 [Hv].  Normalisation
    and gate activation happen inside the prepare kernel; the result equals ``gdn_prepare_inputs`` followed by
    ``gdn_forward`` bit for bit.  Returns (out [B,T,Hv,128] BF16, final state or None)."""
    import torch
    from .sm100 import load_sm100
    from .sm100_policy import select
    from .device import device_profile
    hk, hv = key_heads, value_heads
    if mixed.ndim != 3 or mixed.shape[2] != (2 * hk + hv) * 128 or hv % hk:
        raise ValueError("mixed must be [B,T,(2Hk+Hv)*128] with Hv % Hk == 0")
    _bf16_cuda(mixed, "mixed")
    _bf16_cuda(a, "a")
    _bf16_cuda(b, "b")
    bsz, t = mixed.shape[0], mixed.shape[1]
    if tuple(a.shape) != (bsz, t, hv) or tuple(b.shape) != (bsz, t, hv):
        raise ValueError("a and b must be [B,T,Hv]")
    for name, x in (("a_log", a_log), ("dt_bias", dt_bias)):
        if x.dtype != torch.float32 or x.numel() != hv or x.device != mixed.device or not x.is_contiguous():
            raise ValueError(f"{name} must be contiguous FP32 [Hv] on the inputs' device")
    if initial_state is not None and (tuple(initial_state.shape) != (bsz, hv, 128, 128) or
                                      initial_state.dtype != torch.float32 or not initial_state.is_contiguous()):
        raise ValueError("initial_state must be contiguous FP32 [B,Hv,128,128]")
    owner = load_sm100()
    owner.library.configure(mixed.device)
    lib = owner.library.lib
    config = select((bsz, t, hk, hv, 128, 128), device_profile(mixed.device.index)).configuration_id
    nbytes = lib.actlize_la_sm100_projections_workspace_bytes(bsz, t, hk, hv, config)
    if nbytes < 0:
        raise ValueError("geometry exceeds the native grid limits")
    workspace = owner._workspace(mixed.device, nbytes)
    out = torch.empty((bsz, t, hv, 128), dtype=torch.bfloat16, device=mixed.device)
    final = (torch.empty((bsz, hv, 128, 128), dtype=torch.float32, device=mixed.device)
             if output_final_state else None)
    with torch.cuda.device(mixed.device):
        owner.library.check(lib.actlize_la_sm100_forward_projections(
            mixed.data_ptr(), mixed.shape[2], a.data_ptr(), b.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(),
            initial_state.data_ptr() if initial_state is not None else None, out.data_ptr(),
            final.data_ptr() if final is not None else None, workspace.data_ptr(), nbytes, bsz, t, hk, hv, config,
            torch.cuda.current_stream().cuda_stream))
    return out, final


def _check_step_inputs(k, v, g, beta, state, width_axis):
    import torch
    b_, w, hk = k.shape[0], k.shape[1], k.shape[2]
    hv = v.shape[2] if v is not None else g.shape[2]
    if tuple(state.shape) != (b_, hv, 128, 128) or state.dtype != torch.float32 or not state.is_contiguous():
        raise ValueError("state must be contiguous FP32 [B,Hv,128,128] in K-by-V order")
    if g.dtype not in (torch.bfloat16, torch.float32) or tuple(g.shape) != (b_, w, hv) or hv % hk or not g.is_contiguous():
        raise ValueError("g must be contiguous BF16/FP32 [B,W,Hv] and Hv % Hk == 0")
    if not 1 <= w <= 64:
        raise ValueError("the step width must be 1..64 tokens")
    return b_, w, hk, hv


def gdn_verify_step(q, k, v, g, beta, state):
    """Speculative-decoding verify: q,k [B,W,Hk,128], v [B,W,Hv,128] BF16, g,beta [B,W,Hv]; ``state`` FP32
    [B,Hv,128,128] is READ ONLY.  Returns (out [B,W,Hv,128] BF16, delta [B,W,Hv,128] FP32); ``gdn_commit_step``
    applies the accepted prefix (the reference's verify/commit pair, csrc/serving/gdn.cu:152-217,255-300,
    without its slot pool)."""
    import torch
    for name, x in (("q", q), ("k", k), ("v", v), ("beta", beta)):
        _bf16_cuda(x, name)
    b_, w, hk, hv = _check_step_inputs(k, v, g, beta, state, 1)
    lib = load_library()
    out = torch.empty_like(v)
    delta = torch.empty(v.shape, dtype=torch.float32, device=v.device)
    with torch.cuda.device(q.device):
        lib.check(lib.lib.actlize_la_sm100_verify_step(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), state.data_ptr(),
            out.data_ptr(), delta.data_ptr(), b_, w, hk, hv, int(g.dtype == torch.float32),
            torch.cuda.current_stream().cuda_stream))
    return out, delta


def gdn_commit_step(k, g, delta, counts, state):
    """Apply the first ``counts[b]`` (int32 device tensor [B], 0..W) recorded updates of a verify step to ``state``
    in place: S <- e^{g_t} S + k_t delta_t^T."""
    import torch
    _bf16_cuda(k, "k")
    b_, w, hk, hv = _check_step_inputs(k, None, g, None, state, 1)
    if tuple(delta.shape) != (b_, w, hv, 128) or delta.dtype != torch.float32 or not delta.is_contiguous():
        raise ValueError("delta must be contiguous FP32 [B,W,Hv,128]")
    if counts.dtype != torch.int32 or tuple(counts.shape) != (b_,) or counts.device != state.device:
        raise ValueError("counts must be an int32 device tensor [B]")
    lib = load_library()
    with torch.cuda.device(k.device):
        lib.check(lib.lib.actlize_la_sm100_commit_step(
            k.data_ptr(), g.data_ptr(), delta.data_ptr(), counts.data_ptr(), state.data_ptr(), b_, w, hk, hv,
            int(g.dtype == torch.float32), torch.cuda.current_stream().cuda_stream))
    return state


def rmsnorm_gated(y, z, weight):
    """y, z [..., 128] BF16, weight [128] BF16 -> BF16 tensor shaped like y."""
    import torch
    _bf16_cuda(y, "y", 128)
    _bf16_cuda(z, "z", 128)
    _bf16_cuda(weight, "weight", 128)
    if y.shape != z.shape or weight.numel() != 128:
        raise ValueError("y and z must have the same shape and weight 128 entries")
    lib = load_library()
    out = torch.empty_like(y)
    with torch.cuda.device(y.device):
        lib.check(lib.lib.actlize_la_sm100_rmsnorm_gated(
            y.data_ptr(), z.data_ptr(), weight.data_ptr(), out.data_ptr(), y.numel() // 128,
            torch.cuda.current_stream().cuda_stream))
    return out
