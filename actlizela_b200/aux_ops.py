"""The steps either side of the chunked forward, on the same native library.

* ``gdn_prepare_inputs``: Q/K L2 normalisation, gate activation and beta from a fused projection
  (reference: csrc/serving/prefill.cu:45-70, csrc/serving/runtime.cuh:48-52).
* ``gdn_decode_step``: one token on the FP32 ``[B,Hv,128,128]`` K-by-V state, in place
  (reference: actlize_la/reference/gdn_chunk_ref.py:135-143; csrc/serving/gdn.cu:152).
* ``rmsnorm_gated``: ``y * rsqrt(mean y^2 + 1e-6) * weight * silu(z)`` per 128-wide row
  (reference: actlize_la.rmsnorm_gated, docs/OUTPUT_GATE.md:7-15).
* ``out_proj_gemm``: ``A @ W^T`` with BF16 operands, the output projection behind ``rmsnorm_gated``
  (reference: actlize_la.out_proj_gemm / out_proj_gemm_cutlass, docs/OUTPUT_GATE.md:17-24).
The first three are single memory-bound kernels, the last one a tcgen05 GEMM; all are launched on the caller's
current stream.
"""
from __future__ import annotations

from ._library import load_library


def _operands(*specs):
    """Full check of every operand before a raw pointer of it reaches a kernel: shape and dtype first (so that the
    messages are about the caller's mistake), then one common CUDA device, contiguity, 16-byte alignment and no
    autograd.  ``specs`` are (name, tensor, expected shape, allowed dtypes)."""
    anchor = None
    for name, x, shape, dtypes in specs:
        if tuple(x.shape) != tuple(shape):
            raise ValueError(f"{name} must have shape {tuple(shape)}, not {tuple(x.shape)}")
        if x.dtype not in dtypes:
            raise ValueError(f"{name} must be of dtype {' or '.join(str(d) for d in dtypes)}, not {x.dtype}")
    for name, x, _, _ in specs:
        if x.device.type != "cuda":
            raise ValueError(f"{name} must be a CUDA tensor")
        anchor = anchor if anchor is not None else x.device
        if x.device != anchor:
            raise ValueError(f"{name} is on {x.device}, the other operands on {anchor}")
        if not x.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        if x.data_ptr() % 16:
            raise ValueError(f"{name} must be 16-byte aligned")
        if x.requires_grad:
            raise ValueError(f"{name} requires grad; these are forward-only operators")
    return anchor


def gdn_prepare_inputs(mixed, a, b, a_log, dt_bias, key_heads, value_heads):
    """mixed [N, (2Hk+Hv)*128] BF16, a,b [N,Hv] BF16, a_log, dt_bias [Hv] FP32 ->
    (q [N,Hk,128], k [N,Hk,128], v [N,Hv,128] BF16, g [N,Hv] FP32, beta [N,Hv] BF16)."""
    import torch
    bf16, fp32 = (torch.bfloat16,), (torch.float32,)
    if type(key_heads) is not int or type(value_heads) is not int or key_heads < 1 or value_heads % key_heads:
        raise ValueError("key_heads must be a positive integer that divides value_heads")
    if mixed.ndim != 2 or mixed.shape[1] != (2 * key_heads + value_heads) * 128:
        raise ValueError("mixed must be 2-D and hold [q heads | k heads | v heads] x 128 per row")
    n = mixed.shape[0]
    if mixed.dtype != torch.bfloat16 or mixed.stride(1) != 1 or mixed.stride(0) < mixed.shape[1] or mixed.stride(0) % 8:
        raise ValueError("mixed must be BF16 with unit inner stride and a row stride that is a multiple of 8 elements")
    _operands(("a", a, (n, value_heads), bf16), ("b", b, (n, value_heads), bf16),
              ("a_log", a_log, (value_heads,), fp32), ("dt_bias", dt_bias, (value_heads,), fp32))
    if mixed.device != a.device or mixed.data_ptr() % 16 or mixed.requires_grad:
        raise ValueError("mixed must be on the operands' CUDA device, 16-byte aligned and without grad")
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
    bf16, fp32 = (torch.bfloat16,), (torch.float32,)
    if q.ndim != 3 or v.ndim != 3:
        raise ValueError("q,k must be [B,Hk,128] and v [B,Hv,128]")
    b_, hk = q.shape[0], q.shape[1]
    hv = v.shape[1]
    if min(b_, hk, hv) < 1 or hv % hk:
        raise ValueError("sizes must be positive and Hv % Hk == 0")
    _operands(("q", q, (b_, hk, 128), bf16), ("k", k, (b_, hk, 128), bf16), ("v", v, (b_, hv, 128), bf16),
              ("g", g, (b_, hv), (torch.bfloat16, torch.float32)), ("beta", beta, (b_, hv), bf16),
              ("state", state, (b_, hv, 128, 128), fp32))
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
    bsz, t = mixed.shape[0], mixed.shape[1]
    bf16, fp32 = (torch.bfloat16,), (torch.float32,)
    specs = [("mixed", mixed, mixed.shape, bf16), ("a", a, (bsz, t, hv), bf16), ("b", b, (bsz, t, hv), bf16),
             ("a_log", a_log, (hv,), fp32), ("dt_bias", dt_bias, (hv,), fp32)]
    if initial_state is not None:
        specs.append(("initial_state", initial_state, (bsz, hv, 128, 128), fp32))
    _operands(*specs)
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


def _check_step_inputs(q, k, v, g, beta, state, delta=None, counts=None):
    """Operands of the verify / commit pair; ``q``, ``v``, ``beta`` (verify) and ``delta``, ``counts`` (commit) are
    checked when given."""
    import torch
    bf16, fp32 = (torch.bfloat16,), (torch.float32,)
    if k.ndim != 4 or g.ndim != 3:
        raise ValueError("k must be [B,W,Hk,128] and g [B,W,Hv]")
    b_, w, hk = k.shape[0], k.shape[1], k.shape[2]
    hv = g.shape[2]
    if min(b_, hk, hv) < 1 or hv % hk:
        raise ValueError("sizes must be positive and Hv % Hk == 0")
    if not 1 <= w <= 64:
        raise ValueError("the step width must be 1..64 tokens")
    specs = [("k", k, (b_, w, hk, 128), bf16), ("g", g, (b_, w, hv), (torch.bfloat16, torch.float32)),
             ("state", state, (b_, hv, 128, 128), fp32)]
    if q is not None:
        specs += [("q", q, (b_, w, hk, 128), bf16), ("v", v, (b_, w, hv, 128), bf16), ("beta", beta, (b_, w, hv), bf16)]
    if delta is not None:
        specs += [("delta", delta, (b_, w, hv, 128), fp32), ("counts", counts, (b_,), (torch.int32,))]
    _operands(*specs)
    return b_, w, hk, hv


def gdn_verify_step(q, k, v, g, beta, state):
    """Speculative-decoding verify: q,k [B,W,Hk,128], v [B,W,Hv,128] BF16, g,beta [B,W,Hv]; ``state`` FP32
    [B,Hv,128,128] is READ ONLY.  Returns (out [B,W,Hv,128] BF16, delta [B,W,Hv,128] FP32); ``gdn_commit_step``
    applies the accepted prefix (the reference's verify/commit pair, csrc/serving/gdn.cu:152-217,255-300,
    without its slot pool)."""
    import torch
    b_, w, hk, hv = _check_step_inputs(q, k, v, g, beta, state)
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
    b_, w, hk, hv = _check_step_inputs(None, k, None, g, None, state, delta, counts)
    lib = load_library()
    with torch.cuda.device(k.device):
        lib.check(lib.lib.actlize_la_sm100_commit_step(
            k.data_ptr(), g.data_ptr(), delta.data_ptr(), counts.data_ptr(), state.data_ptr(), b_, w, hk, hv,
            int(g.dtype == torch.float32), torch.cuda.current_stream().cuda_stream))
    return state


def rmsnorm_gated(y, z, weight):
    """y, z [..., 128] BF16, weight [128] BF16 -> BF16 tensor shaped like y."""
    import torch
    if y.ndim < 1 or y.shape[-1] != 128:
        raise ValueError("y must have a last dimension of 128")
    bf16 = (torch.bfloat16,)
    _operands(("y", y, y.shape, bf16), ("z", z, y.shape, bf16), ("weight", weight, (128,), bf16))
    lib = load_library()
    out = torch.empty_like(y)
    with torch.cuda.device(y.device):
        lib.check(lib.lib.actlize_la_sm100_rmsnorm_gated(
            y.data_ptr(), z.data_ptr(), weight.data_ptr(), out.data_ptr(), y.numel() // 128,
            torch.cuda.current_stream().cuda_stream))
    return out


def out_proj_gemm(a, w):
    """C = A @ W^T: A [M,K] BF16 row-major, W [N,K] BF16 (Linear weight layout), FP32 accumulation, C [M,N] BF16.
    K and N must be multiples of 8.  One tcgen05 kernel on the caller's current stream."""
    import torch
    if a.ndim != 2 or w.ndim != 2:
        raise ValueError("A must be [M,K] and W [N,K]")
    m, k = a.shape
    n = w.shape[0]
    if min(m, n, k) < 1 or k % 8 or n % 8:
        raise ValueError("sizes must be positive and K, N multiples of 8")
    bf16 = (torch.bfloat16,)
    device = _operands(("A", a, (m, k), bf16), ("W", w, (n, k), bf16))
    lib = load_library()
    lib.configure(device)
    c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    with torch.cuda.device(device):
        lib.check(lib.lib.actlize_la_sm100_out_proj(a.data_ptr(), w.data_ptr(), c.data_ptr(), m, n, k,
                                                    torch.cuda.current_stream().cuda_stream))
    return c
