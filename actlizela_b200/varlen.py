"""Packed variable-length sequences.

The reference's serving prefill pads every request into a fixed ``[R, W]`` batch before its forward
(csrc/serving/prefill.cu:196-255).  Here the sequences stay packed: ``q,k,v,g,beta`` are
``[1, total_tokens, H, ...]`` and ``cu_seqlens`` (host integers, or an int32 device tensor, length N+1) marks
the boundaries.
The default path is the native entry ``actlize_la_sm100_forward_varlen``: one prepare and one walk launch
for all sequences, every sequence chunked from its own start.  ``per_sequence=True`` instead hands each
sequence (a contiguous slice) to the fixed-shape forward, two launches per sequence; both produce the same
bits and the second exists as a cross-check.
"""
from __future__ import annotations


def gdn_forward_varlen(q, k, v, g, beta, cu_seqlens, initial_states=None, output_final_state=True, *,
                       per_sequence=False, forward_fn=None, **forward_options):
    """Returns (output [1,total,Hv,128] BF16, final states [N,Hv,128,128] FP32 or None).

    ``initial_states`` is FP32 ``[N,Hv,128,128]`` or None; sequences of length 0 keep their state.
    """
    import torch
    if isinstance(cu_seqlens, torch.Tensor) and cu_seqlens.is_cuda and not per_sequence and forward_fn is None:
        # int32 offsets in device memory go to the native entry untouched (no host read; capturable)
        if forward_options:
            raise ValueError("forward options apply to the per-sequence path only")
        from .sm100 import load_sm100
        return load_sm100().varlen(q, k, v, g, beta, cu_seqlens, initial_states, output_final_state)
    bounds = [int(x) for x in cu_seqlens]
    if q.shape[0] != 1 or len(bounds) < 2 or bounds[0] != 0 or bounds[-1] != q.shape[1]:
        raise ValueError("varlen expects batch 1 and cu_seqlens running from 0 to the token count")
    if any(b1 < b0 for b0, b1 in zip(bounds, bounds[1:])):
        raise ValueError("cu_seqlens must be non-decreasing")
    if not per_sequence and forward_fn is None:
        if forward_options:
            raise ValueError("forward options apply to the per-sequence path only")
        from .sm100 import load_sm100
        return load_sm100().varlen(q, k, v, g, beta, bounds, initial_states, output_final_state)
    if forward_fn is None:
        from .gdn_interface import gdn_forward as forward_fn
    n, hv = len(bounds) - 1, v.shape[2]
    out = torch.empty_like(v)
    finals = (torch.empty((n, hv, 128, 128), dtype=torch.float32, device=q.device)
              if output_final_state else None)
    for i, (t0, t1) in enumerate(zip(bounds, bounds[1:])):
        init = initial_states[i:i + 1] if initial_states is not None else None
        if t1 == t0:
            if finals is not None:
                finals[i] = init[0] if init is not None else 0
            continue
        o, s = forward_fn(q[:, t0:t1], k[:, t0:t1], v[:, t0:t1], g[:, t0:t1], beta[:, t0:t1],
                          init, output_final_state, **forward_options)
        out[:, t0:t1] = o
        if finals is not None:
            finals[i] = s[0]
    return out, finals
