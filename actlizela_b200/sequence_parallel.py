"""Sequence-parallel gdn_forward: contiguous token segments, one per rank, one exchange step.

A token segment acts on the recurrent state as an affine map ``S_out = M S_in + b``
(composition rule of the reference's two-level scan, csrc/gdn_chunk/gdn_scan_stage2.cu:4-8;
the reference itself has no multi-device path).  Because the recurrence treats every state
column independently, ``b`` is the final state of the segment run from a zero state and
``M`` is the final state of the same recurrence run with ``v = 0`` from the identity.

Scheme (exact for any decay):
  1. every rank but the first and the last computes (M_r, b_r) of its own segment, in parallel;
  2. the incoming states are chained rank to rank, ``S_in(r+1) = M_r S_in(r) + b_r``, with one
     point-to-point message of B*Hv FP32 128x128 blocks per hop (NCCL send/recv on GPUs);
  3. every rank runs the ordinary forward on its segment from its true incoming state.
Segment boundaries must be multiples of the chunk size (64) so that chunking, and therefore
rounding, is the same as in the unsplit run.
"""
from __future__ import annotations

import torch


def segment_bounds(length, world_size, chunk=64):
    """Token range of each rank: whole chunks, as even as possible."""
    chunks = (length + chunk - 1) // chunk
    bounds = []
    for rank in range(world_size):
        c0, c1 = rank * chunks // world_size, (rank + 1) * chunks // world_size
        bounds.append((min(length, c0 * chunk), min(length, c1 * chunk)))
    return bounds


def _torch_apply_transition(m, b, s):
    return torch.baddbmm(b.flatten(0, 1), m.flatten(0, 1), s.flatten(0, 1)).view_as(s)


def native_apply_transition(m, b, s):
    """out = M @ S + b on the device through the native library (FP32 CUDA-core kernel)."""
    from ._library import load_library
    lib = load_library()
    out = torch.empty_like(s)
    with torch.cuda.device(s.device):
        lib.check(lib.lib.actlize_la_sm100_apply_transition(
            m.data_ptr(), b.data_ptr(), s.data_ptr(), out.data_ptr(),
            s.shape[0] * s.shape[1], torch.cuda.current_stream().cuda_stream))
    return out


def gdn_forward_sequence_parallel(q, k, v, g, beta, initial_state=None, output_final_state=True, *,
                                  group=None, forward_fn=None, apply_transition=None,
                                  **forward_options):
    """Forward over a sequence split across the ranks of ``group``.

    Every rank passes ITS OWN contiguous segment (q,k [B,Tr,Hk,128] ...), segments in rank
    order, every segment except the last a multiple of 64 tokens.  ``initial_state`` is read on
    rank 0 only.  Returns (output of the local segment, final state on the LAST rank or None).
    """
    import torch.distributed as dist
    if forward_fn is None:
        from .gdn_interface import gdn_forward as forward_fn
    if apply_transition is None:
        apply_transition = native_apply_transition if q.is_cuda else _torch_apply_transition
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, t, _, d = q.shape
    hv = v.shape[2]
    if world == 1:
        return forward_fn(q, k, v, g, beta, initial_state, output_final_state, **forward_options)
    if rank < world - 1 and t % 64:
        raise ValueError("every segment but the last must be a multiple of 64 tokens")

    state_shape = (b, hv, d, d)
    if rank == 0:
        incoming = initial_state
    else:
        transition = offset = None
        if rank < world - 1:
            # (M_r, b_r): two state-only passes over the local segment
            _, offset = forward_fn(q, k, v, g, beta, None, True, **forward_options)
            eye = torch.eye(d, dtype=torch.float32, device=q.device).expand(state_shape).contiguous()
            _, transition = forward_fn(q, k, torch.zeros_like(v), g, beta, eye, True, **forward_options)
        incoming = torch.empty(state_shape, dtype=torch.float32, device=q.device)
        dist.recv(incoming, src=dist.get_global_rank(group, rank - 1) if group else rank - 1, group=group)
        if rank < world - 1:
            outgoing = apply_transition(transition, offset, incoming)
            dist.send(outgoing, dst=dist.get_global_rank(group, rank + 1) if group else rank + 1, group=group)
    # rank 0's final state is the next rank's incoming state; the last rank's is the result
    want_final = True if rank == 0 else bool(output_final_state and rank == world - 1)
    out, final = forward_fn(q, k, v, g, beta, incoming, want_final, **forward_options)
    if rank == 0:
        dist.send(final, dst=dist.get_global_rank(group, 1) if group else 1, group=group)
    return out, (final if (output_final_state and rank == world - 1) else None)
