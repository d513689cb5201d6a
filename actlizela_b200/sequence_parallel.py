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


_DECAYED = -40.0      # natural log: below this a segment's transition matrix is treated as zero


def _neighbour(group, rank):
    import torch.distributed as dist
    return dist.get_global_rank(group, rank) if group else rank


def gdn_forward_sequence_parallel(q, k, v, g, beta, initial_state=None, output_final_state=True, *,
                                  group=None, forward_fn=None, apply_transition=None, segment_fn=None,
                                  until_decayed=False, **forward_options):
    """Forward over a sequence split across the ranks of ``group``.

    Every rank passes ITS OWN contiguous segment (q,k [B,Tr,Hk,128] ...), segments in rank
    order, every segment except the last a multiple of 64 tokens.  ``initial_state`` is read on
    rank 0 only.  Returns (output of the local segment, final state on the LAST rank or None).

    On CUDA tensors the ranks behind the first prepare their segment once and walk it several times
    (``Sm100Forward.prepare_segment``): offset and transition pass next to each other, then, once the incoming
    state has arrived, the final pass.  ``until_decayed=True`` replaces that final pass by a walk over the leading
    chunks only, those the incoming state still reaches with a weight above exp(-40) (valid when every chunk
    transition is a contraction, which holds for L2-normalised keys and beta in [0, 1]); the remaining rows keep
    the zero-state outputs and the final state comes from ``M S_in + b``.  ``forward_fn`` (any complete forward)
    selects the generic three-pass form instead; ``segment_fn`` substitutes the prepared-segment factory.
    """
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    b, t, _, d = q.shape
    hv = v.shape[2]
    staged = forward_fn is None and (segment_fn is not None or q.is_cuda)
    if forward_fn is None:
        from .gdn_interface import gdn_forward as forward_fn
    if apply_transition is None:
        apply_transition = native_apply_transition if q.is_cuda else _torch_apply_transition
    if world == 1:
        return forward_fn(q, k, v, g, beta, initial_state, output_final_state, **forward_options)
    if rank < world - 1 and t % 64:
        raise ValueError("every segment but the last must be a multiple of 64 tokens")
    state_shape = (b, hv, d, d)
    last = rank == world - 1

    if rank == 0:
        # the first segment starts from the caller's state; its final state is the next rank's incoming state
        out, final = forward_fn(q, k, v, g, beta, initial_state, True, **forward_options)
        dist.send(final, dst=_neighbour(group, 1), group=group)
        return out, None

    if staged:
        if forward_options:
            raise ValueError("forward options apply to the generic form (forward_fn) only")
        if segment_fn is None:
            from .sm100 import load_sm100
            segment_fn = load_sm100().prepare_segment
        segment = segment_fn(q, k, v, g, beta)
        incoming = torch.empty(state_shape, dtype=torch.float32, device=q.device)
        source, target = _neighbour(group, rank - 1), (None if last else _neighbour(group, rank + 1))
        # the whole segment's decay, per batch and value head: one small reduction and one host read
        if until_decayed and bool((g.float().sum(dim=1).max() < _DECAYED).item()):
            # M_r is below exp(-40): the outgoing state is b_r whatever comes in, so it leaves at once and all
            # hand-offs of the job overlap; the incoming state only reaches the leading chunks of the output
            offset = segment.offset_pipelined()
            ops = [dist.P2POp(dist.irecv, incoming, source, group)]
            if not last:
                ops.append(dist.P2POp(dist.isend, offset, target, group))
            for work in dist.batch_isend_irecv(ops):
                work.wait()
            out = segment.finish_decayed(incoming)
            return out, (offset if (last and output_final_state) else None)
        offset = transition = None
        if not last or until_decayed:
            offset, transition = segment.offset_and_transition(
                need_transition=not last or bool(output_final_state))
        else:
            segment.prepare()
        dist.recv(incoming, src=source, group=group)
        if not last:
            outgoing = apply_transition(transition, offset, incoming)
            dist.send(outgoing, dst=target, group=group)
        if until_decayed:
            out = segment.finish_decayed(incoming)
            final = apply_transition(transition, offset, incoming) if (last and output_final_state) else None
        else:
            out, final = segment.finish(incoming, bool(last and output_final_state))
        return out, (final if (last and output_final_state) else None)

    transition = offset = None
    if not last:
        # (M_r, b_r): two state-only passes over the local segment
        _, offset = forward_fn(q, k, v, g, beta, None, True, **forward_options)
        eye = torch.eye(d, dtype=torch.float32, device=q.device).expand(state_shape).contiguous()
        _, transition = forward_fn(q, k, torch.zeros_like(v), g, beta, eye, True, **forward_options)
    incoming = torch.empty(state_shape, dtype=torch.float32, device=q.device)
    dist.recv(incoming, src=_neighbour(group, rank - 1), group=group)
    if not last:
        outgoing = apply_transition(transition, offset, incoming)
        dist.send(outgoing, dst=_neighbour(group, rank + 1), group=group)
    out, final = forward_fn(q, k, v, g, beta, incoming, bool(output_final_state and last), **forward_options)
    return out, (final if (output_final_state and last) else None)
