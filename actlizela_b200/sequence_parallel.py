"""Sequence-parallel gdn_forward: contiguous token segments, one per rank, one exchange step.

A token segment acts on the recurrent state as an affine map ``S_out = M S_in + b``
(composition rule of the reference's two-level scan, csrc/gdn_chunk/gdn_scan_stage2.cu:4-8;
the reference itself has no multi-device path).  Because the recurrence treats every state
column independently, ``b`` is the final state of the segment run from a zero state and
``M`` is the final state of the same recurrence run with ``v = 0`` from the identity.

Scheme (exact for any decay, no host read anywhere):
  1. every rank prepares its segment once.  One short launch behind the prepare kernel gives the pair early: ``b_r``
     from a zero-state walk of only the suffix of the segment that decides the outgoing state (the chunks since the
     decay fell below exp(-40), counted from the segment's end; the whole segment when there is no such suffix), and
     ``M_r`` from the identity with ``v = 0`` (exact zeros at once for a segment that decays below exp(-40)); both
     decisions are made on the device from the gate sums.  Then the stream walks the segment's output rows from a
     zero state (rank 0: from the caller's state);
  2. next to that walk, one grouped exchange of point-to-point messages: every rank sends its pair ``(M_r, b_r)``
     to every LATER rank (rank 0 sends its true outgoing state as ``b_0``) and receives the pairs of every EARLIER
     rank; the exclusive scan ``S_in(r) = M_{r-1} S_in(r-1) + b_{r-1}`` is then folded locally, in one kernel
     launch.  All messages of the job are in flight at the same time (NCCL send/recv over NVLink on GPUs), so the
     exchange costs one message latency instead of a chain of dependent hops, and that latency hides behind the
     output walk;
  3. every rank rewrites the leading chunks of its output that its incoming state still reaches (the walk stops,
     per batch and value head, at the first chunk boundary where the decay since the segment start is below
     exp(-40); a head that never gets there is rewritten to the end); the last rank forms the final state
     ``M_r S_in + b_r``.
Segment boundaries must be multiples of the chunk size (64) so that chunking, and therefore
rounding, is the same as in the unsplit run.
"""
from __future__ import annotations

import torch


def segment_bounds(length, world_size, chunk=64):
    """Token range of each rank: whole chunks, as even as possible."""
    chunks = (length + chunk - 1) // chunk
    if world_size < 1 or chunks < world_size:
        raise ValueError(f"{length} tokens are {chunks} chunks of {chunk}: too few for {world_size} ranks")
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
            s.shape[0] * s.shape[1], lib.current_stream_handle(s.device.index)))
    return out


def native_fold_transitions(pairs, transition, offset, want_outgoing):
    """Incoming state of a rank from the pairs of all earlier ranks, and optionally its outgoing state
    ``M_r S_in + b_r``, in ONE launch (``actlize_la_sm100_fold_transitions``).  ``pairs`` is
    [n, 2, B, Hv, 128, 128] with (M_j, b_j) of rank j at [j]; M_0 is not read."""
    from ._library import load_library
    lib = load_library()
    incoming = torch.empty_like(pairs[0, 1])
    outgoing = torch.empty_like(incoming) if want_outgoing else None
    with torch.cuda.device(pairs.device):
        lib.check(lib.lib.actlize_la_sm100_fold_transitions(
            pairs.data_ptr(), pairs.shape[0], transition.data_ptr() if want_outgoing else None,
            offset.data_ptr() if want_outgoing else None, incoming.data_ptr(),
            outgoing.data_ptr() if want_outgoing else None, pairs.shape[2] * pairs.shape[3],
            lib.current_stream_handle(pairs.device.index)))
    return incoming, outgoing


def _neighbour(group, rank):
    import torch.distributed as dist
    return dist.get_global_rank(group, rank) if group else rank


def _check_segments(t, rank, world, group, segment_lengths, device):
    """Every rank raises the same error, before any state message is posted: a bad segment must not leave its
    neighbours waiting in a receive.  With ``segment_lengths`` (the token count of every rank, known to all) the
    check is local; without it the lengths are gathered first, which costs one small collective and a host read."""
    import torch.distributed as dist
    if segment_lengths is None:
        mine = torch.tensor([t], dtype=torch.int64, device=device)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine, group=group)
        segment_lengths = [int(x.item()) for x in gathered]
    segment_lengths = [int(x) for x in segment_lengths]
    if len(segment_lengths) != world or segment_lengths[rank] != t:
        raise ValueError("segment_lengths must list the token count of every rank, this rank's included")
    if any(n < 1 for n in segment_lengths):
        raise ValueError("every rank needs at least one token (fewer chunks than ranks?)")
    if any(n % 64 for n in segment_lengths[:-1]):
        raise ValueError("every segment but the last must be a multiple of 64 tokens")


def gdn_forward_sequence_parallel(q, k, v, g, beta, initial_state=None, output_final_state=True, *,
                                  group=None, forward_fn=None, apply_transition=None, segment_fn=None,
                                  until_decayed=False, segment_lengths=None, **forward_options):
    """Forward over a sequence split across the ranks of ``group``.

    Every rank passes ITS OWN contiguous segment (q,k [B,Tr,Hk,128] ...), segments in rank
    order, every segment except the last a multiple of 64 tokens.  ``initial_state`` is read on
    rank 0 only.  Returns (output of the local segment, final state on the LAST rank or None).
    ``segment_lengths`` (token count of every rank) lets the arguments be checked without communication.

    On CUDA tensors every rank prepares its segment once and walks it several times
    (``Sm100Forward.prepare_segment``), see the module text.  ``until_decayed=True`` is the caller's statement
    that every segment forgets its incoming state (decay below exp(-40) within the segment, every token a
    contraction: L2-normalised keys, beta in [0, 1]); the transition pass is then skipped and only ``b_{r-1}``
    travels, from each rank to the next.  ``forward_fn`` (any complete forward) selects the generic three-pass
    form on complete forwards instead; ``segment_fn`` substitutes the prepared-segment factory.
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
    _check_segments(t, rank, world, group, segment_lengths, q.device)
    if staged and forward_options:
        raise ValueError("forward options apply to the generic form (forward_fn) only")
    state_shape = (b, hv, d, d)
    last = rank == world - 1
    new_state = lambda: torch.empty(state_shape, dtype=torch.float32, device=q.device)
    later = [_neighbour(group, r) for r in range(rank + 1, world)]

    fold = native_fold_transitions if (q.is_cuda and apply_transition is native_apply_transition) else None

    def exchange(offset, transition, want_outgoing=False, pair=None):
        """Post this rank's pair to every later rank and collect the pairs of every earlier rank, all at once: one
        message per (source, target), the pair travelling as one [2, B, Hv, 128, 128] block (``pair``, when the
        caller already holds transition and offset back to back).  Returns (incoming state of this rank, its
        outgoing state if asked for); (None, None) on rank 0."""
        ops = []
        pairs = torch.empty((rank, 2) + state_shape, dtype=torch.float32, device=q.device) if rank else None
        for r in range(rank):                              # rank 0 sends its outgoing state only
            ops.append(dist.P2POp(dist.irecv, pairs[r] if r else pairs[0, 1], _neighbour(group, r), group))
        if later:
            if transition is None:
                message = offset
            else:
                message = pair if pair is not None else torch.stack((transition, offset))
            ops += [dist.P2POp(dist.isend, message, target, group) for target in later]
        for work in (dist.batch_isend_irecv(ops) if ops else []):
            work.wait()
        if pairs is None:
            return None, None
        if fold is not None:
            return fold(pairs, transition, offset, want_outgoing)
        state = pairs[0, 1]
        for j in range(1, rank):
            state = apply_transition(pairs[j, 0], pairs[j, 1], state)
        return state, (apply_transition(transition, offset, state) if want_outgoing else None)

    if staged:
        if segment_fn is None:
            # the segment is finished with when this call returns: its workspace can be the stream's standing one
            from .sm100 import load_sm100
            segment = load_sm100().prepare_segment(q, k, v, g, beta, reuse_workspace=True)
        else:
            segment = segment_fn(q, k, v, g, beta)
        # the pair leaves early (one short launch), so the exchange runs on a side stream next to the long output walk
        offset, transition = segment.early_pair(need_transition=not until_decayed)
        segment.walk_outputs(initial_state if rank == 0 else None)
        incoming = final = None
        with segment.side():
            if rank == 0 and transition is not None and initial_state is not None:
                offset = apply_transition(transition, offset, initial_state)     # true outgoing state of rank 0
            if until_decayed:
                # the caller vouches that M_r is below exp(-40): b_r is the outgoing state, whatever comes in
                ops = []
                if rank:
                    incoming = new_state()
                    ops.append(dist.P2POp(dist.irecv, incoming, _neighbour(group, rank - 1), group))
                if not last:
                    ops.append(dist.P2POp(dist.isend, offset, later[0], group))
                for work in dist.batch_isend_irecv(ops):
                    work.wait()
                final = offset
            else:
                incoming, final = exchange(offset, None if rank == 0 else transition,
                                           want_outgoing=bool(rank and last and output_final_state),
                                           pair=getattr(segment, "pair", None))
        segment.join(incoming, final)
        out = segment.finish_decayed(incoming) if rank else segment.output
        return out, (final if (last and output_final_state) else None)

    if rank == 0:
        # the first segment starts from the caller's state; its true outgoing state plays the part of b_0
        out, final = forward_fn(q, k, v, g, beta, initial_state, True, **forward_options)
        exchange(final, None)
        return out, None

    # generic form on complete forwards: (M_r, b_r) by two state-only passes, the same exchange, a third pass
    _, offset = forward_fn(q, k, v, g, beta, None, True, **forward_options)
    eye = torch.eye(d, dtype=torch.float32, device=q.device).expand(state_shape).contiguous()
    _, transition = forward_fn(q, k, torch.zeros_like(v), g, beta, eye, True, **forward_options)
    incoming, _ = exchange(offset, transition)
    out, final = forward_fn(q, k, v, g, beta, incoming, bool(output_final_state and last), **forward_options)
    return out, (final if (output_final_state and last) else None)


def capture_sequence_parallel(q, k, v, g, beta, initial_state=None, output_final_state=True, **options):
    """One ``gdn_forward_sequence_parallel`` call captured in a CUDA graph, on every rank of the group alike.

    Returns ``(graph, output, final_state)``: ``graph.replay()`` runs the whole call again (prepare, the short
    pair launch, the output walk, the NCCL exchange on its side stream, fold and correction) on the CURRENT
    contents of the argument tensors and refills ``output`` / ``final_state`` in place.  A replay costs the host a
    few microseconds instead of the few hundred an eager call needs to enqueue its launches and messages, which is
    what limits many ranks with short segments.  Every rank must capture, and later replay, the same number of
    times in the same order (the exchange inside is a collective).
    """
    if not q.is_cuda:
        raise ValueError("capture needs CUDA tensors")
    call = lambda: gdn_forward_sequence_parallel(q, k, v, g, beta, initial_state, output_final_state, **options)
    current = torch.cuda.current_stream()
    warm = torch.cuda.Stream(device=q.device)
    warm.wait_stream(current)
    with torch.cuda.stream(warm):                # lazy set-up (communicators, streams, caches) happens outside capture
        for _ in range(2):
            call()
    current.wait_stream(warm)
    torch.cuda.synchronize(q.device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        output, final_state = call()
    return graph, output, final_state
