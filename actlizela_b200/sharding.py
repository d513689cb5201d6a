"""(batch, head) sharding of gdn_forward over the GPUs of one node: no collective.

Work units (batch, value head) are independent (the reference's scheduler states that CTAs
do not cooperate: csrc/backends/sm90/cula/kda/sm90/kernel/tile_scheduler.hpp:74).  Units are
dealt out in whole key-head groups (the Hv/Hk value heads that share one q/k head) so that
no q/k slice is needed on two ranks.  Each rank runs the ordinary single-device forward on
its slice; nothing is exchanged on the data path.
"""
from __future__ import annotations


def shard_plan(batch, key_heads, world_size):
    """Contiguous split of the B*Hk (batch, key-head group) units over the ranks.

    Returns, per rank, a list of (batch index, first key head, one-past-last key head).
    """
    if min(batch, key_heads, world_size) < 1:
        raise ValueError("batch, key_heads and world_size must be positive")
    units = batch * key_heads
    plan = []
    for rank in range(world_size):
        first, last = rank * units // world_size, (rank + 1) * units // world_size
        pieces = []
        unit = first
        while unit < last:
            b, h = divmod(unit, key_heads)
            stop = min(key_heads, h + (last - unit))
            pieces.append((b, h, stop))
            unit += stop - h
        plan.append(pieces)
    return plan


def _merge_batches(pieces, key_heads):
    """Fuse runs of whole consecutive batches into (b0, b1, 0, Hk) slabs; keep partial ones."""
    merged = []
    for b, h0, h1 in pieces:
        whole = h0 == 0 and h1 == key_heads
        if whole and merged and merged[-1][2:] == (0, key_heads) and merged[-1][1] == b:
            merged[-1] = (merged[-1][0], b + 1, 0, key_heads)
        else:
            merged.append((b, b + 1, h0, h1))
    return merged


def gdn_forward_sharded(q, k, v, g, beta, initial_state=None, output_final_state=True, *,
                        rank, world_size, forward_fn=None, **forward_options):
    """Run this rank's share of a (batch, head)-sharded forward.

    All ranks pass tensors of the full logical shape (or views of it); only this rank's
    slices are read.  Returns a list of ``((b0, b1, hv0, hv1), output, final_state)`` slabs:
    output [b1-b0, T, hv1-hv0, 128] and the matching final state (or None).
    """
    if forward_fn is None:
        from .gdn_interface import gdn_forward as forward_fn
    hk, hv = q.shape[2], v.shape[2]
    ratio = hv // hk
    results = []
    for b0, b1, h0, h1 in _merge_batches(shard_plan(q.shape[0], hk, world_size)[rank], hk):
        v0, v1 = h0 * ratio, h1 * ratio
        part = [q[b0:b1, :, h0:h1].contiguous(), k[b0:b1, :, h0:h1].contiguous(),
                v[b0:b1, :, v0:v1].contiguous(), g[b0:b1, :, v0:v1].contiguous(),
                beta[b0:b1, :, v0:v1].contiguous()]
        init = initial_state[b0:b1, v0:v1].contiguous() if initial_state is not None else None
        out, final = forward_fn(*part, init, output_final_state, **forward_options)
        results.append(((b0, b1, v0, v1), out, final))
    return results
