"""World-size-2 (and 3) host logic of the multi-GPU paths, run as gloo ranks on CPU.

The device forward is replaced by the CPU oracle (injected as ``forward_fn``); what is under
test is the partitioning, the affine state hand-off and the send/recv choreography.
"""
import contextlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from actlizela_b200.sequence_parallel import gdn_forward_sequence_parallel, segment_bounds
from actlizela_b200.sharding import gdn_forward_sharded, shard_plan
from oracle import gdn_oracle as oracle
from tests.cases import build_case


def _oracle_forward(q, k, v, g, beta, initial_state=None, output_final_state=True, **_):
    out, state = oracle.wy_chunk_forward(q, k, v, g, beta, initial_state, dtype=torch.float64)
    return out.to(torch.float32), (state.to(torch.float32) if output_final_state else None)


class _OracleSegment:
    """CPU stand-in for Sm100Forward.prepare_segment: same methods, the oracle instead of the kernels."""

    def __init__(self, q, k, v, g, beta):
        self.tensors = (q, k, v, g, beta)
        self.output = None

    def early_pair(self, need_transition=True):
        q, k, v, g, beta = self.tensors
        _, offset = _oracle_forward(q, k, v, g, beta, None)
        transition = None
        if need_transition:
            eye = torch.eye(128).expand(q.shape[0], v.shape[2], 128, 128).contiguous()
            _, transition = _oracle_forward(q, k, torch.zeros_like(v), g, beta, eye)
        return offset, transition

    def walk_outputs(self, initial=None):
        self.output, _ = _oracle_forward(*self.tensors, initial)
        return self.output

    def side(self):
        return contextlib.nullcontext()

    def join(self, *tensors):
        pass

    def finish(self, incoming, output_final_state=True):
        return _oracle_forward(*self.tensors, incoming, output_final_state)

    def finish_decayed(self, incoming):
        """Rewrite, per (batch, value head), the chunks up to and including the first one at whose end the decay
        accumulated since the segment start is below exp(-40): the walk kernel's rule."""
        q, k, v, g, beta = self.tensors
        full, _ = _oracle_forward(q, k, v, g, beta, incoming)
        total = g.double().cumsum(1)                                   # [B, T, Hv]
        chunks = (q.shape[1] + 63) // 64
        for b in range(q.shape[0]):
            for h in range(v.shape[2]):
                stop = chunks
                for c in range(chunks):
                    if total[b, min(q.shape[1], (c + 1) * 64) - 1, h] < -40.0:
                        stop = c + 1
                        break
                self.output[b, :stop * 64, h] = full[b, :stop * 64, h]
        return self.output


def test_shard_plan_covers_every_unit_exactly_once():
    for batch, hk, world in [(8, 16, 8), (8, 16, 2), (1, 16, 8), (3, 5, 4), (2, 2, 8), (1, 1, 2)]:
        seen = []
        for pieces in shard_plan(batch, hk, world):
            for b, h0, h1 in pieces:
                assert 0 <= h0 < h1 <= hk
                seen += [(b, h) for h in range(h0, h1)]
        assert sorted(seen) == [(b, h) for b in range(batch) for h in range(hk)]
        assert len(seen) == len(set(seen))


def test_segment_bounds_are_chunk_aligned():
    for length, world in [(131072, 8), (3000, 4), (65, 2), (129, 3), (64, 1)]:
        bounds = segment_bounds(length, world)
        assert bounds[0][0] == 0 and bounds[-1][1] == length
        assert all(b1 > b0 for b0, b1 in bounds)                      # nobody is left without tokens
        for (a0, a1), (b0, _) in zip(bounds, bounds[1:]):
            assert a1 == b0 and a1 % 64 == 0 or a1 == length
    for length, world in [(64, 2), (1, 3), (128, 3)]:                 # fewer chunks than ranks
        with pytest.raises(ValueError, match="too few"):
            segment_bounds(length, world)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, result_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = dict(name="mr", kind="admission", batch=2, length=300, key_heads=2, value_heads=4,
                    gate=-0.05, fp32_gate=True, vary_gate=True, initial=True)
        q, k, v, g, beta, init = build_case(case)
        init = init * 50
        want_out, want_state = _oracle_forward(q, k, v, g, beta, init)
        if mode == "shard":
            worst = 0.0
            for (b0, b1, v0, v1), out, final in gdn_forward_sharded(
                    q, k, v, g, beta, init, True, rank=rank, world_size=world, forward_fn=_oracle_forward):
                worst = max(worst, oracle.max_abs(out, want_out[b0:b1, :, v0:v1]),
                            oracle.max_abs(final, want_state[b0:b1, v0:v1]))
            covered = torch.tensor([sum((b1 - b0) * (v1 - v0) for (b0, b1, v0, v1), _, _ in
                                        gdn_forward_sharded(q, k, v, g, beta, init, False, rank=rank,
                                                            world_size=world, forward_fn=_oracle_forward))])
            dist.all_reduce(covered)
            assert covered.item() == 2 * 4
            result_queue.put((rank, worst))
        else:
            if mode.startswith("sp-decayed"):
                # strong decay: the incoming state is gone within the first chunks of a segment, which is what a
                # caller of until_decayed=True vouches for; the weaker variant does not empty a whole segment and
                # goes through the exact form, whose final pass still stops where a head has decayed
                g = g * (25.0 if mode == "sp-decayed" else 4.0)
                want_out, want_state = _oracle_forward(q, k, v, g, beta, init)
            bounds = segment_bounds(q.shape[1], world)
            lengths = [b1 - b0 for b0, b1 in bounds] if mode != "sp-staged" else None     # None: gathered first
            t0, t1 = bounds[rank]
            part = [x[:, t0:t1].contiguous() for x in (q, k, v, g, beta)]
            if mode == "sp":
                out, final = gdn_forward_sequence_parallel(
                    *part, init if rank == 0 else None, True, forward_fn=_oracle_forward, segment_lengths=lengths)
            else:
                # the staged form: one prepared segment per rank, walked several times
                out, final = gdn_forward_sequence_parallel(
                    *part, init if rank == 0 else None, True, segment_fn=_OracleSegment,
                    until_decayed=(mode == "sp-decayed"), segment_lengths=lengths)
            if mode == "sp" and world == 3:
                # a segment that is not a multiple of 64 tokens is refused on every rank alike, before any message
                try:
                    gdn_forward_sequence_parallel(*part, None, True, forward_fn=_oracle_forward,
                                                  segment_lengths=[64, 63, q.shape[1] - 127])
                except ValueError:
                    pass
                else:
                    raise AssertionError("bad segment lengths were accepted")
            worst = oracle.max_abs(out, want_out[:, t0:t1])
            if rank == world - 1:
                worst = max(worst, oracle.rel_frobenius(final, want_state))
            else:
                assert final is None
            result_queue.put((rank, worst))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,world", [("shard", 2), ("sp", 2), ("sp", 3), ("sp-staged", 2), ("sp-staged", 3),
                                        ("sp-staged", 4), ("sp-decayed", 3), ("sp-decayed-partly", 3)])
def test_two_rank_paths_match_the_unsplit_run(mode, world):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert len(results) == world
    for rank, worst in results:
        assert worst < 2e-5, (mode, rank, worst)
