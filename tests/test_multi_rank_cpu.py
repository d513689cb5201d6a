"""World-size-2 (and 3) host logic of the multi-GPU paths, run as gloo ranks on CPU.

The device forward is replaced by the CPU oracle (injected as ``forward_fn``); what is under
test is the partitioning, the affine state hand-off and the send/recv choreography.
"""
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
    for length, world in [(131072, 8), (3000, 4), (65, 2), (64, 2), (1, 3)]:
        bounds = segment_bounds(length, world)
        assert bounds[0][0] == 0 and bounds[-1][1] == length
        for (a0, a1), (b0, _) in zip(bounds, bounds[1:]):
            assert a1 == b0 and a1 % 64 == 0 or a1 == length


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
            t0, t1 = segment_bounds(q.shape[1], world)[rank]
            part = [x[:, t0:t1].contiguous() for x in (q, k, v, g, beta)]
            out, final = gdn_forward_sequence_parallel(
                *part, init if rank == 0 else None, True, forward_fn=_oracle_forward)
            worst = oracle.max_abs(out, want_out[:, t0:t1])
            if rank == world - 1:
                worst = max(worst, oracle.rel_frobenius(final, want_state))
            else:
                assert final is None
            result_queue.put((rank, worst))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,world", [("shard", 2), ("sp", 2), ("sp", 3)])
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
