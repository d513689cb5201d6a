"""Worker of tests/test_multi_gpu.py: one rank per GPU under torch.distributed.run.

Checks, against the CPU restatement of the reference (the stated tolerances) and against the unsplit
single-GPU forward on the same seeded inputs, that
(1) the sequence-parallel forward reproduces the output segments and the final state, for a slowly decaying
    gate (every rank's transition matrix matters: FP32 rounding of the affine fold `M S + b`) and for the
    benchmark gate (segments forget their incoming state; only the leading chunks are rewritten), and
(2) the (batch, head)-sharded forward returns bit-identical slabs.
Prints one line per rank that starts with "OK" or "FAIL".
"""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist

from actlizela_b200 import gdn_forward
from actlizela_b200.sequence_parallel import (capture_sequence_parallel, gdn_forward_sequence_parallel,
                                               segment_bounds)
from actlizela_b200.sharding import gdn_forward_sharded
from actlizela_b200.workloads import WORKLOADS, make_inputs


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        from oracle import gdn_oracle as oracle

        def against_oracle(out, final, want_out, want_state, rows):
            out, want = out.float().cpu(), want_out[:, rows[0]:rows[1]].float()
            fine = (out - want).abs().max().item() <= 2e-2 and ((out - want).norm() / want.norm()).item() <= 1e-2
            if final is not None:
                fine = fine and ((final.cpu() - want_state).norm() / want_state.norm()).item() <= 1e-3
            return fine

        w = WORKLOADS["cfg3"].sliced(batch=2, length=64 * 40 + 24, key_heads=2, value_heads=8)
        cpu = make_inputs(w)
        oracle_out, oracle_state = oracle.chunk_forward_fp32(*cpu, output_final_state=True)
        dev = [x.cuda() if x is not None else None for x in cpu]
        full_out, full_state = gdn_forward(*dev, output_final_state=True)
        bounds = segment_bounds(w.length, world)
        t0, t1 = bounds[rank]
        part = [x[:, t0:t1].contiguous() for x in dev[:5]]
        out, final = gdn_forward_sequence_parallel(*part, dev[5] if rank == 0 else None, True,
                                                   segment_lengths=[b1 - b0 for b0, b1 in bounds])
        torch.cuda.synchronize()
        want = full_out[:, t0:t1].float()
        rel_out = ((out.float() - want).norm() / want.norm()).item()
        ok = torch.equal(out, full_out[:, t0:t1]) if rank == 0 else rel_out < 1e-3
        ok = ok and against_oracle(out, final, oracle_out, oracle_state, (t0, t1))
        if rank < world - 1:
            ok = ok and final is None
        else:
            rel_state = ((final - full_state).norm() / full_state.norm()).item()
            ok = ok and rel_state < 1e-5
        pieces = gdn_forward_sharded(*dev, True, rank=rank, world_size=world)
        ok = ok and all(torch.equal(o, full_out[b0:b1, :, v0:v1]) and torch.equal(s, full_state[b0:b1, v0:v1])
                        for (b0, b1, v0, v1), o, s in pieces)
        # decayed form: with the benchmark gate the incoming state is gone after a few chunks of a segment, so the
        # ranks behind the first rewrite only those and keep the zero-state rows elsewhere
        w2 = WORKLOADS["cfg0"].sliced(batch=1, length=64 * 48 + 10, key_heads=2, value_heads=4, initial=0.1)
        cpu2 = make_inputs(w2)
        oracle_out2, oracle_state2 = oracle.chunk_forward_fp32(*cpu2, output_final_state=True)
        dev2 = [x.cuda() if x is not None else None for x in cpu2]
        full_out2, full_state2 = gdn_forward(*dev2, output_final_state=True)
        bounds2 = segment_bounds(w2.length, world)
        s0, s1 = bounds2[rank]
        part2 = [x[:, s0:s1].contiguous() for x in dev2[:5]]
        for vouched in (False, True):        # the exact form (decides on the device) and the caller's statement
            out2, final2 = gdn_forward_sequence_parallel(*part2, dev2[5] if rank == 0 else None, True,
                                                         until_decayed=vouched,
                                                         segment_lengths=[b1 - b0 for b0, b1 in bounds2])
            torch.cuda.synchronize()
            want2 = full_out2[:, s0:s1].float()
            ok = ok and ((out2.float() - want2).norm() / want2.norm()).item() < 1e-3
            ok = ok and (out2.float() - want2).abs().max().item() < 2e-2
            ok = ok and against_oracle(out2, final2, oracle_out2, oracle_state2, (s0, s1))
            if rank == world - 1:
                ok = ok and ((final2 - full_state2).norm() / full_state2.norm()).item() < 1e-4
        # the exact form captured in a CUDA graph (every launch and the exchange inside it) and replayed twice
        graph, out3, final3 = capture_sequence_parallel(*part2, dev2[5] if rank == 0 else None, True,
                                                        segment_lengths=[b1 - b0 for b0, b1 in bounds2])
        exact2, exact_final2 = gdn_forward_sequence_parallel(*part2, dev2[5] if rank == 0 else None, True,
                                                             segment_lengths=[b1 - b0 for b0, b1 in bounds2])
        for _ in range(2):
            out3.zero_()
            graph.replay()
            torch.cuda.synchronize()
            ok = ok and torch.equal(out3, exact2) and (final3 is None or torch.equal(final3, exact_final2))
        del graph
        print(f"{'OK' if ok else 'FAIL'} rank {rank} of {world}: tokens [{t0},{t1}), "
              f"slabs {[p[0] for p in pieces]}", flush=True)
        dist.barrier()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
