"""Worker of tests/test_multi_gpu.py: one rank per GPU under torch.distributed.run.

Checks, against the unsplit single-GPU forward on the same seeded inputs, that
(1) the sequence-parallel forward returns bit-identical output segments and final state
    (segments are chunk aligned, so chunking and rounding are the same), and
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
from actlizela_b200.sequence_parallel import gdn_forward_sequence_parallel, segment_bounds
from actlizela_b200.sharding import gdn_forward_sharded
from actlizela_b200.workloads import WORKLOADS, make_inputs


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        w = WORKLOADS["cfg3"].sliced(batch=2, length=64 * 40 + 24, key_heads=2, value_heads=8)
        dev = [x.cuda() if x is not None else None for x in make_inputs(w)]
        full_out, full_state = gdn_forward(*dev, output_final_state=True)
        t0, t1 = segment_bounds(w.length, world)[rank]
        part = [x[:, t0:t1].contiguous() for x in dev[:5]]
        out, final = gdn_forward_sequence_parallel(*part, dev[5] if rank == 0 else None, True)
        torch.cuda.synchronize()
        ok = torch.equal(out, full_out[:, t0:t1])
        ok = ok and ((final is None) if rank < world - 1 else torch.equal(final, full_state))
        pieces = gdn_forward_sharded(*dev, True, rank=rank, world_size=world)
        ok = ok and all(torch.equal(o, full_out[b0:b1, :, v0:v1]) and torch.equal(s, full_state[b0:b1, v0:v1])
                        for (b0, b1, v0, v1), o, s in pieces)
        print(f"{'OK' if ok else 'FAIL'} rank {rank} of {world}: tokens [{t0},{t1}), "
              f"slabs {[p[0] for p in pieces]}", flush=True)
        dist.barrier()
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
