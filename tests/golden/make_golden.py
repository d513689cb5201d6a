#!/usr/bin/env python3
"""Generate the golden fixtures from the reference project itself and pin the CPU oracle.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/actlizeLA

For every case it (1) builds the seeded inputs, (2) runs the reference's own CPU path
(``actlize_la.reference.gdn_chunk_ref.torch_chunk_gated_delta_rule`` in FP32, with q/k
repeated over the value-head group as the reference's callers do), (3) cross-checks it
against the reference's independent algebra (``tests/wy_cpu.recurrent_double``,
``tests/residual_cpu.residual_forward(rounded=False)``, ``tests/wy_cpu.wy_forward``),
(4) checks this repository's CPU restatement (``oracle/gdn_oracle.py``) against all of
them, and (5) stores the reference's output and final state in ``golden_cases.npz``
together with a SHA-256 of the input bytes, so that the fixtures are usable where the
reference is absent.  The reference ships no stored tensors of its own; its tests pin the
path through seeded fixtures and FP64 identities, which is what is reproduced here.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.cases import ADMISSION_CASES, SCALED_WORKLOAD_CASES, build_case  # noqa: E402
from oracle import gdn_oracle as oracle  # noqa: E402


def digest(tensors):
    h = hashlib.sha256()
    for t in tensors:
        if t is not None:
            h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", type=Path, required=True, help="checkout of the reference project")
    ap.add_argument("--out", type=Path, default=Path(__file__).with_name("golden_cases.npz"))
    args = ap.parse_args()
    sys.path[:0] = [str(args.reference), str(args.reference / "tests")]
    from actlize_la.reference.gdn_chunk_ref import (torch_chunk_gated_delta_rule,
                                                     torch_recurrent_gated_delta_rule)
    from residual_cpu import residual_forward
    from wy_cpu import recurrent_double, wy_forward

    torch.manual_seed(0)
    arrays, index = {}, {}
    for case in ADMISSION_CASES + SCALED_WORKLOAD_CASES:
        q, k, v, g, beta, init = build_case(case)
        ratio = v.shape[2] // q.shape[2]
        qe, ke = q.repeat_interleave(ratio, 2), k.repeat_interleave(ratio, 2)
        ref_out, ref_state = torch_chunk_gated_delta_rule(
            qe, ke, v, g, beta, initial_state=init, output_final_state=True)
        rec_out, rec_state = torch_recurrent_gated_delta_rule(
            qe, ke, v, g, beta, initial_state=init, output_final_state=True)
        dbl_out, dbl_state = recurrent_double((q, k, v, g, beta), init)
        res_out, res_state = residual_forward((q, k, v, g, beta), init, rounded=False)
        wyr_out, wyr_state = wy_forward((q, k, v, g, beta), init, rounded=False)

        # the reference's own paths agree with each other
        assert oracle.rel_frobenius(res_out, dbl_out) < 1e-12 and oracle.rel_frobenius(res_state, dbl_state) < 1e-12
        assert oracle.rel_frobenius(wyr_out, dbl_out) < 1e-12 and oracle.rel_frobenius(wyr_state, dbl_state) < 1e-12
        assert oracle.rel_frobenius(ref_state, dbl_state) < 2e-5, case["name"]
        assert oracle.rel_frobenius(rec_state, dbl_state) < 2e-5, case["name"]

        # this repository's restatement agrees with the reference
        mine_out, mine_state = oracle.chunk_forward_fp32(q, k, v, g, beta, init, True)
        assert torch.equal(mine_out, ref_out) or oracle.max_abs(mine_out, ref_out) < 2e-2 * 2 ** -7, case["name"]
        assert oracle.rel_frobenius(mine_state, ref_state) < 1e-6, case["name"]
        r_out, r_state = oracle.recurrent_forward(q, k, v, g, beta, init)
        assert oracle.rel_frobenius(r_out, dbl_out) < 1e-13 and oracle.rel_frobenius(r_state, dbl_state) < 1e-13
        w_out, w_state = oracle.wy_chunk_forward(q, k, v, g, beta, init)
        assert oracle.rel_frobenius(w_out, dbl_out) < 1e-11 and oracle.rel_frobenius(w_state, dbl_state) < 1e-11

        name = case["name"]
        arrays[f"{name}.out_bf16"] = ref_out.view(torch.int16).numpy()
        arrays[f"{name}.state_f32"] = ref_state.numpy()
        arrays[f"{name}.state_f64_fro"] = np.array(dbl_state.norm().item())
        index[name] = dict(case=case, input_sha256=digest((q, k, v, g, beta, init)),
                           reference_functions=["actlize_la.reference.gdn_chunk_ref.torch_chunk_gated_delta_rule"],
                           fp32_vs_fp64_state_rel_frobenius=oracle.rel_frobenius(ref_state, dbl_state),
                           fp32_vs_fp64_out_rel_frobenius=oracle.rel_frobenius(ref_out.double(), dbl_out))
        print(f"{name:28s} ok  state relF(fp32 ref vs fp64)={index[name]['fp32_vs_fp64_state_rel_frobenius']:.2e}")
    # ---- the step before the forward: the reference's serving recurrence on raw projection inputs
    from serving_reference import gdn_reference
    from tests.cases import prestep_case
    mixed, a, b, a_log, dt_bias, hk, hv = prestep_case()
    ref_out, ref_state_vk, _, ref_key, ref_decay = gdn_reference(
        mixed, a, b, a_log, dt_bias, torch.zeros(hv, 128, 128), hk)
    q, k, v, g, beta = oracle.prepare_inputs_ref(mixed, a, b, a_log, dt_bias, hk, hv)
    assert (k.float() - ref_key).abs().max() <= 2 ** -8 * ref_key.abs().max()          # BF16 rounding of k only
    assert oracle.rel_frobenius(g.exp(), ref_decay) < 1e-6
    mine_out, mine_state = oracle.recurrent_forward(q[None], k[None], v[None], g[None], beta[None], None)
    assert oracle.max_abs(mine_out[0], ref_out.double()) < 2e-2
    assert oracle.rel_frobenius(mine_state[0].transpose(-1, -2), ref_state_vk.double()) < 1e-2   # ref state is V-by-K
    arrays["prestep.key_f32"] = ref_key.numpy()
    arrays["prestep.decay_f32"] = ref_decay.numpy()
    arrays["prestep.out_bf16"] = ref_out.view(torch.int16).numpy()
    print("prestep                      ok")

    np.savez_compressed(args.out, **arrays)
    args.out.with_suffix(".json").write_text(json.dumps(
        dict(schema=1, torch=torch.__version__, cases=index), indent=1, sort_keys=True) + "\n")
    print(f"wrote {args.out} ({args.out.stat().st_size/1e6:.2f} MB) with {len(index)} cases")


if __name__ == "__main__":
    main()
