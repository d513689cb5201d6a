"""Seeded parity cases shared by the golden-fixture generator and the test-suite.

``ADMISSION_CASES`` follows the reference's device admission denominator
(tests/run_sm90_hopper_cases.py:14-29: lengths 1..257 around the chunk boundaries,
grouped value heads, both gate dtypes, with/without initial state), with inputs drawn
the way its fixture does (tests/test_ppu_gdn_backend.py:22-32, tools/run_sm90_gdn.py:70-77:
0.05*N(0,1) BF16 q/k/v, constant or per-token varied natural-log gate in [-1,0],
beta = sigmoid(U(0,1)), optional 0.005*N(0,1) initial state).
``SCALED_WORKLOAD_CASES`` uses the benchmark distributions at sizes a CPU finishes in
seconds.
"""
from __future__ import annotations

import torch

from actlizela_b200.workloads import WORKLOADS, make_inputs


def _case(name, batch, length, key_heads, value_heads, gate, *flags):
    return dict(name=name, kind="admission", batch=batch, length=length, key_heads=key_heads,
                value_heads=value_heads, gate=gate, fp32_gate="fp32" in flags,
                vary_gate="vary" in flags, initial="initial" in flags)


ADMISSION_CASES = [
    _case("full64", 1, 64, 1, 1, -0.1),
    _case("fp32-no-initial", 1, 65, 1, 2, -0.1, "fp32", "vary"),
    _case("tail1-initial", 2, 1, 1, 2, -0.1, "initial", "fp32", "vary"),
    _case("tail31-gva", 1, 31, 2, 6, -0.1, "vary"),
    _case("half32-initial", 1, 32, 1, 2, -0.1, "initial"),
    _case("tail63-distinct", 1, 63, 2, 4, -0.1, "vary"),
    _case("tail65-initial", 2, 65, 1, 2, -0.1, "initial", "fp32", "vary"),
    _case("tail127", 1, 127, 2, 4, -0.1, "vary"),
    _case("full128-strong", 1, 128, 1, 1, -1.0),
    _case("tail129-zero-decay", 1, 129, 2, 4, 0.0, "initial", "fp32"),
    _case("tail257-wrap", 1, 257, 2, 4, -1.0, "vary"),
]


def _scaled(name, base, **size):
    return dict(name=name, kind="workload", base=base, **size)


SCALED_WORKLOAD_CASES = [
    _scaled("cfg0-scaled", "cfg0", batch=1, length=320, key_heads=2, value_heads=4),
    _scaled("cfg1-scaled", "cfg1", batch=1, length=256, key_heads=1, value_heads=3),
    _scaled("cfg2-scaled", "cfg2", batch=2, length=192, key_heads=1, value_heads=2),
    _scaled("cfg3-scaled", "cfg3", batch=1, length=184, key_heads=1, value_heads=4),
]

ALL_CASES = ADMISSION_CASES + SCALED_WORKLOAD_CASES


def build_case(case):
    """Returns CPU tensors (q, k, v, g, beta, initial_state_or_None)."""
    if case["kind"] == "workload":
        w = WORKLOADS[case["base"]].sliced(batch=case["batch"], length=case["length"],
                                           key_heads=case["key_heads"], value_heads=case["value_heads"])
        return make_inputs(w)
    b, t, hk, hv = case["batch"], case["length"], case["key_heads"], case["value_heads"]
    gen = torch.Generator().manual_seed(0x6A09E667)
    q, k, v = ((0.05 * torch.randn(b, t, h, 128, generator=gen)).to(torch.bfloat16)
               for h in (hk, hk, hv))
    gate_dtype = torch.float32 if case["fp32_gate"] else torch.bfloat16
    g = torch.full((b, t, hv), case["gate"], dtype=gate_dtype)
    beta = torch.sigmoid(torch.rand(b, t, hv, generator=gen)).to(torch.bfloat16)
    if case["vary_gate"]:
        spread = torch.rand(b, t, hv, generator=torch.Generator().manual_seed(101))
        g = (case["gate"] * (0.25 + 0.75 * spread)).to(gate_dtype)
    initial = None
    if case["initial"]:
        initial = 0.005 * torch.randn(b, hv, 128, 128, generator=torch.Generator().manual_seed(17))
    return q, k, v, g, beta, initial


def prestep_case():
    """Raw projection inputs of the step before the forward (shapes of tests/serving_reference.py:7-23)."""
    gen = torch.Generator().manual_seed(4711)
    hk, hv, n = 2, 4, 70
    mixed = torch.randn(n, (2 * hk + hv) * 128, generator=gen).to(torch.bfloat16)
    a = torch.randn(n, hv, generator=gen).to(torch.bfloat16)
    b = torch.randn(n, hv, generator=gen).to(torch.bfloat16)
    a_log = torch.randn(hv, generator=gen) * 0.5
    dt_bias = torch.randn(hv, generator=gen)
    return mixed, a, b, a_log, dt_bias, hk, hv
