"""The CPU oracle against the golden fixtures produced from the reference itself.

Mirrors the reference's CPU algebra tier (tests/test_sm90_algebra.py:55-76,
tests/test_ppu_wy_algebra.py:12-55): chunked == recurrent in FP64, fixtures pinned by
input hash, planted bugs must be detected.
"""
import hashlib

import pytest
import torch

from oracle import gdn_oracle as oracle
from tests.cases import ALL_CASES, build_case

torch.set_num_threads(max(1, min(8, torch.get_num_threads())))


def _digest(tensors):
    h = hashlib.sha256()
    for t in tensors:
        if t is not None:
            h.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("case", ALL_CASES, ids=lambda c: c["name"])
def test_fp32_chunk_oracle_matches_reference_fixture(case, golden):
    inputs = build_case(case)
    out_ref, state_ref, meta = golden[case["name"]]
    assert _digest(inputs) == meta["input_sha256"], "seeded inputs differ from the fixture's"
    out, state = oracle.chunk_forward_fp32(*inputs, output_final_state=True)
    assert out.dtype == torch.bfloat16 and out.shape == out_ref.shape
    # same arithmetic as the reference: identical up to BF16 rounding of a last-bit difference
    assert oracle.max_abs(out, out_ref) <= 2e-2 * 2 ** -7
    assert oracle.rel_frobenius(out.float(), out_ref.float()) < 1e-4
    assert oracle.rel_frobenius(state, state_ref) < 1e-6


@pytest.mark.parametrize("case", ALL_CASES, ids=lambda c: c["name"])
def test_fp64_forms_agree_and_match_fixture(case, golden):
    inputs = build_case(case)
    out_ref, state_ref, _ = golden[case["name"]]
    r_out, r_state = oracle.recurrent_forward(*inputs)
    w_out, w_state = oracle.wy_chunk_forward(*inputs)
    assert oracle.rel_frobenius(w_out, r_out) < 1e-11
    assert oracle.rel_frobenius(w_state, r_state) < 1e-11
    # the FP32 reference result sits within FP32 noise of the exact answer
    assert oracle.rel_frobenius(state_ref, r_state) < 2e-5
    assert oracle.max_abs(out_ref.double(), r_out) < 2e-2


PLANTS = ["reset", "gva", "inverse-sign", "snapshot-after-update", "causal", "state-transpose",
          "cross-chunk-prefix", "wrong-log-base", "query-scale-twice", "gate-omitted",
          "beta-outside-inverse", "inverse-identity"]


@pytest.mark.parametrize("plant", PLANTS)
def test_planted_bugs_are_detected(plant):
    case = dict(name="neg", kind="admission", batch=1, length=129, key_heads=2, value_heads=4,
                gate=-0.1, fp32_gate=True, vary_gate=True, initial=True)
    q, k, v, g, beta, init = build_case(case)
    init = init * 20       # make the incoming state matter
    want_out, want_state = oracle.recurrent_forward(q, k, v, g, beta, init)
    got_out, got_state = oracle.wy_chunk_forward(q, k, v, g, beta, init, plant=plant)
    wrong = max(oracle.rel_frobenius(got_out, want_out), oracle.rel_frobenius(got_state, want_state))
    assert wrong > 1e-3, f"planted bug {plant} was not detected"


def test_intermediates_satisfy_their_definitions():
    case = dict(name="im", kind="admission", batch=1, length=100, key_heads=1, value_heads=2,
                gate=-0.5, fp32_gate=True, vary_gate=True, initial=False)
    q, k, v, g, beta, _ = build_case(case)
    _, _, im = oracle.wy_chunk_forward(q, k, v, g, beta, return_intermediates=True)
    t = im["T"]
    eye = torch.eye(64, dtype=torch.float64)
    assert torch.allclose(t.triu(1), torch.zeros_like(t))
    assert torch.allclose(torch.diagonal(t, dim1=-2, dim2=-1), torch.ones(1, 2, 2, 64, dtype=torch.float64))
    # T (I + A) = I  with A rebuilt from its definition
    kk = k.double().transpose(1, 2)[:, [0, 0]]
    kk = torch.nn.functional.pad(kk, (0, 0, 0, 28)).reshape(1, 2, 2, 64, 128)
    p = im["prefix"]
    bb = torch.nn.functional.pad(beta.double().transpose(1, 2), (0, 28)).reshape(1, 2, 2, 64)
    a = (kk @ kk.transpose(-1, -2)) * bb[..., :, None] * (p[..., :, None] - p[..., None, :]).exp()
    a = a.tril(-1)
    assert (t @ (eye + a) - eye).abs().max() < 1e-12


def test_segment_chaining_and_affine_transition():
    """final -> initial chaining equals the unsplit run; the affine map reproduces it too."""
    case = dict(name="seg", kind="admission", batch=1, length=256, key_heads=1, value_heads=2,
                gate=-0.05, fp32_gate=True, vary_gate=True, initial=True)
    q, k, v, g, beta, init = build_case(case)
    full_out, full_state = oracle.recurrent_forward(q, k, v, g, beta, init)
    cut = 128
    head = [x[:, :cut] for x in (q, k, v, g, beta)]
    tail = [x[:, cut:] for x in (q, k, v, g, beta)]
    o1, s1 = oracle.recurrent_forward(*head, init)
    o2, s2 = oracle.recurrent_forward(*tail, s1)
    assert oracle.rel_frobenius(torch.cat([o1, o2], 1), full_out) < 1e-13
    assert oracle.rel_frobenius(s2, full_state) < 1e-13
    m = oracle.segment_transition(tail[1], tail[3], tail[4])
    _, b_tail = oracle.recurrent_forward(*tail, None)
    assert oracle.rel_frobenius(m @ s1 + b_tail, full_state) < 1e-12


def test_prestep_oracle_matches_reference_fixture():
    """Q/K normalisation, gate activation and beta against the reference's serving recurrence."""
    import numpy as np
    from pathlib import Path
    from tests.cases import prestep_case
    arrays = np.load(Path(__file__).with_name("golden") / "golden_cases.npz")
    mixed, a, b, a_log, dt_bias, hk, hv = prestep_case()
    q, k, v, g, beta = oracle.prepare_inputs_ref(mixed, a, b, a_log, dt_bias, hk, hv)
    key = torch.from_numpy(arrays["prestep.key_f32"])
    assert (k.float() - key).abs().max() <= 2 ** -8 * key.abs().max()
    assert oracle.rel_frobenius(g.exp(), torch.from_numpy(arrays["prestep.decay_f32"])) < 1e-6
    out, _ = oracle.recurrent_forward(q[None], k[None], v[None], g[None], beta[None], None)
    ref_out = torch.from_numpy(arrays["prestep.out_bf16"].copy()).view(torch.bfloat16)
    assert oracle.max_abs(out[0], ref_out.double()) < 2e-2
