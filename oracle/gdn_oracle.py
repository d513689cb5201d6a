"""CPU oracle for the chunked gated-delta-rule (GDN) forward.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module; it is the checker used by the
tests, the smoke entry and the CPU-baseline leg of the benchmark.

It restates, in plain torch CPU code, the algorithm of the reference project
(paths relative to the reference tree):

* ``chunk_forward_fp32``      follows actlize_la/reference/gdn_chunk_ref.py:20-100
  (FP32, chunk 64, all-chunk triangular solve, Python chunk loop) but takes the
  grouped-value heads natively instead of asking the caller to repeat q/k
  (the reference's callers do ``repeat_interleave``: tests/test_gdn_chunk.py:28-30).
* ``recurrent_forward``       follows actlize_la/reference/gdn_chunk_ref.py:103-147 and
  tests/wy_cpu.py:91-103 (token recurrence, any dtype; FP64 is the exact anchor).
* ``wy_chunk_forward``        follows tests/wy_cpu.py:44-88 (WY association, unrounded)
  and tests/residual_cpu.py:6-49; it also returns the per-chunk intermediates the
  device prepare kernel materialises (prefix, T, W, U, P) and accepts the reference's
  planted-bug switches so the negative controls can be reproduced.
* ``segment_transition``      is the affine state map of a token segment
  (``S_out = M @ S_in + b``), the composition rule of csrc/gdn_chunk/gdn_scan_stage2.cu:4-8.

Parity pin: ``tests/golden/make_golden.py`` imports the reference itself, checks these
restatements against it, and stores the reference's outputs as golden fixtures; the CPU
test-suite re-checks this file against those fixtures.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

CHUNK = 64
DIM = 128


# --------------------------------------------------------------------------- metrics
def max_abs(got, want):
    return (got.double() - want.double()).abs().max().item()


def rel_frobenius(got, want):
    want = want.double()
    return ((got.double() - want).norm() / want.norm().clamp_min(1e-30)).item()


def max_over_max(got, want):
    """The reference's 2 % criterion (tests/test_ppu_gdn_backend.py:42-47)."""
    got, want = got.double(), want.double()
    if not torch.isfinite(got).all():
        return float("inf")
    return ((got - want).abs().max() / (want.abs().max() + 1e-9)).item()


# --------------------------------------------------------------------------- helpers
def _expand_heads(x, hv):
    hk = x.shape[2]
    if hv % hk:
        raise ValueError("value heads must be a multiple of key heads")
    return x if hk == hv else x.repeat_interleave(hv // hk, dim=2)


# --------------------------------------------------------------------------- FP32 chunk form
def chunk_forward_fp32(q, k, v, g, beta, initial_state=None, output_final_state=True):
    """actlize_la/reference/gdn_chunk_ref.py:20-100 restated (FP32, chunk 64).

    q,k [B,T,Hk,128]; v [B,T,Hv,128]; g,beta [B,T,Hv]; state [B,Hv,128,128] (K by V).
    Returns (out in q.dtype [B,T,Hv,128], final FP32 state or None).
    """
    out_dtype = q.dtype
    b, t, _, d = k.shape
    hv = v.shape[2]
    q, k = _expand_heads(q, hv), _expand_heads(k, hv)
    q, k, v, beta, g = (x.transpose(1, 2).to(torch.float32).contiguous() for x in (q, k, v, beta, g))
    q = q * d ** -0.5
    pad = (-t) % CHUNK
    q, k, v = (F.pad(x, (0, 0, 0, pad)) for x in (q, k, v))
    beta, g = (F.pad(x, (0, pad)) for x in (beta, g))
    n = (t + pad) // CHUNK
    vb, kb = v * beta[..., None], k * beta[..., None]
    q, k, kb, vb = (x.reshape(b, hv, n, CHUNK, d) for x in (q, k, kb, vb))
    p = g.reshape(b, hv, n, CHUNK).cumsum(-1)
    upper = torch.ones(CHUNK, CHUNK, dtype=torch.bool).triu(1)
    pair = (p[..., :, None] - p[..., None, :]).masked_fill(upper, float("-inf")).exp()
    system = (kb @ k.transpose(-1, -2)) * pair          # unit-lower system incl. diagonal
    intra = (q @ k.transpose(-1, -2)) * pair
    kbg = kb * p.exp()[..., None]
    u = torch.linalg.solve_triangular(system, vb, upper=False, unitriangular=True)
    w = torch.linalg.solve_triangular(system, kbg, upper=False, unitriangular=True)
    state = (torch.zeros(b, hv, d, d) if initial_state is None
             else initial_state.to(torch.float32).clone())
    out = torch.zeros_like(u)
    qg = q * p.exp()[..., None]
    kr = k * (p[..., -1:] - p).exp()[..., None]
    gamma = p[..., -1].exp()[..., None, None]
    for i in range(n):
        new = u[:, :, i] - w[:, :, i] @ state
        out[:, :, i] = qg[:, :, i] @ state + intra[:, :, i] @ new
        state = state * gamma[:, :, i] + kr[:, :, i].transpose(-1, -2) @ new
    out = out.reshape(b, hv, -1, d)[:, :, :t].transpose(1, 2).contiguous().to(out_dtype)
    return out, (state if output_final_state else None)


# --------------------------------------------------------------------------- token recurrence
def recurrent_forward(q, k, v, g, beta, initial_state=None, output_final_state=True,
                      dtype=torch.float64):
    """gdn_chunk_ref.py:103-147 / tests/wy_cpu.py:91-103 restated; exact in FP64.

    Returns (out in ``dtype`` [B,T,Hv,128], final state in ``dtype`` or None).
    """
    b, t, _, d = k.shape
    hv = v.shape[2]
    q, k = _expand_heads(q, hv).to(dtype), _expand_heads(k, hv).to(dtype)
    v, g, beta = v.to(dtype), g.to(dtype), beta.to(dtype)
    h = (torch.zeros(b, hv, d, d, dtype=dtype) if initial_state is None
         else initial_state.to(dtype).clone())
    out = torch.empty(b, t, hv, d, dtype=dtype)
    scale = d ** -0.5
    for i in range(t):
        h = h * g[:, i].exp()[..., None, None]
        delta = (v[:, i] - (k[:, i, :, :, None] * h).sum(-2)) * beta[:, i, :, None]
        h = h + k[:, i, :, :, None] * delta[..., None, :]
        out[:, i] = (q[:, i, :, :, None] * h).sum(-2) * scale
    return out, (h if output_final_state else None)


# --------------------------------------------------------------------------- WY chunk form
def wy_chunk_forward(q, k, v, g, beta, initial_state=None, *, dtype=torch.float64,
                     plant=None, return_intermediates=False):
    """WY association per 64-token chunk (tests/wy_cpu.py:44-88, unrounded).

    ``plant`` reproduces the reference's negative controls
    (tests/test_ppu_wy_algebra.py, tests/test_sm90_algebra.py:55-76):
    reset, gva, inverse-sign, snapshot-after-update, causal, state-transpose,
    cross-chunk-prefix, wrong-log-base, query-scale-twice, gate-omitted,
    beta-outside-inverse, inverse-identity.
    Returns (out [B,T,Hv,128] dtype, state [B,Hv,128,128] dtype[, intermediates]).
    Intermediates (all [B,Hv,N,...]): prefix[64], T[64,64], W[64,128], U[64,128],
    P[64,64] (causal, decay-masked, already multiplied by 1/sqrt(128)).
    """
    b, t, hk, d = q.shape
    hv = v.shape[2]
    mapping = torch.arange(hv) // (hv // hk)
    if plant == "gva":
        mapping = (mapping + 1) % hk
    q, k = q[:, :, mapping], k[:, :, mapping]
    pad = (-t) % CHUNK
    q, k, v = (F.pad(x.transpose(1, 2).to(dtype), (0, 0, 0, pad)).reshape(b, hv, -1, CHUNK, d)
               for x in (q, k, v))
    g, beta = (F.pad(x.transpose(1, 2).to(dtype), (0, pad)).reshape(b, hv, -1, CHUNK)
               for x in (g, beta))
    n = q.shape[2]
    prefix = g.cumsum(-1)
    if plant == "cross-chunk-prefix":
        carry = torch.cumsum(prefix[..., -1], -1) - prefix[..., -1]
        prefix = prefix + carry[..., None]
    logbase = 1.0 if plant != "wrong-log-base" else math.log(2.0)
    strict = torch.ones(CHUNK, CHUNK, dtype=torch.bool).tril(-1)
    causal = torch.ones(CHUNK, CHUNK, dtype=torch.bool).tril()
    diff = (prefix[..., :, None] - prefix[..., None, :]) * logbase
    lower = torch.where(strict, (k @ k.transpose(-1, -2)) * beta[..., :, None]
                        * torch.where(strict, diff, 0).exp(), 0)
    if plant == "inverse-sign":
        lower = -lower
    eye = torch.eye(CHUNK, dtype=dtype)
    tmat = torch.linalg.solve_triangular(eye + lower, eye.expand_as(lower).contiguous(), upper=False)
    if plant == "inverse-identity":
        tmat = eye.expand_as(lower).contiguous()
    gam = (prefix * logbase).exp()
    if plant == "gate-omitted":
        gam = torch.ones_like(gam)
    if plant == "beta-outside-inverse":
        w = beta[..., :, None] * (tmat @ (k * gam[..., :, None]))
        u = beta[..., :, None] * (tmat @ v)
    else:
        w = tmat @ (k * (beta * gam)[..., :, None])
        u = tmat @ (v * beta[..., :, None])
    scale = d ** -0.5 if plant != "query-scale-twice" else 1.0 / d
    pmat = torch.where(causal, (q @ k.transpose(-1, -2))
                       * torch.where(causal, diff, 0).exp(), 0) * scale
    if plant == "causal":
        pmat = (q @ k.transpose(-1, -2)) * diff.exp() * scale
    if initial_state is None:
        state = torch.zeros(b, hv, d, d, dtype=dtype)
    else:
        state = initial_state.to(dtype).clone()
        if plant == "state-transpose":
            state = state.transpose(-1, -2).contiguous()
    out = torch.zeros_like(v)
    for c in range(n):
        valid = min(CHUNK, t - c * CHUNK)
        pc = prefix[:, :, c] * logbase
        if plant == "reset":
            state = torch.zeros_like(state)
        old = state
        new = u[:, :, c] - w[:, :, c] @ old
        new[..., valid:, :] = 0
        last = pc[..., valid - 1]
        nxt = (state * last.exp()[..., None, None]
               + k[:, :, c].transpose(-1, -2) @ (new * (last[..., None] - pc).exp()[..., :, None]))
        if plant == "snapshot-after-update":
            old = nxt
        out[:, :, c] = (q[:, :, c] @ old) * (gam[:, :, c][..., :, None] * scale) + pmat[:, :, c] @ new
        state = nxt
    out = out.reshape(b, hv, -1, d)[:, :, :t].transpose(1, 2).contiguous()
    if return_intermediates:
        return out, state, dict(prefix=prefix, T=tmat, W=w, U=u, P=pmat)
    return out, state


# --------------------------------------------------------------------------- affine transition
def segment_transition(k, g, beta, dtype=torch.float64):
    """Homogeneous part ``M`` of a segment's state map ``S_out = M @ S_in + b``.

    ``M`` is the final state of the recurrence started from ``S_in = I`` with ``v = 0``
    (the recurrence acts on every state column independently); ``b`` is the ordinary
    forward's final state from a zero initial state.  Composition of two consecutive
    segments is ``(M2 @ M1, M2 @ b1 + b2)`` (csrc/gdn_chunk/gdn_scan_stage2.cu:4-8).
    k [B,T,Hk,128], g,beta [B,T,Hv] -> M [B,Hv,128,128].
    """
    b, t, _, d = k.shape
    hv = g.shape[2]
    zero_v = torch.zeros(b, t, hv, d, dtype=dtype)
    eye = torch.eye(d, dtype=dtype).expand(b, hv, d, d).contiguous()
    _, m = recurrent_forward(k, k, zero_v, g, beta, initial_state=eye, dtype=dtype)
    return m


# --------------------------------------------------------------------------- neighbouring steps
def prepare_inputs_ref(mixed, a, b, a_log, dt_bias, key_heads, value_heads):
    """The step before the forward, as the reference's serving path defines it
    (tests/serving_reference.py:11-23; csrc/serving/prefill.cu:45-70, runtime.cuh:48-52):
    q,k = x / sqrt(sum x^2 + 1e-6) rounded to BF16 (no 1/sqrt(128): the forward applies it),
    v copied, g = -exp(A_log) * softplus(a + dt_bias) in FP32, beta = sigmoid(b) rounded to BF16."""
    n = mixed.shape[0]
    x = mixed.float()
    hk, hv = key_heads, value_heads
    q = x[:, :hk * 128].reshape(n, hk, 128)
    k = x[:, hk * 128:2 * hk * 128].reshape(n, hk, 128)
    v = mixed[:, 2 * hk * 128:].reshape(n, hv, 128)
    q = (q / torch.sqrt(q.square().sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    k = (k / torch.sqrt(k.square().sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    g = -a_log.float().exp() * F.softplus(a.float() + dt_bias.float(), threshold=20)
    beta = b.float().sigmoid().to(torch.bfloat16)
    return q, k, v.clone(), g, beta


def rmsnorm_gated_ref(y, z, weight, eps=1e-6):
    """tests/test_output_gate.py:12-16 restated: RMSNorm(y) * weight * silu(z), FP32 math, input dtype out."""
    yf = y.float()
    normed = yf * torch.rsqrt(yf.square().mean(-1, keepdim=True) + eps)
    return (normed * weight.float() * F.silu(z.float())).to(y.dtype)
