"""Device parity of the steps either side of the forward and of the packed-sequence wrapper."""
import pytest
import torch

from oracle import gdn_oracle as oracle
from tests.cases import prestep_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _library(native_library):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device; there is no CPU fallback to test")


def test_prepare_inputs_matches_oracle():
    from actlizela_b200 import gdn_prepare_inputs
    mixed, a, b, a_log, dt_bias, hk, hv = prestep_case()
    want = oracle.prepare_inputs_ref(mixed, a, b, a_log, dt_bias, hk, hv)
    got = gdn_prepare_inputs(mixed.cuda(), a.cuda(), b.cuda(), a_log.cuda(), dt_bias.cuda(), hk, hv)
    for name, x, y in zip(("q", "k", "v", "g", "beta"), got, want):
        x, y = x.float().cpu(), y.float()
        # identical up to one BF16 ulp where rsqrt / exp differ in the last FP32 bit
        assert (x - y).abs().max() <= 2 ** -7 * y.abs().max() + 1e-6, name
        assert oracle.rel_frobenius(x, y) < 1e-3, name
    assert torch.equal(got[2].cpu(), want[2])          # v is a copy


@pytest.mark.parametrize("batch,hk,hv,gate", [(1, 1, 1, torch.float32), (3, 2, 8, torch.bfloat16), (16, 16, 32, torch.float32)])
def test_decode_step_matches_recurrence(batch, hk, hv, gate):
    from actlizela_b200 import gdn_decode_step
    gen = torch.Generator().manual_seed(batch * 100 + hv)
    norm = torch.nn.functional.normalize
    q = norm(torch.randn(batch, hk, 128, generator=gen), dim=-1).to(torch.bfloat16)
    k = norm(torch.randn(batch, hk, 128, generator=gen), dim=-1).to(torch.bfloat16)
    v = torch.randn(batch, hv, 128, generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(batch, hv, generator=gen) + 2).to(gate)
    beta = torch.sigmoid(torch.randn(batch, hv, generator=gen)).to(torch.bfloat16)
    state = torch.randn(batch, hv, 128, 128, generator=gen) * 0.3
    dev_state = state.cuda()
    for step in range(3):                      # three tokens in a row on the same state
        want_out, want_state = oracle.recurrent_forward(q[:, None], k[:, None], v[:, None], g[:, None],
                                                        beta[:, None], state, dtype=torch.float64)
        out = gdn_decode_step(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), dev_state)
        assert oracle.max_abs(out.float().cpu(), want_out[:, 0]) <= 2e-2
        assert oracle.rel_frobenius(out.float().cpu(), want_out[:, 0]) <= 1e-2
        assert oracle.rel_frobenius(dev_state.cpu(), want_state) <= 1e-5
        state = want_state.float()
        dev_state.copy_(state)


def test_decode_step_equals_forward_with_one_token():
    from actlizela_b200 import gdn_decode_step, gdn_forward
    gen = torch.Generator().manual_seed(11)
    q = torch.nn.functional.normalize(torch.randn(2, 1, 2, 128, generator=gen), dim=-1).to(torch.bfloat16).cuda()
    k = torch.nn.functional.normalize(torch.randn(2, 1, 2, 128, generator=gen), dim=-1).to(torch.bfloat16).cuda()
    v = torch.randn(2, 1, 4, 128, generator=gen).to(torch.bfloat16).cuda()
    g = (-torch.rand(2, 1, 4, generator=gen)).cuda()
    beta = torch.rand(2, 1, 4, generator=gen).to(torch.bfloat16).cuda()
    state = (torch.randn(2, 4, 128, 128, generator=gen) * 0.2).cuda()
    out_f, state_f = gdn_forward(q, k, v, g, beta, state, True)
    mine = state.clone()
    out_d = gdn_decode_step(q[:, 0].contiguous(), k[:, 0].contiguous(), v[:, 0].contiguous(),
                            g[:, 0].contiguous(), beta[:, 0].contiguous(), mine)
    assert oracle.max_abs(out_d.float(), out_f[:, 0].float()) <= 2e-2
    assert oracle.rel_frobenius(mine.cpu(), state_f.cpu()) <= 1e-3


def test_rmsnorm_gated_matches_oracle():
    from actlizela_b200 import rmsnorm_gated
    gen = torch.Generator().manual_seed(3)
    y = torch.randn(1000, 32, 128, generator=gen).to(torch.bfloat16)
    z = torch.randn(1000, 32, 128, generator=gen).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(128, generator=gen)).to(torch.bfloat16)
    want = oracle.rmsnorm_gated_ref(y, z, w)
    got = rmsnorm_gated(y.cuda(), z.cuda(), w.cuda()).cpu()
    assert oracle.rel_frobenius(got.float(), want.float()) < 1e-2       # the reference's own criterion
    assert (got.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()


def test_varlen_matches_per_sequence_oracle():
    from actlizela_b200 import gdn_forward_varlen
    from actlizela_b200.workloads import WORKLOADS, make_inputs
    lengths = [130, 1, 64, 0, 257, 63]
    bounds = [0]
    for n in lengths:
        bounds.append(bounds[-1] + n)
    w = WORKLOADS["cfg3"].sliced(batch=1, length=bounds[-1], key_heads=2, value_heads=4, initial=None)
    q, k, v, g, beta, _ = make_inputs(w)
    init = 0.1 * torch.randn(len(lengths), 4, 128, 128, generator=torch.Generator().manual_seed(5))
    out, finals = gdn_forward_varlen(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), bounds, init.cuda(), True)
    for i, (t0, t1) in enumerate(zip(bounds, bounds[1:])):
        if t1 == t0:
            assert torch.equal(finals[i].cpu(), init[i])
            continue
        want_out, want_state = oracle.chunk_forward_fp32(q[:, t0:t1], k[:, t0:t1], v[:, t0:t1], g[:, t0:t1],
                                                         beta[:, t0:t1], init[i:i + 1], True)
        assert oracle.max_abs(out[:, t0:t1].float().cpu(), want_out.float()) <= 2e-2
        assert oracle.rel_frobenius(out[:, t0:t1].float().cpu(), want_out.float()) <= 1e-2
        assert oracle.rel_frobenius(finals[i:i + 1].cpu(), want_state) <= 1e-3


@pytest.mark.parametrize("lengths", [[130, 1, 64, 0, 257, 63], [5], [64, 64], [0, 200, 0], [1] * 9, [700, 3, 129]])
def test_native_varlen_equals_the_per_sequence_forward_bitwise(lengths):
    """One prepare and one walk launch for all sequences give the bits of N fixed-shape forwards: the rows behind a
    ragged sequence end (the next sequence's tokens) only ever meet exact zeros."""
    from actlizela_b200 import gdn_forward_varlen
    from actlizela_b200.workloads import WORKLOADS, make_inputs
    bounds = [0]
    for n in lengths:
        bounds.append(bounds[-1] + n)
    w = WORKLOADS["cfg1"].sliced(batch=1, length=bounds[-1], key_heads=2, value_heads=6, initial=None)   # group of 3
    q, k, v, g, beta, _ = [x.cuda() if x is not None else None for x in make_inputs(w)]
    init = (0.1 * torch.randn(len(lengths), 6, 128, 128, generator=torch.Generator().manual_seed(7))).cuda()
    for initial in (init, None):
        out, finals = gdn_forward_varlen(q, k, v, g, beta, bounds, initial, True)
        ref_out, ref_finals = gdn_forward_varlen(q, k, v, g, beta, bounds, initial, True, per_sequence=True,
                                                 algorithm="wy_sm100", backend="cuda_sm100", configuration="umma")
        torch.cuda.synchronize()
        assert torch.equal(out, ref_out)
        assert torch.equal(finals, ref_finals)
        out_only, none = gdn_forward_varlen(q, k, v, g, beta, bounds, initial, False)
        assert none is None and torch.equal(out_only, out)
        # the same offsets as an int32 device tensor: nothing is read on the host, the grids cover an upper bound
        on_device = torch.tensor(bounds, dtype=torch.int32, device="cuda")
        dev_out, dev_finals = gdn_forward_varlen(q, k, v, g, beta, on_device, initial, True)
        assert torch.equal(dev_out, out) and torch.equal(dev_finals, finals)


def test_native_varlen_rejects_bad_offsets(native_library):
    from actlizela_b200 import gdn_forward_varlen
    from actlizela_b200.workloads import WORKLOADS, make_inputs
    w = WORKLOADS["cfg3"].sliced(batch=1, length=100, key_heads=1, value_heads=2, initial=None)
    q, k, v, g, beta, _ = [x.cuda() if x is not None else None for x in make_inputs(w)]
    for bad in ([0, 50], [1, 100], [0, 60, 40, 100], [0]):
        with pytest.raises(ValueError):
            gdn_forward_varlen(q, k, v, g, beta, bad)
    # the C entry checks on its own as well
    import ctypes
    lib = native_library.lib
    nbytes = lib.actlize_la_sm100_varlen_workspace_bytes(100, 2, 1, 2)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.empty_like(v)
    offsets = (ctypes.c_int * 3)(0, 70, 60)
    rc = lib.actlize_la_sm100_forward_varlen(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), None,
                                             out.data_ptr(), None, ws.data_ptr(), nbytes, offsets, 2, 1, 2, 1,
                                             torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert lib.actlize_la_sm100_varlen_workspace_bytes(0, 1, 1, 2) < 0


def test_verify_and_commit_steps():
    """Verify runs W draft tokens without touching the state; committing all of them equals W decode steps bit for
    bit, committing a prefix equals the oracle recurrence over that prefix."""
    from actlizela_b200 import gdn_commit_step, gdn_decode_step, gdn_verify_step
    gen = torch.Generator().manual_seed(11)
    b, w, hk, hv = 3, 5, 2, 6
    q = torch.nn.functional.normalize(torch.randn(b, w, hk, 128, generator=gen), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(b, w, hk, 128, generator=gen), dim=-1).to(torch.bfloat16)
    v = torch.randn(b, w, hv, 128, generator=gen).to(torch.bfloat16)
    g = -torch.rand(b, w, hv, generator=gen)
    beta = torch.rand(b, w, hv, generator=gen).to(torch.bfloat16)
    state0 = 0.1 * torch.randn(b, hv, 128, 128, generator=gen)
    dev = [x.cuda() for x in (q, k, v, g, beta)]
    state = state0.cuda()
    out, delta = gdn_verify_step(*dev, state)
    assert torch.equal(state.cpu(), state0)                                   # read only
    want_out, _ = oracle.recurrent_forward(q, k, v, g, beta, state0)
    assert oracle.max_abs(out.float().cpu(), want_out.float()) < 2e-2
    # W decode steps on a copy
    stepped = state0.cuda()
    for t in range(w):
        o = gdn_decode_step(dev[0][:, t].contiguous(), dev[1][:, t].contiguous(), dev[2][:, t].contiguous(),
                            dev[3][:, t].contiguous(), dev[4][:, t].contiguous(), stepped)
        assert torch.equal(o, out[:, t])
    full = gdn_commit_step(dev[1], dev[3], delta, torch.full((b,), w, dtype=torch.int32, device="cuda"), state0.cuda())
    assert torch.equal(full, stepped)
    # accepted prefixes of different lengths, including none
    counts = torch.tensor([0, 2, 5], dtype=torch.int32)
    partial = gdn_commit_step(dev[1], dev[3], delta, counts.cuda(), state0.cuda()).cpu()
    for i, n in enumerate(counts.tolist()):
        if n == 0:
            assert torch.equal(partial[i], state0[i])
            continue
        _, want = oracle.recurrent_forward(q[i:i + 1, :n], k[i:i + 1, :n], v[i:i + 1, :n], g[i:i + 1, :n],
                                           beta[i:i + 1, :n], state0[i:i + 1])
        assert oracle.rel_frobenius(partial[i:i + 1], want) < 1e-5
    with pytest.raises(ValueError):
        gdn_commit_step(dev[1], dev[3], delta, counts.cuda().long(), state)


@pytest.mark.parametrize("shape", [(1, 300, 2, 4), (3, 200, 2, 6), (2, 64, 1, 1), (1, 2048, 16, 32)])
def test_forward_on_projections_equals_prepare_then_forward(shape):
    """Normalisation and gate activation inside the prepare kernel give the bits of the separate input-preparation
    kernel followed by the forward (batch tails read the next element's rows, which only meet exact zeros)."""
    from actlizela_b200 import gdn_forward, gdn_forward_projections, gdn_prepare_inputs
    bsz, t, hk, hv = shape
    gen = torch.Generator().manual_seed(21 + t)
    mixed = torch.randn(bsz, t, (2 * hk + hv) * 128, generator=gen).to(torch.bfloat16).cuda()
    a = torch.randn(bsz, t, hv, generator=gen).to(torch.bfloat16).cuda()
    b = torch.randn(bsz, t, hv, generator=gen).to(torch.bfloat16).cuda()
    a_log = (0.5 * torch.randn(hv, generator=gen)).cuda()
    dt_bias = (0.5 * torch.randn(hv, generator=gen)).cuda()
    init = (0.1 * torch.randn(bsz, hv, 128, 128, generator=gen)).cuda()
    q, k, v, g, beta = gdn_prepare_inputs(mixed.view(bsz * t, -1), a.view(bsz * t, hv), b.view(bsz * t, hv), a_log,
                                          dt_bias, hk, hv)
    view = lambda x, h: x.view(bsz, t, h, 128)
    for initial in (init, None):
        want_out, want_state = gdn_forward(view(q, hk), view(k, hk), view(v, hv), g.view(bsz, t, hv),
                                           beta.view(bsz, t, hv), initial, True)
        out, state = gdn_forward_projections(mixed, a, b, a_log, dt_bias, hk, hv, initial, True)
        torch.cuda.synchronize()
        assert torch.equal(out, want_out)
        assert torch.equal(state, want_state)
    out_only, none = gdn_forward_projections(mixed, a, b, a_log, dt_bias, hk, hv, None, False)
    assert none is None and torch.equal(out_only, out)


@pytest.mark.parametrize("m,k,n", [(512, 4096, 2560), (2048, 4096, 2560), (37, 4096, 2560), (100, 128, 64),
                                   (129, 72, 136), (8192, 4096, 2560)])
def test_out_proj_gemm_matches_fp32_matmul(m, k, n):
    """The reference's shapes (tests/test_output_gate.py:31-40) plus ragged tiles in every dimension; the
    comparison is the reference's own (FP32 matmul of the BF16 operands, rounded to BF16, 1 % of the largest
    entry) and a tighter one that only allows the final BF16 rounding and FP32 summation order."""
    from actlizela_b200 import out_proj_gemm
    gen = torch.Generator().manual_seed(m + k + n)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16).cuda()
    w = torch.randn(n, k, generator=gen).to(torch.bfloat16).cuda()
    want = a.float() @ w.float().t()                                   # plain PyTorch FP32 reference of the same op
    got = out_proj_gemm(a, w)
    torch.cuda.synchronize()
    assert got.shape == (m, n) and got.dtype == torch.bfloat16
    rel = (got.float() - want.to(torch.bfloat16).float()).abs().max().item() / want.abs().max().item()
    assert rel < 1e-2, rel
    # BF16 rounding of the result (2^-8 relative) plus FP32 accumulation noise
    assert ((got.float() - want).abs() <= 2 ** -7 * want.abs() + 1e-3 * k ** 0.5).all()


def test_rmsnorm_gated_then_out_proj_shape_chain():
    """[T*32,128] -> gated RMSNorm -> reshape [T,4096] -> out_proj [T,2560] (tests/test_output_gate.py:55-65)."""
    from actlizela_b200 import out_proj_gemm, rmsnorm_gated
    gen = torch.Generator().manual_seed(3)
    t = 64
    y = torch.randn(t * 32, 128, generator=gen).to(torch.bfloat16).cuda()
    z = torch.randn(t * 32, 128, generator=gen).to(torch.bfloat16).cuda()
    weight = torch.randn(128, generator=gen).to(torch.bfloat16).cuda()
    w = (torch.randn(2560, 4096, generator=gen) / 64).to(torch.bfloat16).cuda()
    gated = rmsnorm_gated(y, z, weight).reshape(t, 32 * 128)
    out = out_proj_gemm(gated, w)
    want = gated.float() @ w.float().t()
    assert out.shape == (t, 2560)
    assert oracle.rel_frobenius(out.float().cpu(), want.cpu()) < 5e-3
