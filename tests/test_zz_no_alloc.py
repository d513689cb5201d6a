"""The allocation-free forward entry point against the ordinary one.

Some callers of this library cannot allocate device memory: a plugin inside a host framework that
owns every allocation, or a loop that must not call cudaMalloc.  For them the library offers
`actlize_la_sm100_forward_static_scratch`, which keeps the workspace in an array built into the
library.  This test calls it through the C ABI twice in a row (the array is shared and keeps the
previous call's contents, so the second call runs on a dirty array) and compares both results with
the ordinary `forward_prepared` path.  It also checks that an oversized geometry is refused.
The file name sorts last so that a run stopping at the first failure has already run everything else.
"""
import pytest
import torch

from oracle import gdn_oracle as oracle
from tests.cases import build_case

pytestmark = pytest.mark.gpu

MAX_BLOCKS = 64
TOO_SMALL = -2


def _call(lib, tensors, config=1):
    q, k, v, g, beta, init = tensors
    b, t, hk, _ = q.shape
    hv = v.shape[2]
    out = torch.empty_like(v)
    final = torch.empty(b, hv, 128, 128, device=q.device)
    rc = lib.actlize_la_sm100_forward_static_scratch(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
        init.data_ptr() if init is not None else None, out.data_ptr(), final.data_ptr(),
        b, t, hk, hv, int(g.dtype == torch.float32), config, torch.cuda.current_stream().cuda_stream)
    return rc, out, final


def test_static_scratch_entry_matches_the_ordinary_entry_twice(native_library):
    from actlizela_b200.sm100 import Sm100Forward
    lib = native_library.lib
    first = dict(name="na1", kind="admission", batch=1, length=300, key_heads=1, value_heads=2,
                 gate=-0.1, fp32_gate=True, vary_gate=True, initial=True)
    second = dict(name="na2", kind="admission", batch=2, length=129, key_heads=2, value_heads=4,
                  gate=-1.0, fp32_gate=False, vary_gate=True, initial=False)
    torch.cuda.set_device(0)
    reference = Sm100Forward(native_library)
    for case in (first, second):            # two calls in a row on the shared array
        tensors = [x.cuda() if x is not None else None for x in build_case(case)]
        blocks = case["batch"] * case["value_heads"] * ((case["length"] + 63) // 64)
        assert blocks <= MAX_BLOCKS
        rc, out, final = _call(lib, tensors)
        assert rc == 0
        want_out, want_final = reference(*tensors, True, configuration="umma")
        torch.cuda.synchronize()
        assert oracle.max_abs(out.float(), want_out.float()) <= 2e-2
        assert oracle.rel_frobenius(out.float().cpu(), want_out.float().cpu()) <= 1e-2
        assert oracle.rel_frobenius(final.cpu(), want_final.cpu()) <= 1e-3
        assert torch.equal(out, want_out) and torch.equal(final, want_final)


def test_static_scratch_entry_refuses_an_oversized_geometry(native_library):
    lib = native_library.lib
    case = dict(name="na3", kind="admission", batch=1, length=64 * 33, key_heads=1, value_heads=2,
                gate=-0.1, fp32_gate=True, vary_gate=False, initial=False)     # 66 blocks > 64
    tensors = [x.cuda() if x is not None else None for x in build_case(case)]
    rc, out, _ = _call(lib, tensors)
    assert rc == TOO_SMALL
