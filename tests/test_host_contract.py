"""Host-side contract: routing, policy, catalog, loader identity and the exported C ABI.

Follows the reference's host tier (tests/test_gdn_route.py:17-117, tests/test_sm90_auto.py,
tests/test_backend_boundaries.py): tensors are duck-typed metadata objects whose data access
raises, native calls are mocked, nothing needs a GPU.
"""
import ctypes
import json
import re
from pathlib import Path
from types import SimpleNamespace
from unittest import mock

import pytest
import torch

import actlizela_b200
from actlizela_b200 import _library, device, gdn_interface, gdn_route, sm100, sm100_policy
from actlizela_b200.backends import registry

ROOT = Path(__file__).resolve().parents[1]


class Meta:
    """Tensor metadata only; touching data fails the test."""

    def __init__(self, shape, dtype=torch.bfloat16, dev="cuda:0"):
        self.shape, self.dtype, self.device = torch.Size(shape), dtype, torch.device(dev)
        self.ndim = len(shape)

    def stride(self):
        return tuple(torch.empty(self.shape, device="meta").stride())

    def cpu(self):
        raise AssertionError("route inspection must not read tensor data")

    data_ptr = cpu


B200 = device.DeviceProfile("NVIDIA B200", 148, (10, 0))
H800 = device.DeviceProfile("NVIDIA H800", 114, (9, 0))


def _args(b=1, t=8192, hk=16, hv=32):
    return (Meta((b, t, hk, 128)), Meta((b, t, hk, 128)), Meta((b, t, hv, 128)),
            Meta((b, t, hv), torch.float32), Meta((b, t, hv)))


def test_catalog_semantics():
    inv = actlizela_b200.backend_inventory()
    inv["targets"].clear()
    assert "cuda_sm100" in registry.backend_inventory()["targets"]
    with pytest.raises(ValueError):
        registry.require_backend("cuda_sm90")
    with pytest.raises(ValueError):
        registry.require_implementation("fused_sm90", "cuda_sm100")
    impl = registry.require_implementation("wy_sm100", "cuda_sm100")
    assert impl["final_state_dtype"] == "fp32" and impl["initial_state"] is True
    assert set(impl["gate_dtypes"]) == {"bf16", "fp32"}


def test_policy_table_is_well_formed_and_exact_match():
    data = sm100_policy.policy()
    assert data["device"]["capability"] == [10, 0] and data["head_dimensions"] == [128, 128]
    sel = sm100_policy.select((1, 8192, 16, 32, 128, 128), B200)
    assert sel.basis == "b200-measured-shape" and sel.configuration in data["configurations"]
    assert sm100_policy.select((3, 777, 2, 4, 128, 128), B200).basis == "unmeasured-shape-default"
    other = device.DeviceProfile("NVIDIA B100", 132, (10, 0))
    assert sm100_policy.select((1, 8192, 16, 32, 128, 128), other).basis == "unmeasured-device-default"
    configured = device.get_device_profile(mode="perfmodel", backend="cuda_sm100", sm_count=20)
    assert sm100_policy.select((1, 64, 1, 1, 128, 128), configured).basis == "perfmodel-unmeasured-default"
    with pytest.raises(ValueError):
        sm100_policy.select((1, 64, 3, 4, 128, 128), B200)        # Hv % Hk != 0
    with pytest.raises(ValueError):
        sm100_policy.select((1, 64, 1, 1, 64, 128), B200)         # K != 128
    with pytest.raises(ValueError):
        sm100_policy.select((1, 64, 1, 1, 128, 128), H800)        # another target


def test_policy_rejects_duplicate_rows(tmp_path, monkeypatch):
    data = json.loads(sm100_policy.POLICY_FILE.read_text())
    data["rows"].append(dict(data["rows"][0]))
    bad = tmp_path / "policy.json"
    bad.write_text(json.dumps(data))
    monkeypatch.setattr(sm100_policy, "POLICY_FILE", bad)
    sm100_policy.policy.cache_clear()
    try:
        with pytest.raises(ValueError):
            sm100_policy.policy()
    finally:
        monkeypatch.undo()
        sm100_policy.policy.cache_clear()


def test_auto_route_on_b200_and_no_fallback_elsewhere():
    q = Meta((1, 64, 1, 128))
    with mock.patch.object(sm100_policy, "device_profile", return_value=B200):
        route = gdn_interface._resolve_forward(q)
    assert (route["backend"], route["algorithm"], route["selected"]) == ("cuda_sm100", "wy_sm100", "auto")
    with mock.patch.object(sm100_policy, "device_profile", return_value=H800):
        with pytest.raises(ValueError):
            gdn_interface._resolve_forward(q)
    with pytest.raises(ValueError):
        gdn_interface._resolve_forward(Meta((1, 64, 1, 128), dev="cpu"))


def test_option_validation_matches_reference_rules():
    q = Meta((1, 64, 1, 128))
    with mock.patch.object(sm100_policy, "device_profile", return_value=B200):
        with pytest.raises(ValueError):
            gdn_interface._resolve_forward(q, configuration="umma")          # auto owns selection
        with pytest.raises(ValueError):
            gdn_interface._resolve_forward(q, delivery="scalar")
        with pytest.raises(ValueError):
            gdn_interface._resolve_forward(q, sm_count=20)                   # needs perfmodel
        with pytest.raises(ValueError):
            gdn_interface._resolve_forward(q, mode="perfmodel", sm_count=20)  # needs a backend
        with pytest.raises(ValueError):
            gdn_interface._resolve_forward(q, algorithm="wy_sm100")          # explicit needs backend
        with pytest.raises(ValueError):
            gdn_interface._resolve_forward(q, algorithm="original", backend="cuda_sm100")
    route = gdn_interface._resolve_forward(q, algorithm="wy_sm100", backend="cuda_sm100",
                                           configuration="simt")
    assert route["configuration"] == "simt"


def test_gdn_forward_passes_tensors_through_untouched():
    args = _args(1, 64, 1, 2)
    fake = mock.Mock(return_value=("out", None))
    with mock.patch.object(sm100_policy, "device_profile", return_value=B200), \
            mock.patch.object(sm100, "gdn_chunk_sm100", fake):
        result = actlizela_b200.gdn_forward(*args, None, False)
    assert result == ("out", None)
    called = fake.call_args
    assert all(a is b for a, b in zip(called.args, args))
    assert called.kwargs["backend"] == "cuda_sm100" and called.kwargs["output_final_state"] is False


def test_route_info_reads_metadata_only_and_does_not_launch():
    args = _args()
    with mock.patch.object(sm100_policy, "device_profile", return_value=B200):
        info = gdn_route.get_gdn_route_info(*args, load_binary=False)
    assert info["backend"] == "cuda_sm100" and info["device_execution"] == "NOT_RUN"
    assert info["native_entry"] == "actlize_la_sm100_forward_prepared"
    assert info["native_status"] == "NOT_LOADED" and info["state_layout"] == "B,Hv,K,V"
    assert info["inputs"]["q"]["shape"] == [1, 8192, 16, 128] and info["inputs"]["initial_state"] is None
    assert info["configuration_basis"] == "b200-measured-shape"
    json.dumps(info)


def test_route_info_with_binary_records_library_identity(native_library):
    with mock.patch.object(sm100_policy, "device_profile", return_value=B200):
        info = gdn_route.get_gdn_route_info(*_args())
    image = info["native_images"][0]
    assert image["sha256"] == _library._sha(image["path"])
    assert info["native_status"] == "LOADED_FILES_VERIFIED_NOT_DEVICE_ADMITTED"


def test_header_and_library_export_the_same_symbols(native_library):
    header = (ROOT / "include" / "actlize_la_sm100.h").read_text()
    declared = set(re.findall(r"\b(actlize_la_sm100_\w+)\s*\(", header))
    assert declared == set(_library.EXPORTS), declared ^ set(_library.EXPORTS)
    raw = ctypes.CDLL(native_library.info["library_path"])
    for name in declared:
        assert getattr(raw, name) is not None
    assert native_library.lib.actlize_la_sm100_abi_version() == 1
    assert native_library.lib.actlize_la_sm100_target_arch() == 100
    assert native_library.numerical_contract == sm100.MATH_CONTRACT


def test_native_select_agrees_with_python_policy(native_library):
    lib = native_library.lib
    ids = sm100_policy.policy()["configuration_ids"]
    for row in sm100_policy.policy()["rows"]:
        want = ids[row["configuration"]] | (row.get("segments", 1) << 8) | (row.get("parallel", 1) << 16)
        assert lib.actlize_la_sm100_select(*row["shape"], 1) == want
        profile_choice = sm100_policy.select((*row["shape"], 128, 128), B200)
        assert profile_choice.configuration_id == want
    # shapes without a measured row: the default configuration with the rule's segment count, same on both sides
    for shape in [(3, 100, 2, 4), (1, 65536, 16, 32), (1, 16384, 16, 32), (2, 4096, 8, 48), (16, 8192, 16, 32),
                  (1, 511, 1, 1), (1, 513, 1, 64), (3, 1025, 16, 48), (1, 1 << 20, 1, 2)]:
        want = sm100_policy.select((*shape, 128, 128), B200)
        assert want.basis == "unmeasured-shape-default"
        assert lib.actlize_la_sm100_select(*shape, 0) == want.configuration_id, shape
    # the walk of up to 74 heads is split into parallel sub-segments (then one sequence segment); 75..148 heads
    # leave SMs idle without room for a second CTA per head, so the prepare of later segments overlaps the walk
    assert sm100_policy.default_parallel(1, 65536, 32) == 4 and sm100_policy.default_segments(1, 65536, 32) == 1
    assert sm100_policy.default_parallel(1, 16384, 48) == 3 and sm100_policy.default_parallel(1, 1024, 16) == 2
    assert sm100_policy.default_parallel(1, 16384, 100) == 1 and sm100_policy.default_segments(1, 16384, 64) == 1
    assert sm100_policy.default_parallel(1, 1 << 20, 2) == 8 and sm100_policy.default_parallel(1, 511, 1) == 1
    assert sm100_policy.default_segments(3, 100, 4) == 1 and sm100_policy.default_segments(16, 8192, 32) == 1
    assert lib.actlize_la_sm100_select(1, 64, 3, 4, 0) < 0
    assert lib.actlize_la_sm100_select(0, 64, 1, 1, 0) < 0


def test_native_argument_rejection_without_a_device(native_library):
    lib = native_library.lib
    invalid = 1   # cudaErrorInvalidValue
    n = lib.actlize_la_sm100_workspace_bytes(1, 8192, 16, 32, 1)
    assert n == 32 * 128 * (16384 * 2 + 32768 + 8192 + 768)       # W^T hi/lo, U, P, gate vector per block
    # a segmented walk carries one FP32 128x128 state per (batch, value head) between segments
    assert lib.actlize_la_sm100_workspace_bytes(1, 8192, 16, 32, 1 | (4 << 8)) == n + 32 * 65536
    assert lib.actlize_la_sm100_launches_per_forward(1 | (4 << 8)) == 8
    assert lib.actlize_la_sm100_workspace_bytes(1, 64, 3, 4, 1) < 0
    assert lib.actlize_la_sm100_workspace_bytes(1, 64, 1, 1, 9) < 0
    # the offset pass of the sequence-parallel scheme is a walk-only call of the tcgen05 configuration, on its own
    offset_pass = 0x100000
    assert lib.actlize_la_sm100_workspace_bytes(1, 64, 1, 1, 1 | 0x20 | offset_pass) > 0
    for bad in (1 | offset_pass, 0 | 0x20 | offset_pass, 1 | 0x20 | 0x40 | offset_pass, 1 | 0x20 | (2 << 16) | offset_pass):
        assert lib.actlize_la_sm100_workspace_bytes(1, 64, 1, 1, bad) < 0, hex(bad)
    pair_pass = 0x200000                          # offset and transition pass in one launch: likewise on its own
    assert lib.actlize_la_sm100_workspace_bytes(1, 64, 1, 1, 1 | 0x20 | pair_pass) > 0
    for bad in (1 | pair_pass, 1 | 0x20 | pair_pass | offset_pass, 1 | 0x20 | 0x80 | pair_pass, 3 | 0x20 | pair_pass):
        assert lib.actlize_la_sm100_workspace_bytes(1, 64, 1, 1, bad) < 0, hex(bad)
    big = 1 << 40
    walk_args = [ptr_ := 0x1000] * 5 + [None, ptr_ + 256, None, ptr_ + 512, big, 1, 64, 1, 1, 1, 1 | 0x20 | offset_pass, None]
    assert lib.actlize_la_sm100_forward_prepared(*walk_args) == invalid     # the offset pass needs final_state
    args = [None] * 9 + [0, 1, 64, 1, 1, 1, 1, None]
    assert lib.actlize_la_sm100_forward_prepared(*args) == invalid
    ptr = 0x1000
    args = [ptr] * 5 + [None, ptr + 256, None, ptr + 512, 10, 1, 64, 1, 1, 1, 1, None]
    assert lib.actlize_la_sm100_forward_prepared(*args) == invalid     # workspace too small
    assert lib.actlize_la_sm100_launches_per_forward(1) == 2
    assert lib.actlize_la_sm100_host_arena_bytes(1, 64, 1, 1, 1, 0, 1, 1) > n // 32 // 128


def test_loader_rejects_missing_and_tampered_binaries(tmp_path, monkeypatch, native_library):
    monkeypatch.setenv(_library.ENVIRONMENT_OVERRIDE, str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError):
        _library.get_library_info()
    monkeypatch.setenv(_library.ENVIRONMENT_OVERRIDE, "relative.so")
    with pytest.raises(RuntimeError):
        _library.get_library_info()
    source = Path(native_library.info["library_path"])
    copy = tmp_path / source.name
    copy.write_bytes(source.read_bytes() + b"\0")
    (tmp_path / "build.json").write_text(source.with_name("build.json").read_text())
    monkeypatch.setenv(_library.ENVIRONMENT_OVERRIDE, str(copy))
    with pytest.raises(RuntimeError, match="hash differs"):
        _library.get_library_info()
    (tmp_path / "build.json").unlink()
    with pytest.raises(RuntimeError, match="receipt"):
        _library.get_library_info()


def test_forward_validation_errors_are_value_errors():
    good = dict(b=1, t=64, hk=1, hv=2)
    def tensors(**over):
        b, t, hk, hv = (good[k] for k in ("b", "t", "hk", "hv"))
        q = torch.zeros(b, t, hk, 128, dtype=torch.bfloat16)
        base = dict(q=q, k=q.clone(), v=torch.zeros(b, t, hv, 128, dtype=torch.bfloat16),
                    g=torch.zeros(b, t, hv), beta=torch.zeros(b, t, hv, dtype=torch.bfloat16))
        base.update(over)
        return base
    def check(**over):
        x = tensors(**over)
        with pytest.raises(ValueError):
            sm100._validate(x["q"], x["k"], x["v"], x["g"], x["beta"], x.get("initial_state"))
    check()                                                        # CPU tensors are rejected
    check(g=torch.zeros(1, 64, 2, dtype=torch.float16))
    check(v=torch.zeros(1, 64, 3, 64, dtype=torch.bfloat16))
    check(beta=torch.zeros(1, 64, 2))
    check(initial_state=torch.zeros(1, 2, 128, 128, dtype=torch.float64))
    with pytest.raises(ValueError):
        sm100.configuration_id("value64")
    # the graph-capture form of the sequence-parallel call refuses host tensors before anything else happens
    x = tensors()
    with pytest.raises(ValueError, match="CUDA"):
        actlizela_b200.capture_sequence_parallel(x["q"], x["k"], x["v"], x["g"], x["beta"])


def test_build_entry_and_arch_guard_are_present():
    entry = ROOT / "actlizela_b200" / registry.require_backend("cuda_sm100")["build_entry"]
    text = entry.read_text()
    assert 'STREQUAL "cuda_sm100"' in text and "FATAL_ERROR" in text
    common = (ROOT / "actlizela_b200/csrc/backends/sm100/gdn_common.cuh").read_text()
    assert "__CUDA_ARCH__ != 1000" in common and "#error" in common
    receipt = json.loads((ROOT / "actlizela_b200/_native/build.json").read_text())
    assert "arch=compute_100a,code=sm_100a" in receipt["flags"]


def test_no_file_io_or_hashing_per_call(native_library):
    """After the first load, resolving the library must not touch the file system
    (the reference tests the same property: tests/test_gdn_route.py:112-117)."""
    first = _library.load_library()
    with mock.patch.object(_library, "_sha", side_effect=AssertionError("hashing on the call path")), \
            mock.patch.object(_library.Path, "is_file", side_effect=AssertionError("file system on the call path")):
        for _ in range(3):
            assert _library.load_library() is first


def test_auxiliary_wrappers_reject_ill_formed_operands_before_any_launch():
    """Every operand of the decode / verify / commit / input-preparation / gated-RMSNorm wrappers is checked for
    shape, dtype, device, contiguity and alignment before a pointer reaches the library: CPU tensors only here,
    so nothing can be launched (a well-formed CPU call fails on the device check)."""
    from actlizela_b200 import aux_ops
    bf16 = dict(dtype=torch.bfloat16)
    b, w, hk, hv = 2, 3, 2, 4
    q, k = torch.zeros(b, hk, 128, **bf16), torch.zeros(b, hk, 128, **bf16)
    v, g, beta = torch.zeros(b, hv, 128, **bf16), torch.zeros(b, hv), torch.zeros(b, hv, **bf16)
    state = torch.zeros(b, hv, 128, 128)
    bad_decode = [
        dict(k=torch.zeros(b, hk + 1, 128, **bf16)), dict(k=torch.zeros(b, hk, 64, **bf16)),
        dict(v=torch.zeros(b + 1, hv, 128, **bf16)), dict(beta=torch.zeros(b, hv + 1, **bf16)),
        dict(beta=torch.zeros(b, hv)), dict(g=torch.zeros(b, hv, dtype=torch.float64)),
        dict(state=torch.zeros(b, hv, 128, 64)), dict(q=torch.zeros(b, 3, 128, **bf16), k=torch.zeros(b, 3, 128, **bf16)),
    ]
    for change in bad_decode:
        args = {**dict(q=q, k=k, v=v, g=g, beta=beta, state=state), **change}
        with pytest.raises(ValueError, match="shape|dtype|Hv % Hk"):
            aux_ops.gdn_decode_step(**args)
    with pytest.raises(ValueError, match="CUDA"):
        aux_ops.gdn_decode_step(q, k, v, g, beta, state)

    q4, k4 = torch.zeros(b, w, hk, 128, **bf16), torch.zeros(b, w, hk, 128, **bf16)
    v4, g3, beta3 = torch.zeros(b, w, hv, 128, **bf16), torch.zeros(b, w, hv), torch.zeros(b, w, hv, **bf16)
    for change in (dict(q=torch.zeros(b, w, hk, 64, **bf16)), dict(v=torch.zeros(b, w, hv + 1, 128, **bf16)),
                   dict(beta=torch.zeros(b, w + 1, hv, **bf16)), dict(k=torch.zeros(b, 65, hk, 128, **bf16),
                                                                     g=torch.zeros(b, 65, hv))):
        args = {**dict(q=q4, k=k4, v=v4, g=g3, beta=beta3, state=state), **change}
        with pytest.raises(ValueError, match="shape|width"):
            aux_ops.gdn_verify_step(**args)
    delta, counts = torch.zeros(b, w, hv, 128), torch.zeros(b, dtype=torch.int32)
    for change in (dict(delta=torch.zeros(b, w, hv, 64)), dict(counts=torch.zeros(b + 1, dtype=torch.int32)),
                   dict(counts=torch.zeros(b)), dict(g=torch.zeros(b, w, hv)[:, :, ::1].transpose(0, 1))):
        args = {**dict(k=k4, g=g3, delta=delta, counts=counts, state=state), **change}
        with pytest.raises(ValueError, match="shape|dtype"):
            aux_ops.gdn_commit_step(**args)

    n = 5
    mixed = torch.zeros(n, (2 * hk + hv) * 128, **bf16)
    a, a_log = torch.zeros(n, hv, **bf16), torch.zeros(hv)
    for change in (dict(a=torch.zeros(n + 1, hv, **bf16)), dict(b=torch.zeros(n, hv)), dict(a_log=torch.zeros(hv + 1)),
                   dict(dt_bias=torch.zeros(hv, dtype=torch.float64)), dict(mixed=torch.zeros(n, 100, **bf16))):
        args = {**dict(mixed=mixed, a=a, b=a, a_log=a_log, dt_bias=a_log, key_heads=hk, value_heads=hv), **change}
        with pytest.raises(ValueError):
            aux_ops.gdn_prepare_inputs(**args)
    y = torch.zeros(7, 128, **bf16)
    for change in (dict(z=torch.zeros(6, 128, **bf16)), dict(weight=torch.zeros(64, **bf16)), dict(y=torch.zeros(7, 64, **bf16))):
        args = {**dict(y=y, z=y, weight=torch.zeros(128, **bf16)), **change}
        with pytest.raises(ValueError):
            aux_ops.rmsnorm_gated(**args)
