"""CPU-side checks of the drop-in boundary: the library loads, exports every symbol the header
declares, and refuses to run without a GPU (no CPU fallback).  No compute calls here."""
import os
import re

import pytest

import mer_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "mer_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mer_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = mer_b200.load_library()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/mer_b200.h but not exported"
    assert sorted(mer_b200.ABI_SYMBOLS) == declared, "ctypes table and header disagree"


def test_abi_version_and_names():
    lib = mer_b200.load_library()
    assert lib.mer_abi_version() == 1
    # Display strings of GpuExpertDispatchErrorKind, backend/mod.rs:403-418
    names = {1: "residency-miss", 2: "physical-capacity", 3: "upload", 4: "validation-dispatch", 5: "submission",
             6: "readback-channel", 7: "readback-map", 8: "device-lost", 9: "runtime-invariant"}
    for kind, name in names.items():
        assert lib.mer_error_kind_name(kind).decode() == name
        assert str(mer_b200.GpuExpertDispatchErrorKind(kind)) == name


def test_expert_bytes_match_reference_sizes(golden):
    for c in golden["expert_bytes"]:
        dt = mer_b200.DTYPE_Q4_0 if c["dtype"] == "q4_0" else mer_b200.DTYPE_Q8_0
        assert mer_b200.expert_bytes(dt, c["d_model"], c["d_ff"]) == c["bytes"]


def test_compatibility_rule():
    # routed_expert_gpu_compatibility, backend/mod.rs:4691-4720 (extended: Q8_0 is eligible here)
    assert mer_b200.routed_expert_gpu_compatibility(mer_b200.DTYPE_Q4_0, 4096, 14336)
    assert mer_b200.routed_expert_gpu_compatibility(mer_b200.DTYPE_Q8_0, 2048, 768)
    assert not mer_b200.routed_expert_gpu_compatibility(7, 2048, 768)
    assert not mer_b200.routed_expert_gpu_compatibility(mer_b200.DTYPE_Q4_0, 0, 768)


def test_no_cpu_fallback_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(mer_b200.GpuExpertDispatchError) as e:
        mer_b200.Backend(mer_b200.DTYPE_Q8_0, 64, 64, 1 << 20, 8)
    assert e.value.kind == mer_b200.GpuExpertDispatchErrorKind.DeviceLost


def test_unbound_gate_refuses_to_route_on_the_host():
    gate = mer_b200.LinearGate([0.0] * 8, 4, 2, 2)
    with pytest.raises(RuntimeError):
        gate.route([0.0, 0.0])
    with pytest.raises(ValueError):
        mer_b200.LinearGate([0.0] * 8, 4, 2, 5)


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "micro-expert-router-ssd-streamed-moe-mer_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "import oracle" not in text and "mer_oracle" not in text, f
