"""CPU-side checks of the drop-in boundary: the shared library loads, exports every entry point include/ojas_cuda.h
declares, and refuses to open without a device (no silent host fallback)."""
import re

import pytest


def test_library_exports_every_declared_entry_point():
    from ojas_b200._lib import HEADER_PATH, lib
    names = sorted(set(re.findall(r"\b(ojc_[a-z0-9_]+)\s*\(", HEADER_PATH.read_text())))
    assert len(names) >= 60
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_status_names_mirror_the_reference_error_variants():
    from ojas_b200 import STATUS_NAMES
    from ojas_b200._lib import lib
    for code, name in enumerate(STATUS_NAMES):
        assert lib.ojc_status_name(code).decode() == name
    # ojas-core/src/error.rs:18-118
    for variant in ("Shape", "Dtype", "OutOfRange", "NonFinite", "UnsupportedHeadDim", "CapacityExceeded", "Poisoned", "DeviceLost", "WaitTimeout",
                    "Backend", "Unsupported", "Placement"):
        assert variant in STATUS_NAMES


def test_open_without_a_device_is_an_explicit_error():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from ojas_b200 import CudaBackend, OjasError
    with pytest.raises(OjasError) as e:
        CudaBackend(0)
    assert e.value.kind == "NoDevice" and not e.value.retryable


def test_flops_per_token_matches_the_scope_table():
    from ojas_b200 import ModelSpec
    spec = ModelSpec.nanolab_124m()
    assert spec.matmul_params() == 123_678_720
    assert abs(spec.flops_per_token(1024) - 7.9870e8) / 7.9870e8 < 1e-4
    assert ModelSpec.nanolab_124m(hidden=3072).matmul_params() == 151_990_272
