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


def test_schedule_multipliers_of_the_library_match_nanolab(golden_dir):
    """ojc_lr_multiplier is host arithmetic (no device): pinned to the reference's schedule fixture at LR_MULT_REL_TOL 1e-12
    (ojas-oracle/src/parity.rs:60) and to the refusals of ojas-cpu/src/schedule.rs."""
    import json
    from ojas_b200 import OjasError, TrainConfig
    fx = json.loads((golden_dir / "tiny/lr_schedules.json").read_text())
    for name in ("acceptance_cosine", "acceptance_wsd", "tiny_cosine", "tiny_wsd"):
        s = fx[name]
        cfg = TrainConfig(schedule=s["schedule"], warmup_steps=s["warmup_steps"], total_steps=s["total_steps"], decay_frac=s["wsd_decay_frac"])
        for step, want in enumerate(s["multipliers"]):
            assert abs(cfg.lr_multiplier(step) - want) <= 1e-12 * abs(want), (name, step)
    assert TrainConfig().lr_multiplier(123) == 1.0
    assert TrainConfig(schedule="cosine", total_steps=10).lr_multiplier(0) == 1.0        # warmup 0: the decay branch at t = 0
    assert abs(TrainConfig(schedule="cosine", total_steps=10).lr_multiplier(5000) - 0.1) < 1e-15
    for bad, step in ((TrainConfig(schedule="wsd", total_steps=10), 11), (TrainConfig(schedule="cosine", total_steps=0), 0),
                      (TrainConfig(schedule="wsd", total_steps=10, decay_frac=1.5), 0), (TrainConfig(schedule="cosine", total_steps=10), (1 << 64) - 1)):
        with pytest.raises(OjasError) as e:
            bad.lr_multiplier(step)
        assert e.value.kind == "OutOfRange"


def test_a_session_without_a_device_reports_the_open_error_and_leaves_no_thread_behind():
    import threading
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from ojas_b200 import OjasError, Session
    before = threading.active_count()
    with pytest.raises(OjasError) as e:
        Session(0, 1 << 30, open_timeout_ms=30_000)
    assert e.value.kind == "NoDevice" and threading.active_count() == before


def test_the_communicator_reaches_nccl_without_a_device():
    """ojc_comm_unique_id loads NCCL with dlopen on first use and needs no GPU: two ids differ, and ojc_comm_init without a device is refused
    by the backend check, not by a crash."""
    import ctypes as C
    from ojas_b200._lib import lib
    a, b = (C.c_uint8 * 128)(), (C.c_uint8 * 128)()
    st = lib.ojc_comm_unique_id(a)
    if st == 11:        # Unsupported: no libnccl.so.2 on this machine
        pytest.skip(lib.ojc_last_error().decode())
    assert st == 0 and lib.ojc_comm_unique_id(b) == 0
    assert any(bytes(a)) and bytes(a) != bytes(b)
    out = C.c_void_p()
    assert lib.ojc_comm_init(None, C.c_int32(0), C.c_int32(1), a, C.byref(out)) != 0 and not out.value
