"""Loads libojas_cuda.so (the C ABI of include/ojas_cuda.h). There is no fallback: a missing library is an ImportError."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libojas_cuda.so"
HEADER_PATH = _PKG.parent / "include" / "ojas_cuda.h"

MAX_RANK = 6


class CTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_int64 * MAX_RANK), ("stride", C.c_int64 * MAX_RANK)]


class AdamWConfig(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("lr", "beta1", "beta2", "eps", "weight_decay")]


class MuonConfig(C.Structure):
    _fields_ = [("lr", C.c_double), ("momentum", C.c_double), ("weight_decay", C.c_double), ("nesterov", C.c_int32), ("ns5_bf16", C.c_int32)]


class ModelSpec(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("vocab", "n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "hidden", "max_seq", "window")] + [
        ("rope_base", C.c_double), ("rms_eps", C.c_float)]


class TrainConfig(C.Structure):
    _fields_ = [("autocast_bf16", C.c_int32), ("optimizer", C.c_int32),
                ("adam_lr", C.c_double), ("adam_beta1", C.c_double), ("adam_beta2", C.c_double), ("adam_eps", C.c_double), ("adam_weight_decay", C.c_double),
                ("matrix_lr", C.c_double), ("muon_momentum", C.c_double), ("muon_weight_decay", C.c_double),
                ("ns5_bf16", C.c_int32), ("grad_clip", C.c_float), ("has_ignore", C.c_int32), ("ignore_index", C.c_uint32),
                ("ce_chunk_rows", C.c_int64), ("loss_seed", C.c_float), ("checkpoint_blocks", C.c_int32),
                ("schedule", C.c_int32), ("warmup_steps", C.c_uint64), ("total_steps", C.c_uint64), ("decay_frac", C.c_double), ("on_nonfinite", C.c_int32)]


class StepReport(C.Structure):
    _fields_ = [("loss", C.c_float), ("grad_norm", C.c_float), ("step", C.c_uint64), ("tokens", C.c_uint64), ("lr_multiplier", C.c_double)]


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: build it with `make -C {_PKG / 'csrc'}` (or __graft_entry__.build()); "
                          "this package has no CPU or library fallback")
    lib = C.CDLL(str(LIB_PATH))
    lib.ojc_last_error.restype = C.c_char_p
    lib.ojc_status_name.restype = C.c_char_p
    lib.ojc_stream.restype = C.c_void_p
    lib.ojc_kernel_launches.restype = C.c_uint64
    lib.ojc_trainer_param_count.restype = C.c_int64
    lib.ojc_trainer_steps_done.restype = C.c_uint64
    lib.ojc_fnv1a64.restype = C.c_uint64
    lib.ojc_fnv1a64.argtypes = [C.c_uint64, C.c_void_p, C.c_uint64]
    lib.ojc_trainer_bucket_count.restype = C.c_int64
    return lib


lib = load()
