"""The trainer's checkpoint directory, byte for byte as the reference writes it (ojas-model/src/checkpoint.rs:1-33):

    model.safetensors   F32 weights under their nanolab names in param_table order; metadata ojas.spec, ojas.step, ojas.run
    optim.safetensors   muon.<name> | adam_m.<name>, adam_v.<name> for every trained parameter; metadata ojas.step, ojas.run
    state.ojck          checkpoint v1 with empty tensor sections: config JSON {"format","run","spec","train"}, tokenizer
                        hash, git sha, step, data cursor and the sampler's 16-byte rng_state (docs/checkpoint-v1.md)

`save` reads one tensor at a time off the device (one download each, as checkpoint.rs:15-19), builds the three files in a
staging directory beside the target and swaps it in; a target that is neither empty nor an earlier checkpoint is refused
untouched (checkpoint.rs:9-13). `resume` checks step and run across the three files, the saved train config against the
caller's, the rng_state against the caller's data_seed, and every tensor's name, dtype and shape before the first upload
(checkpoint.rs:21-29). Under data parallelism rank 0 saves (all ranks hold the same bits) and every rank resumes.
"""
from __future__ import annotations

import json
import os
import shutil
import struct
from dataclasses import dataclass, field
from decimal import Decimal
from pathlib import Path

import numpy as np

from .data import DataCursor, DataError, SamplerRngState

MODEL_FILE, OPTIM_FILE, STATE_FILE = "model.safetensors", "optim.safetensors", "state.ojck"
SPEC_METADATA_KEY, STEP_METADATA_KEY, RUN_METADATA_KEY = "ojas.spec", "ojas.step", "ojas.run"
STATE_FORMAT = "ojas-train-v1"
CHECKPOINT_MAGIC, CHECKPOINT_VERSION = b"OJAS0001", 1      # ojas-core/src/checkpoint.rs:31-50
MAX_STATE_BYTES = 1 << 20                                  # checkpoint.rs:69: the state file holds no tensors
_PIECE = 64 * 1024                                         # bytes written per piece (checkpoint.rs:71)
_MASK64 = (1 << 64) - 1


class CheckpointError(ValueError):
    """A refusal of save or resume; `kind` is the reference's error variant (OutOfRange for refusals, Shape for layout)."""

    def __init__(self, kind: str, detail: str):
        super().__init__(f"{kind}: {detail}")
        self.kind, self.detail = kind, detail


def _refuse(detail: str) -> CheckpointError:
    return CheckpointError("OutOfRange", detail)


# ------------------------------------------------------------------------------------------------ text forms
def rust_float(x: float) -> str:
    """An f64 as Rust's `{:?}` prints it (shortest digits that round-trip; plain decimal with at least one fractional digit
    for 1e-4 <= |x| < 1e16, otherwise `d.ddde-N`), the form ModelSpec::to_json and TrainConfig::to_json use."""
    x = float(x)
    if x != x:
        return "NaN"
    if x in (float("inf"), float("-inf")):
        return "inf" if x > 0 else "-inf"
    if x == 0.0:
        return "-0.0" if str(x).startswith("-") else "0.0"
    sign, digits, exp = Decimal(repr(x)).as_tuple()
    while len(digits) > 1 and digits[-1] == 0:
        digits, exp = digits[:-1], exp + 1
    ds = "".join(map(str, digits))
    point = len(ds) + exp                                    # position of the decimal point relative to the digits
    if 1e-4 <= abs(x) < 1e16:
        if point <= 0:
            body = "0." + "0" * (-point) + ds
        elif point >= len(ds):
            body = ds + "0" * (point - len(ds)) + ".0"
        else:
            body = ds[:point] + "." + ds[point:]
    else:
        body = ds[0] + ("." + ds[1:] if len(ds) > 1 else "") + "e" + str(point - 1)
    return ("-" if sign else "") + body


def rust_f32(x: float) -> str:
    """An f32 as Rust's `{:?}` prints it (TrainConfig.grad_clip is f32)."""
    v = np.float32(x)
    if not np.isfinite(v) or v == 0:
        return rust_float(float(v))
    sign, digits, exp = Decimal(np.format_float_scientific(v, unique=True, trim="-")).as_tuple()
    # the shortest digits that identify the f32, laid out by the same rule as an f64
    ds = "".join(map(str, digits)).rstrip("0") or "0"
    exp += len(digits) - len(ds)
    point, a = len(ds) + exp, abs(float(v))
    if 1e-4 <= a < 1e16:
        body = "0." + "0" * (-point) + ds if point <= 0 else (ds + "0" * (point - len(ds)) + ".0" if point >= len(ds) else ds[:point] + "." + ds[point:])
    else:
        body = ds[0] + ("." + ds[1:] if len(ds) > 1 else "") + "e" + str(point - 1)
    return ("-" if sign else "") + body


def quote(s: str) -> str:
    """ojas-io/src/json_write.rs:99-119: the five short escapes, \\u00XX below 0x20, everything else as it is."""
    out = ['"']
    for ch in s:
        if ch == '"':
            out.append('\\"')
        elif ch == "\\":
            out.append("\\\\")
        elif ch == "\n":
            out.append("\\n")
        elif ch == "\r":
            out.append("\\r")
        elif ch == "\t":
            out.append("\\t")
        elif ord(ch) < 0x20:
            out.append("\\u%04x" % ord(ch))
        else:
            out.append(ch)
    out.append('"')
    return "".join(out)


def spec_json(spec) -> str:
    """ModelSpec::to_json (ojas-model/src/spec.rs:246-268): ojas-spec-v1, or v2 with a trailing window."""
    fmt, window = ("ojas-spec-v1", "") if spec.window is None else ("ojas-spec-v2", f',"window":{spec.window}')
    return (f'{{"format":"{fmt}","arch":"nanolab-gpt","vocab":{spec.vocab},"n_embd":{spec.n_embd},"n_layer":{spec.n_layer},"n_head":{spec.n_head},'
            f'"n_kv_head":{spec.n_kv_head},"head_dim":{spec.head_dim},"hidden":{spec.hidden},"max_seq":{spec.max_seq},"rope_base":{rust_float(spec.rope_base)},'
            f'"rms_eps":{rust_float(spec.rms_eps)},"tie_embeddings":true,"qk_norm":true,"gated_attention":true,"value_residual":true{window}}}')


def spec_from_json(text: str):
    from .backend import ModelSpec
    d = json.loads(text)
    if d.get("arch") != "nanolab-gpt" or d.get("format") not in ("ojas-spec-v1", "ojas-spec-v2"):
        raise _refuse(f"spec format {d.get('format')!r} / arch {d.get('arch')!r} is not one this trainer reads")
    if (d["format"] == "ojas-spec-v2") != ("window" in d):
        raise _refuse("window is required in ojas-spec-v2 and refused in ojas-spec-v1")
    return ModelSpec(vocab=d["vocab"], n_embd=d["n_embd"], n_layer=d["n_layer"], n_head=d["n_head"], n_kv_head=d["n_kv_head"], head_dim=d["head_dim"],
                     hidden=d["hidden"], max_seq=d["max_seq"], window=d.get("window"), rope_base=float(d["rope_base"]), rms_eps=float(d["rms_eps"]))


@dataclass
class RunConfig:
    """The fields TrainConfig::to_json serializes (ojas-model/src/trainer.rs:179-221), plus the two hashes the state file
    carries in their own fields. `schedule` is "cosine" (decay_frac prints as 0.0) or "wsd"."""
    batch: int
    seq_len: int
    accum: int = 1
    data_seed: int = 0
    schedule: str = "cosine"
    decay_frac: float = 0.0
    total_steps: int = 0
    warmup_steps: int = 0
    matrix_lr: float = 0.025
    adam_lr: float = 6e-4
    grad_clip: float = 1.0
    on_nonfinite: str = "abort"
    ignore_index: int | None = None
    chunk_rows: int = 1024
    chunk_cols: int = 8192
    autocast_bf16: bool = False
    muon_ns5_bf16: bool = False
    tokenizer_hash: bytes = field(default=bytes(32))
    git_sha: bytes = field(default=bytes(20))

    def to_json(self) -> str:
        # keys in sorted order; autocast and muon_ns5 are absent at their defaults so older texts stay the same
        autocast = '"autocast":"bf16",' if self.autocast_bf16 else ""
        ns5 = '"muon_ns5":"bf16",' if self.muon_ns5_bf16 else ""
        decay = self.decay_frac if self.schedule == "wsd" else 0.0
        return (f'{{"accum":{self.accum},"adam_lr":{rust_float(self.adam_lr)},{autocast}"batch":{self.batch},"chunk_cols":{self.chunk_cols},'
                f'"chunk_rows":{self.chunk_rows},"data_seed":{self.data_seed},"decay_frac":{rust_float(decay)},"grad_clip":{rust_f32(self.grad_clip)},'
                f'"ignore":{"true" if self.ignore_index is not None else "false"},"ignore_index":{self.ignore_index or 0},"matrix_lr":{rust_float(self.matrix_lr)},'
                f'{ns5}"on_nonfinite":{quote(self.on_nonfinite)},"schedule":{quote(self.schedule)},"seq_len":{self.seq_len},"total_steps":{self.total_steps},'
                f'"warmup_steps":{self.warmup_steps}}}')


def state_config(run: str, spec_text: str, train_text: str) -> str:
    """checkpoint.rs:246-255: four string values; the spec and the train config ride as quoted JSON texts."""
    return f'{{"format":{quote(STATE_FORMAT)},"run":{quote(run)},"spec":{quote(spec_text)},"train":{quote(train_text)}}}'


def _fnv1a(data: bytes, h: int = 0xCBF29CE484222325) -> int:
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & _MASK64
    return h


def compute_run_id(spec_text: str, train_text: str, params) -> str:
    """ojas-model/src/trainer.rs:436-456: FNV-1a over the tag, both config texts (each followed by a zero byte) and every
    parameter's f32 bytes in table order, as 16 lowercase hex digits."""
    h = _fnv1a(b"ojas-run-v1\0")
    for text in (spec_text, train_text):
        h = _fnv1a(text.encode() + b"\0", h)
    prime, mask = 0x100000001B3, _MASK64
    for p in params:
        for b in np.ascontiguousarray(p, "<f4").tobytes():     # small models only: the step driver takes a run id as given for large ones
            h = ((h ^ b) * prime) & mask
    return "%016x" % h


def is_run_id(run: str) -> bool:
    return len(run) == 16 and all(c in "0123456789abcdef" for c in run)
