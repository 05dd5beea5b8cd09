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
    from ._lib import lib
    for p in params:
        a = np.ascontiguousarray(p, "<f4")
        h = lib.ojc_fnv1a64(h, a.ctypes.data, a.nbytes)
    return "%016x" % h


def is_run_id(run: str) -> bool:
    return len(run) == 16 and all(c in "0123456789abcdef" for c in run)


# ------------------------------------------------------------------------------------------------ safetensors
def safetensors_header(tensors, metadata) -> tuple[bytes, int]:
    """The header ojas-io lays out (safetensors.rs:1305-1398): `__metadata__` first with its keys in the order given, then
    the tensors in declared (= data) order as {"dtype","shape","data_offsets"}, no whitespace, space-padded to a multiple of
    eight. `tensors` is [(name, shape)], all F32. Returns the padded header and the data length."""
    seen, cursor, parts = set(), 0, []
    if metadata:
        keys = [k for k, _ in metadata]
        if len(set(keys)) != len(keys):
            raise _refuse("duplicate metadata key")
        parts.append('"__metadata__":{' + ",".join(f"{quote(k)}:{quote(v)}" for k, v in metadata) + "}")
    for name, shape in tensors:
        if not name or name == "__metadata__" or name in seen:
            raise _refuse(f"tensor name {name!r} is empty, reserved or repeated")
        seen.add(name)
        nbytes = 4 * int(np.prod(shape, dtype=np.int64)) if len(shape) else 4
        parts.append(f'{quote(name)}:{{"dtype":"F32","shape":[{",".join(str(int(d)) for d in shape)}],"data_offsets":[{cursor},{cursor + nbytes}]}}')
        cursor += nbytes
    header = ("{" + ",".join(parts) + "}").encode()
    header += b" " * ((8 - len(header) % 8) % 8)
    return header, cursor


def write_safetensors(path: Path, tensors, metadata, fetch) -> None:
    """Streams the file: header first, then fetch(i) -> float32 array for each tensor in turn, written in 64 KiB pieces so
    the host holds one tensor at a time (checkpoint.rs:15-19, 462-520)."""
    header, _ = safetensors_header([(n, s) for n, s in tensors], metadata)
    with open(path, "xb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        for i, (name, shape) in enumerate(tensors):
            a = np.ascontiguousarray(fetch(i), "<f4")
            if tuple(a.shape) != tuple(shape):
                raise CheckpointError("Shape", f"{name}: {a.shape} read back, {tuple(shape)} declared")
            raw = memoryview(a).cast("B")
            for off in range(0, len(raw), _PIECE):
                f.write(raw[off:off + _PIECE])
        f.flush()
        os.fsync(f.fileno())


class SafeTensorsFile:
    """Header of a safetensors file plus positioned reads of one tensor at a time."""

    def __init__(self, path: Path):
        self.path = Path(path)
        size = self.path.stat().st_size
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise _refuse(f"{path}: shorter than its length prefix")
            (n,) = struct.unpack("<Q", head)
            if n == 0 or 8 + n > size:
                raise _refuse(f"{path}: header length {n} does not fit {size} bytes")
            doc = json.loads(f.read(n).decode())
        self.metadata = dict(doc.pop("__metadata__", {}))
        self.tensors = doc                         # name -> {"dtype","shape","data_offsets"}; insertion order = file order
        self.data_start = 8 + n
        end = max((t["data_offsets"][1] for t in doc.values()), default=0)
        if self.data_start + end != size:
            raise _refuse(f"{path}: {size} bytes, header and data account for {self.data_start + end}")

    def read(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        lo, hi = t["data_offsets"]
        with open(self.path, "rb") as f:
            f.seek(self.data_start + lo)
            raw = f.read(hi - lo)
        if len(raw) != hi - lo:
            raise _refuse(f"{self.path}: {name} is truncated")
        return np.frombuffer(raw, "<f4").reshape(t["shape"])


# ------------------------------------------------------------------------------------------------ state.ojck
def encode_state(config: bytes, tokenizer_hash: bytes, git_sha: bytes, step: int, cursor: DataCursor, rng_state: bytes) -> bytes:
    """Checkpoint v1 with four empty record sections (ojas-io/src/checkpoint.rs:170-185, 286-296): an empty section is its
    body length 8 and a record count 0."""
    if len(tokenizer_hash) != 32 or len(git_sha) != 20:
        raise _refuse("tokenizer_hash is 32 bytes and git_sha 20")
    lp = lambda b: struct.pack("<Q", len(b)) + b
    empty = struct.pack("<QQ", 8, 0)
    return (CHECKPOINT_MAGIC + struct.pack("<I", CHECKPOINT_VERSION) + lp(config) + tokenizer_hash + git_sha +
            struct.pack("<QQQ", step, cursor.shard, cursor.token_index) + lp(rng_state) + empty * 4)


def decode_state(data: bytes) -> dict:
    """The inverse, refusing a wrong magic or version, a truncated field, trailing bytes, or a section that holds records."""
    if len(data) > MAX_STATE_BYTES:
        raise _refuse(f"state file of {len(data)} bytes: the trainer's holds no tensors and stays under {MAX_STATE_BYTES}")
    pos = 0

    def take(n: int) -> bytes:
        nonlocal pos
        if n < 0 or pos + n > len(data):
            raise _refuse("truncated checkpoint")
        pos += n
        return data[pos - n:pos]

    if take(8) != CHECKPOINT_MAGIC:
        raise _refuse("read_prefix: not an OJAS0001 checkpoint")
    (version,) = struct.unpack("<I", take(4))
    if version != CHECKPOINT_VERSION:
        raise _refuse(f"read_prefix: version {version}, this reader takes {CHECKPOINT_VERSION}")
    take_lp = lambda: take(struct.unpack("<Q", take(8))[0])
    config = take_lp()
    tokenizer_hash, git_sha = take(32), take(20)
    step, shard, token_index = struct.unpack("<QQQ", take(24))
    rng_state = take_lp()
    for what in ("weights", "muon_momentum", "adamw_first_moment", "adamw_second_moment"):
        body, count = struct.unpack("<QQ", take(16))
        if body != 8 or count != 0:
            raise _refuse(f"{what}: the trainer's state file keeps its tensors in the safetensors files; this section holds {count} records")
    if pos != len(data):
        raise _refuse("trailing bytes after the last section")
    return {"config": config, "tokenizer_hash": tokenizer_hash, "git_sha": git_sha, "step": step, "cursor": DataCursor(shard, token_index), "rng_state": rng_state}


def parse_state_config(config: bytes) -> dict:
    """Exactly the four string keys of state_config, format ojas-train-v1 and a well-formed run id (checkpoint.rs:265-289)."""
    try:
        d = json.loads(config.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise _refuse(f"state config: {e}") from None
    if not isinstance(d, dict) or sorted(d) != ["format", "run", "spec", "train"] or not all(isinstance(v, str) for v in d.values()):
        raise _refuse("state config: expected exactly the string keys format, run, spec, train")
    if d["format"] != STATE_FORMAT:
        raise _refuse(f"state format {d['format']!r}, expected {STATE_FORMAT!r}")
    if not is_run_id(d["run"]):
        raise _refuse(f"run id {d['run']!r} is not 16 lowercase hex digits")
    return d


# ------------------------------------------------------------------------------------------------ the directory
def moment_names(info, hybrid: bool) -> list[str]:
    """checkpoint.rs:225-243: nothing for a frozen parameter, muon.<name> for a Muon matrix, adam_m / adam_v otherwise."""
    if not info.trains:
        return []
    if hybrid and info.group == "muon":
        return [f"muon.{info.name}"]
    return [f"adam_m.{info.name}", f"adam_v.{info.name}"]


def _check_save_target(path: Path) -> None:
    """An existing target is replaced only when it is empty or an earlier checkpoint (checkpoint.rs:9-13)."""
    if not path.exists():
        return
    if path.is_symlink() or not path.is_dir():
        raise _refuse(f"{path}: not a directory; nothing was written")
    names = {p.name for p in path.iterdir()} - {".DS_Store"}
    if names and names != {MODEL_FILE, OPTIM_FILE, STATE_FILE}:
        raise _refuse(f"{path}: holds {sorted(names)}, which is neither empty nor a checkpoint; nothing was written")


def save(trainer, directory, run_cfg: RunConfig, cursor: DataCursor, run: str) -> None:
    """Trainer::save (checkpoint.rs:527-690) for the C++ step driver: free-space check, three files in a staging directory
    beside the target, then the swap. `run` is the run id fixed when training began (compute_run_id)."""
    directory = Path(directory)
    if not is_run_id(run):
        raise _refuse(f"run id {run!r} is not 16 lowercase hex digits")
    hybrid = trainer.config.optimizer != "adamw"
    step = trainer.steps_done
    spec_text, train_text = spec_json(trainer.spec), run_cfg.to_json()
    model = [(p.name, p.shape) for p in trainer.params]
    optim, source = [], []
    for i, p in enumerate(trainer.params):
        for slot, name in enumerate(moment_names(p, hybrid)):
            optim.append((name, p.shape))
            source.append((i, slot))
    model_meta = [(SPEC_METADATA_KEY, spec_text), (STEP_METADATA_KEY, str(step)), (RUN_METADATA_KEY, run)]
    optim_meta = [(STEP_METADATA_KEY, str(step)), (RUN_METADATA_KEY, run)]
    state = encode_state(state_config(run, spec_text, train_text).encode(), run_cfg.tokenizer_hash, run_cfg.git_sha, step, cursor,
                         SamplerRngState(run_cfg.data_seed).encode())
    # every byte is new space (the old checkpoint stays until the swap); 1 MiB per file for block rounding
    need = sum(8 + len(h) + n + (1 << 20) for h, n in (safetensors_header(model, model_meta), safetensors_header(optim, optim_meta))) + len(state) + (1 << 20)
    parent = directory.resolve().parent
    recover_replaced_dir(directory)      # an earlier save of this name may have died mid-swap
    _check_save_target(directory)
    try:
        st = os.statvfs(parent)
        have = st.f_bavail * st.f_frsize
    except OSError as e:
        raise _refuse(f"{parent}: free disk space could not be read ({e}); nothing was written") from None
    if have < need:
        raise _refuse(f"{parent}: the checkpoint needs {need} bytes, {have} are free; nothing was written")
    stage = parent / f".{directory.name}.stage-{os.getpid()}"
    if stage.exists():
        shutil.rmtree(stage)
    stage.mkdir()
    try:
        write_safetensors(stage / MODEL_FILE, model, model_meta, trainer.get_param)
        write_safetensors(stage / OPTIM_FILE, optim, optim_meta, lambda j: trainer.get_moment(*source[j]))
        with open(stage / STATE_FILE, "xb") as f:
            f.write(state)
            f.flush()
            os.fsync(f.fileno())
        old = parent / f".{directory.name}.old-{os.getpid()}"
        if directory.exists():
            os.rename(directory, old)
        os.rename(stage, directory)
        if old.exists():
            shutil.rmtree(old)
    except BaseException:
        shutil.rmtree(stage, ignore_errors=True)
        raise


def recover_replaced_dir(directory) -> bool:
    """What a save that died between its two renames left behind (ojas_io::recover_replaced_dir, ojas-io/src/replace.rs:372-378, which
    Trainer::resume_from runs first, checkpoint.rs:699): the target was moved aside to `.<name>.old-<pid>` and the new directory never
    took its place. With the target missing, the newest such sibling is moved back; with the target present, leftovers of finished or
    abandoned saves (`.old-*`, and half-written `.stage-*` directories) are removed. The pid in the names is the dead process's, so
    the scan goes by prefix. Returns whether the old checkpoint was restored."""
    directory = Path(directory)
    parent = directory.resolve().parent
    if not parent.is_dir():
        return False
    olds = sorted((p for p in parent.glob(f".{directory.name}.old-*") if p.is_dir()), key=lambda p: p.stat().st_mtime)
    restored = False
    if not directory.exists() and olds:
        os.rename(olds.pop(), directory)
        restored = True
    for leftover in olds + [p for p in parent.glob(f".{directory.name}.stage-*") if p.is_dir()]:
        shutil.rmtree(leftover, ignore_errors=True)
    return restored


def resume(trainer, directory, run_cfg: RunConfig) -> tuple[DataCursor, str]:
    """Trainer::resume_from (checkpoint.rs:692-800) into an open trainer of the same spec: every check first, then the
    tensors, one at a time; returns the data cursor and the run id. `git_sha` may differ from the saved one; the train
    config and the tokenizer hash may not."""
    directory = Path(directory)
    recover_replaced_dir(directory)
    for name in (STATE_FILE, MODEL_FILE, OPTIM_FILE):
        f = directory / name
        if f.is_symlink() or not f.is_file():
            raise _refuse(f"{f}: not a regular file")
    if (directory / STATE_FILE).stat().st_size > MAX_STATE_BYTES:
        raise _refuse(f"{STATE_FILE}: larger than {MAX_STATE_BYTES} bytes")
    state = decode_state((directory / STATE_FILE).read_bytes())
    cfg = parse_state_config(state["config"])
    try:
        rng = SamplerRngState.decode(state["rng_state"])
    except DataError as e:
        raise _refuse(str(e)) from None
    if rng.seed != run_cfg.data_seed & _MASK64:
        raise _refuse(f"rng_state seed {rng.seed}, the config's data_seed is {run_cfg.data_seed}")
    if cfg["train"] != run_cfg.to_json():
        raise _refuse(f"the saved train config {cfg['train']} differs from the caller's {run_cfg.to_json()}")
    if state["tokenizer_hash"] != run_cfg.tokenizer_hash:
        raise _refuse("the saved tokenizer hash differs from the caller's")
    if cfg["spec"] != spec_json(trainer.spec):
        raise _refuse(f"the saved spec {cfg['spec']} differs from the trainer's {spec_json(trainer.spec)}")
    step, run = state["step"], cfg["run"]
    model, optim = SafeTensorsFile(directory / MODEL_FILE), SafeTensorsFile(directory / OPTIM_FILE)
    for what, f, want in (("model", model, {SPEC_METADATA_KEY: cfg["spec"], STEP_METADATA_KEY: str(step), RUN_METADATA_KEY: run}),
                          ("optim", optim, {STEP_METADATA_KEY: str(step), RUN_METADATA_KEY: run})):
        if f.metadata != want:
            raise _refuse(f"{what}: metadata {f.metadata} disagrees with the state file ({want})")
    hybrid = trainer.config.optimizer != "adamw"
    expect_model = [(p.name, list(p.shape)) for p in trainer.params]
    expect_optim, target = [], []
    for i, p in enumerate(trainer.params):
        for slot, name in enumerate(moment_names(p, hybrid)):
            expect_optim.append((name, list(p.shape)))
            target.append((i, slot))
    for what, f, expect in (("model", model, expect_model), ("optim", optim, expect_optim)):
        found = [(n, t["shape"]) for n, t in f.tensors.items()]
        if found != expect or any(t["dtype"] != "F32" for t in f.tensors.values()):
            bad = next((a for a, b in zip(found, expect) if a != b), found[len(expect):] or expect[len(found):])
            raise CheckpointError("Shape", f"{what}: tensors differ from the parameter table (first difference {bad})")
    for i, p in enumerate(trainer.params):
        trainer.set_param(i, model.read(p.name))
    for (i, slot), (name, _) in zip(target, expect_optim):
        trainer.set_moment(i, slot, optim.read(name))
    trainer.steps_done = step
    return state["cursor"], run
