"""The checkpoint directory (model.safetensors + optim.safetensors + state.ojck): byte layouts against the reference's
writers (ojas-io/src/safetensors.rs:1305-1398, ojas-io/src/checkpoint.rs:170-185, ojas-model/src/checkpoint.rs), the
refusals of save and resume, and on the GPU the bitwise-resume gate (ojas-model/tests/checkpoint.rs:178: N steps, a save,
a resume into a fresh trainer and N more equal 2N uninterrupted steps, bit for bit).
"""
import json
import struct
from dataclasses import dataclass

import numpy as np
import pytest

from ojas_b200 import checkpoint as ck
from ojas_b200.data import DataCursor, SamplerRngState


def test_floats_print_as_rusts_debug_form():
    # shortest round-trip digits; plain decimal with at least one fractional digit inside [1e-4, 1e16), d.ddde-N outside
    for x, want in [(10000.0, "10000.0"), (1e-6, "1e-6"), (6e-4, "0.0006"), (0.025, "0.025"), (0.95, "0.95"), (1.0, "1.0"), (0.0, "0.0"),
                    (1e16, "1e16"), (1e15, "1000000000000000.0"), (1e-4, "0.0001"), (9.9e-5, "9.9e-5"), (1.5e-7, "1.5e-7"), (123456.789, "123456.789"),
                    (-2.5, "-2.5"), (0.1 + 0.2, "0.30000000000000004")]:
        assert ck.rust_float(x) == want, (x, ck.rust_float(x))
    for x, want in [(1.0, "1.0"), (0.1, "0.1"), (3.4028235e38, "3.4028235e38"), (1e-5, "1e-5"), (0.3, "0.3"), (16777216.0, "16777216.0")]:
        assert ck.rust_f32(x) == want, (x, ck.rust_f32(x))


def test_spec_and_train_config_texts_are_the_references():
    from ojas_b200 import ModelSpec
    spec = ModelSpec.nanolab_124m()
    text = ck.spec_json(spec)
    assert text == ('{"format":"ojas-spec-v1","arch":"nanolab-gpt","vocab":50304,"n_embd":768,"n_layer":12,"n_head":12,"n_kv_head":12,"head_dim":64,'
                    '"hidden":2048,"max_seq":1024,"rope_base":10000.0,"rms_eps":1e-6,"tie_embeddings":true,"qk_norm":true,"gated_attention":true,'
                    '"value_residual":true}')
    assert ck.spec_from_json(text) == spec
    windowed = ModelSpec(vocab=256, n_embd=64, n_layer=2, n_head=4, n_kv_head=2, head_dim=16, hidden=192, max_seq=32, window=8)
    assert ck.spec_json(windowed).startswith('{"format":"ojas-spec-v2"') and ck.spec_json(windowed).endswith(',"value_residual":true,"window":8}')
    assert ck.spec_from_json(ck.spec_json(windowed)) == windowed
    # sorted keys; autocast and muon_ns5 only appear when they are not the default (trainer.rs:188-198)
    plain = ck.RunConfig(batch=2, seq_len=32, data_seed=7, total_steps=40, warmup_steps=4, ignore_index=5).to_json()
    assert plain == ('{"accum":1,"adam_lr":0.0006,"batch":2,"chunk_cols":8192,"chunk_rows":1024,"data_seed":7,"decay_frac":0.0,"grad_clip":1.0,"ignore":true,'
                     '"ignore_index":5,"matrix_lr":0.025,"on_nonfinite":"abort","schedule":"cosine","seq_len":32,"total_steps":40,"warmup_steps":4}')
    both = ck.RunConfig(batch=2, seq_len=32, autocast_bf16=True, muon_ns5_bf16=True, schedule="wsd", decay_frac=0.2).to_json()
    assert '"adam_lr":0.0006,"autocast":"bf16","batch":2' in both and '"matrix_lr":0.025,"muon_ns5":"bf16","on_nonfinite"' in both and '"decay_frac":0.2' in both
    assert json.loads(both)["schedule"] == "wsd"


def test_the_oracle_fixtures_spec_text_parses(golden_dir):
    f = ck.SafeTensorsFile(golden_dir / "tiny" / "init.safetensors")      # written by the python safetensors package, spaces and all
    spec = ck.spec_from_json(f.metadata["ojas.spec"])
    assert (spec.vocab, spec.n_embd, spec.n_layer, spec.head_dim, spec.hidden) == (256, 64, 2, 16, 192)
    from safetensors import safe_open
    ref = safe_open(str(golden_dir / "tiny" / "init.safetensors"), "np")
    for name in list(f.tensors)[:5]:
        assert np.array_equal(f.read(name), ref.get_tensor(name))


def test_safetensors_bytes_are_the_reference_writers(tmp_path):
    a, b = np.arange(6, dtype=np.float32).reshape(2, 3), np.array([1.5], np.float32)
    path = tmp_path / "x.safetensors"
    ck.write_safetensors(path, [("w.a", (2, 3)), ("b", (1,))], [("ojas.step", "3"), ("ojas.run", "00000000000000ff")], lambda i: (a, b)[i])
    header = ('{"__metadata__":{"ojas.step":"3","ojas.run":"00000000000000ff"},"w.a":{"dtype":"F32","shape":[2,3],"data_offsets":[0,24]},'
              '"b":{"dtype":"F32","shape":[1],"data_offsets":[24,28]}}').encode()
    header += b" " * (-len(header) % 8)
    assert path.read_bytes() == struct.pack("<Q", len(header)) + header + a.tobytes() + b.tobytes()
    from safetensors import safe_open           # an independent reader agrees
    f = safe_open(str(path), "np")
    assert np.array_equal(f.get_tensor("w.a"), a) and np.array_equal(f.get_tensor("b"), b) and f.metadata() == {"ojas.step": "3", "ojas.run": "00000000000000ff"}
    with pytest.raises(ck.CheckpointError):
        ck.safetensors_header([("a", (1,)), ("a", (1,))], [])
    with pytest.raises(ck.CheckpointError):
        ck.safetensors_header([("__metadata__", (1,))], [])


def test_state_file_layout_and_refusals():
    cfg = ck.state_config("0123456789abcdef", '{"a":1}', '{"b":"x"}').encode()
    assert cfg == b'{"format":"ojas-train-v1","run":"0123456789abcdef","spec":"{\\"a\\":1}","train":"{\\"b\\":\\"x\\"}"}'
    rng = SamplerRngState(9).encode()
    assert rng == struct.pack("<IIQ", 1, 1, 9)
    blob = ck.encode_state(cfg, bytes(range(32)), bytes(range(20)), 20, DataCursor(1, 5), rng)
    want = (b"OJAS0001" + struct.pack("<I", 1) + struct.pack("<Q", len(cfg)) + cfg + bytes(range(32)) + bytes(range(20)) + struct.pack("<QQQ", 20, 1, 5) +
            struct.pack("<Q", 16) + rng + struct.pack("<QQ", 8, 0) * 4)
    assert blob == want
    got = ck.decode_state(blob)
    assert got["step"] == 20 and got["cursor"] == DataCursor(1, 5) and got["rng_state"] == rng and got["tokenizer_hash"] == bytes(range(32))
    assert ck.parse_state_config(got["config"])["run"] == "0123456789abcdef"
    for bad in (b"OJAS0002" + blob[8:], blob[:8] + struct.pack("<I", 2) + blob[12:], blob[:-1], blob + b"\0", blob[:40],
                blob[:-16] + struct.pack("<QQ", 8, 1)):
        with pytest.raises(ck.CheckpointError):
            ck.decode_state(bad)
    for bad in (b'{"format":"ojas-train-v1","run":"xyz","spec":"","train":""}', b'{"format":"other","run":"0123456789abcdef","spec":"","train":""}',
                b'{"format":"ojas-train-v1","run":"0123456789abcdef","spec":""}', b"not json"):
        with pytest.raises(ck.CheckpointError):
            ck.parse_state_config(bad)


def test_run_id_is_fnv1a_over_texts_and_parameter_bytes():
    assert ck._fnv1a(b"") == 0xCBF29CE484222325 and ck._fnv1a(b"a") == 0xAF63DC4C8601EC8C and ck._fnv1a(b"foobar") == 0x85944171F73967E8
    params = [np.array([1.0, -2.0], np.float32), np.array([[0.5]], np.float32)]
    h = ck._fnv1a(b"ojas-run-v1\0")
    for t in ("S", "T"):
        h = ck._fnv1a(t.encode() + b"\0", h)
    for p in params:
        h = ck._fnv1a(p.tobytes(), h)
    assert ck.compute_run_id("S", "T", params) == "%016x" % h and ck.is_run_id("%016x" % h)


# ---- save / resume against a host stand-in for the trainer (the directory logic needs no device)
@dataclass
class _Info:
    name: str
    shape: tuple
    group: str
    trains: bool


class _Config:
    optimizer = "muon"


class HostTrainer:
    def __init__(self, spec, seed=0):
        rng = np.random.default_rng(seed)
        self.spec, self.config, self.steps_done = spec, _Config(), 0
        self.params = [_Info("tok_emb.weight", (8, 4), "adamw", True), _Info("blocks.0.mixer.q_proj.weight", (4, 4), "muon", True),
                       _Info("blocks.0.mixer.vr_lambda", (1,), "adamw", False), _Info("norm_f.weight", (4,), "adamw", True)]
        self.w = [rng.standard_normal(p.shape).astype(np.float32) for p in self.params]
        self.m = {(i, s): rng.standard_normal(p.shape).astype(np.float32) for i, p in enumerate(self.params) for s in range(len(ck.moment_names(p, True)))}

    def get_param(self, i): return self.w[i]
    def get_moment(self, i, s): return self.m[(i, s)]
    def set_param(self, i, v): self.w[i] = np.array(v)
    def set_moment(self, i, s, v): self.m[(i, s)] = np.array(v)


@pytest.fixture
def host_pair():
    from ojas_b200 import ModelSpec
    spec = ModelSpec(vocab=8, n_embd=4, n_layer=1, n_head=1, n_kv_head=1, head_dim=4, hidden=8, max_seq=8)
    return HostTrainer(spec, 1), HostTrainer(spec, 2), ck.RunConfig(batch=2, seq_len=8, data_seed=11, tokenizer_hash=bytes([7]) * 32)


def test_save_then_resume_restores_every_tensor_the_step_and_the_cursor(tmp_path, host_pair):
    src, dst, cfg = host_pair
    src.steps_done = 20
    run = ck.compute_run_id(ck.spec_json(src.spec), cfg.to_json(), src.w)
    target = tmp_path / "ckpt"
    ck.save(src, target, cfg, DataCursor(2, 9), run)
    assert sorted(p.name for p in target.iterdir()) == [ck.MODEL_FILE, ck.OPTIM_FILE, ck.STATE_FILE]
    optim = ck.SafeTensorsFile(target / ck.OPTIM_FILE)
    assert list(optim.tensors) == ["adam_m.tok_emb.weight", "adam_v.tok_emb.weight", "muon.blocks.0.mixer.q_proj.weight", "adam_m.norm_f.weight", "adam_v.norm_f.weight"]
    assert optim.metadata == {"ojas.step": "20", "ojas.run": run}
    cursor, got_run = ck.resume(dst, target, cfg)
    assert cursor == DataCursor(2, 9) and got_run == run and dst.steps_done == 20
    assert all(np.array_equal(a, b) for a, b in zip(src.w, dst.w)) and all(np.array_equal(src.m[k], dst.m[k]) for k in src.m)
    # a later save replaces an earlier checkpoint; no staging directory is left behind
    src.steps_done = 21
    ck.save(src, target, cfg, DataCursor(2, 10), run)
    assert ck.decode_state((target / ck.STATE_FILE).read_bytes())["step"] == 21 and [p.name for p in tmp_path.iterdir()] == ["ckpt"]


def test_a_save_that_died_between_its_two_renames_is_recovered(tmp_path, host_pair):
    """recover_replaced_dir (ojas-io/src/replace.rs:372-378): the old checkpoint was moved aside under another process's pid and the new
    one never took its place. resume finds it by prefix and moves it back; a later save sweeps every leftover."""
    import os
    src, dst, cfg = host_pair
    src.steps_done = 5
    run = ck.compute_run_id(ck.spec_json(src.spec), cfg.to_json(), src.w)
    target = tmp_path / "ckpt"
    ck.save(src, target, cfg, DataCursor(0, 3), run)
    os.rename(target, tmp_path / ".ckpt.old-424242")                 # the crash: first rename done, second never happened
    (tmp_path / ".ckpt.stage-424242").mkdir()                        # ... and the half-written new directory is still there
    (tmp_path / ".ckpt.stage-424242" / ck.MODEL_FILE).write_bytes(b"partial")
    cursor, got_run = ck.resume(dst, target, cfg)
    assert cursor == DataCursor(0, 3) and got_run == run and dst.steps_done == 5
    assert [p.name for p in tmp_path.iterdir()] == ["ckpt"]
    # with the target present, leftovers are swept and the checkpoint in place is the one that counts
    (tmp_path / ".ckpt.old-7").mkdir()
    assert ck.recover_replaced_dir(target) is False and [p.name for p in tmp_path.iterdir()] == ["ckpt"]
    # a save over a died swap restores first, then replaces
    os.rename(target, tmp_path / ".ckpt.old-99")
    src.steps_done = 6
    ck.save(src, target, cfg, DataCursor(0, 4), run)
    assert ck.decode_state((target / ck.STATE_FILE).read_bytes())["step"] == 6 and [p.name for p in tmp_path.iterdir()] == ["ckpt"]


def test_save_and_resume_refusals_leave_things_untouched(tmp_path, host_pair):
    src, dst, cfg = host_pair
    run = "00000000000000aa"
    foreign = tmp_path / "notes"
    foreign.mkdir()
    (foreign / "keep.txt").write_text("mine")
    with pytest.raises(ck.CheckpointError):
        ck.save(src, foreign, cfg, DataCursor(), run)
    assert [p.name for p in foreign.iterdir()] == ["keep.txt"] and [p.name for p in tmp_path.iterdir()] == ["notes"]
    with pytest.raises(ck.CheckpointError):
        ck.save(src, tmp_path / "x", cfg, DataCursor(), "not-a-run-id")
    target = tmp_path / "ckpt"
    ck.save(src, target, cfg, DataCursor(0, 3), run)
    before = [w.copy() for w in dst.w]
    from dataclasses import replace
    for other in (replace(cfg, data_seed=12), replace(cfg, batch=4), replace(cfg, tokenizer_hash=bytes(32))):
        with pytest.raises(ck.CheckpointError):
            ck.resume(dst, target, other)
    assert ck.resume(HostTrainer(src.spec, 5), target, replace(cfg, git_sha=bytes([1]) * 20))[0] == DataCursor(0, 3)     # git_sha may differ
    # the three files must agree on the step
    state = (target / ck.STATE_FILE).read_bytes()
    d = ck.decode_state(state)
    (target / ck.STATE_FILE).write_bytes(ck.encode_state(d["config"], d["tokenizer_hash"], d["git_sha"], d["step"] + 1, d["cursor"], d["rng_state"]))
    with pytest.raises(ck.CheckpointError):
        ck.resume(dst, target, cfg)
    (target / ck.STATE_FILE).write_bytes(state)
    # a trainer with another parameter table refuses before it writes anything
    dst.params[1] = _Info("blocks.0.mixer.q_proj.weight", (4, 8), "muon", True)
    with pytest.raises(ck.CheckpointError) as e:
        ck.resume(dst, target, cfg)
    assert e.value.kind == "Shape" and all(np.array_equal(a, b) for a, b in zip(before, dst.w))


# ---- the bitwise-resume gate on the device
@pytest.mark.gpu
@pytest.mark.parametrize("autocast", [False, True])
def test_steps_save_resume_steps_equal_uninterrupted_steps_bit_for_bit(tmp_path, golden_dir, autocast):
    from safetensors import safe_open
    from ojas_b200 import CudaBackend, TrainConfig, Trainer
    f = safe_open(str(golden_dir / "tiny" / "init.safetensors"), "np")
    spec = ck.spec_from_json(f.metadata()["ojas.spec"])
    weights = {k: f.get_tensor(k) for k in f.keys()}
    B, T, N = 2, 32, 4
    rng = np.random.default_rng(3)
    batches = [rng.integers(0, spec.vocab, (B, T + 1), dtype=np.uint32) for _ in range(2 * N)]
    cfg = ck.RunConfig(batch=B, seq_len=T, data_seed=5, autocast_bf16=autocast, muon_ns5_bf16=autocast)
    be = CudaBackend(0, 8 << 30)

    def fresh():
        tr = Trainer(be, spec, TrainConfig(optimizer="muon", autocast_bf16=autocast, ns5_bf16=autocast), B, T)
        tr.set_params([weights[p.name] for p in tr.params])
        return tr

    def run_steps(tr, lo, hi):
        return [tr.step(b[:, :-1], b[:, 1:]).loss for b in batches[lo:hi]]

    def snapshot(tr):
        hybrid = True
        return [tr.get_param(i) for i in range(len(tr.params))] + [tr.get_moment(i, s) for i, p in enumerate(tr.params) for s in range(len(ck.moment_names(p, hybrid)))]

    try:
        whole = fresh()
        losses_whole = run_steps(whole, 0, 2 * N)
        want = snapshot(whole)
        whole.close()

        first = fresh()
        run = ck.compute_run_id(ck.spec_json(spec), cfg.to_json(), [weights[p.name] for p in first.params])
        losses_a = run_steps(first, 0, N)
        ck.save(first, tmp_path / "ckpt", cfg, DataCursor(0, N), run)
        first.close()                                   # the trainer is dropped; only the directory carries the state over

        second = fresh()
        cursor, got_run = ck.resume(second, tmp_path / "ckpt", cfg)
        assert cursor == DataCursor(0, N) and got_run == run and second.steps_done == N
        losses_b = run_steps(second, N, 2 * N)
        got = snapshot(second)
        second.close()
    finally:
        be.close()
    assert losses_a + losses_b == losses_whole
    assert len(got) == len(want) and all(a.tobytes() == b.tobytes() for a, b in zip(got, want))
