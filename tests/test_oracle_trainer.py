"""Pins the oracle's restatement of the trainer's host logic (schedule, micro-batch weights, accumulation, clip, hybrid
optimizer) to the reference's own fixtures: the nanolab schedule multipliers (ojas-oracle/fixtures/tiny/lr_schedules.json,
gate LR_MULT_REL_TOL 1e-12), the sampler's window starts of the 40-step trace (batch_starts.json, exact) and the torch traces
themselves (trace_ns5_{f32,bf16}.safetensors) under the gates of ojas-oracle/src/parity.rs:29-74 for CpuBackend (Exact)."""
import json
import math

import numpy as np
import pytest
from safetensors import safe_open

from oracle import oracle as orc
from ojas_b200.data import BatchSampler, TokenBin

TRACE_LOSS_ABS, TRACE_PARAM, TRACE_BF16_PARAM = 1e-4, 1e-4, 5e-2     # parity.rs:36-51
CURVE_EARLY_ABS, CURVE_EARLY_STEPS, CURVE_LATE_ABS, CURVE_MIN_DROP = 2e-4, 10, 2e-3, 1.0   # parity.rs:53-58
GRAD_NORM_REL = 1e-4                                                 # ojas-model/tests/oracle_parity.rs:391-400


def load(path):
    f = safe_open(str(path), "np")
    return {k: f.get_tensor(k) for k in f.keys()}, f.metadata()


def tiny(golden_dir):
    init, meta = load(golden_dir / "tiny/init.safetensors")
    s = json.loads(meta["ojas.spec"])
    spec = orc.Spec(**{k: s[k] for k in ("vocab", "n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "hidden", "max_seq", "rope_base", "rms_eps")})
    return spec, init


def trace_setup(golden_dir, ns5):
    want, meta = load(golden_dir / f"tiny/trace_ns5_{ns5}.safetensors")
    info = json.loads(meta["ojas.oracle"])
    return want, info, info["config"]


def trace_batches(golden_dir, cfg, steps):
    bin_ = TokenBin.open(golden_dir / "tiny/tokens.bin")
    sampler = BatchSampler(len(bin_), cfg["block_size"], cfg["batch_size"], cfg["seed"])
    return [[sampler.next_batch(bin_) for _ in range(cfg["grad_accum"])] for _ in range(steps)]


@pytest.mark.parametrize("name", ["acceptance_cosine", "acceptance_wsd", "tiny_cosine", "tiny_wsd"])
def test_schedule_multipliers_match_nanolab(golden_dir, name):
    s = json.loads((golden_dir / "tiny/lr_schedules.json").read_text())[name]
    for step, want in enumerate(s["multipliers"]):
        got = orc.lr_multiplier(s["schedule"], s["warmup_steps"], s["total_steps"], step, s["wsd_decay_frac"])
        assert abs(got - want) <= 1e-12 * abs(want), (name, step, got, want)


def test_schedule_edges():
    # warmup 0 runs the decay branch from the first step, whose multiplier at t = 0 is 1 (schedule.rs:17-22)
    assert orc.lr_multiplier("cosine", 0, 10, 0) == 1.0
    assert orc.lr_multiplier("cosine", 0, 10, 10) == pytest.approx(0.1, abs=1e-15)
    assert orc.lr_multiplier("cosine", 0, 10, 500) == pytest.approx(0.1, abs=1e-15)     # clamped past the end
    assert orc.lr_multiplier("wsd", 2, 10, 7) == 1.0 and orc.lr_multiplier("wsd", 2, 10, 10) == pytest.approx(0.1, abs=1e-15)
    with pytest.raises(orc.OracleError):
        orc.lr_multiplier("wsd", 2, 10, 11)                                             # a step past the schedule is refused


def test_micro_weights():
    w, uniform, run = orc.micro_weights([64, 64])
    assert uniform and run == 2 and w == [np.float32(0.5)] * 2
    w, uniform, run = orc.micro_weights([64, 0, 64, 64])                               # an all-ignored micro-batch weighs nothing
    assert uniform and run == 3 and w[1] == 0 and w[0] == np.float32(1.0) / np.float32(3)
    w, uniform, run = orc.micro_weights([10, 30])
    assert not uniform and w == [np.float32(0.25), np.float32(0.75)]
    with pytest.raises(orc.OracleError):
        orc.micro_weights([0, 0])


def test_sampler_reads_the_trace_batches(golden_dir):
    want = json.loads((golden_dir / "tiny/batch_starts.json").read_text())
    bin_ = TokenBin.open(golden_dir / "tiny/tokens.bin")
    assert len(bin_) == want["bin_tokens"]
    s = BatchSampler(len(bin_), want["seq_len"], want["batch"], want["seed"])
    assert s.windows_per_epoch() == want["windows_per_epoch"]
    starts = np.concatenate([s.next_starts() for _ in range(want["steps"] * want["accum"])])
    assert starts.tolist() == want["starts"]
    c = s.cursor()
    assert [c.shard, c.token_index] == want["cursor_after"]


@pytest.mark.parametrize("ns5", ["f32", "bf16"])
def test_forty_step_trace_matches_torch(golden_dir, ns5):
    spec, init = tiny(golden_dir)
    want, info, cfg = trace_setup(golden_dir, ns5)
    table = orc.param_table(spec)
    tr = orc.TrainerOracle(spec, [init[i.name] for i in table], schedule=(cfg["schedule"], cfg["warmup_steps"], cfg["lr_max_steps"] or cfg["max_steps"], cfg["wsd_decay_frac"]),
                           matrix_lr=cfg["matrix_lr"], adam_lr=cfg["lr"], grad_clip=cfg["grad_clip"], ns5_bf16=ns5 == "bf16", muon_momentum=cfg["muon_momentum"])
    last = None
    for step, batches in enumerate(trace_batches(golden_dir, cfg, info["steps"])):
        loss, norm, mult = tr.run(batches)
        d = abs(loss - info["mean_loss"][step])
        if step < info["params_after_step"]:
            assert d <= TRACE_LOSS_ABS, (step, d)
            assert abs(norm - info["grad_norm"][step]) <= GRAD_NORM_REL * info["grad_norm"][step], step
        assert d <= (CURVE_EARLY_ABS if step < CURVE_EARLY_STEPS else CURVE_LATE_ABS), (step, d)
        assert abs(mult - info["lr_mult"][step]) <= 1e-12 * abs(info["lr_mult"][step]), step
        if step + 1 == info["params_after_step"]:
            tol = TRACE_PARAM if ns5 == "f32" else TRACE_BF16_PARAM
            for p, i in zip(tr.params, table):
                w = want[i.name].astype(np.float64)
                if not np.any(w):
                    assert not np.any(p), i.name
                else:
                    assert np.linalg.norm(p - w) / np.linalg.norm(w) <= tol, i.name
        last = loss
    assert math.log(spec.vocab) - last >= CURVE_MIN_DROP


def test_a_non_finite_gradient_changes_nothing(golden_dir):
    spec, init = tiny(golden_dir)
    table = orc.param_table(spec)
    params = [init[i.name].copy() for i in table]
    params[1][0] = np.nan                                    # the first block's norm weight
    tr = orc.TrainerOracle(spec, params)
    before = [p.copy() for p in tr.params]
    _, _, cfg = trace_setup(golden_dir, "f32")
    with pytest.raises(orc.OracleError):
        tr.run(trace_batches(golden_dir, cfg, 1)[0])
    assert tr.step == 0 and all(a.tobytes() == b.tobytes() for a, b in zip(before, tr.params))
