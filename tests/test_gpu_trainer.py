"""Whole-step parity of the C++ step driver: against the reference's torch goldens (tests/golden) and against the CPU
oracle on BASELINE config 1 (tiny GPT, one full AdamW step, f32), plus the bf16-autocast tolerance of the north star.

Gates (ojas-oracle/src/parity.rs:29-45 and the north star): f32 mode loss 1e-5 relative, every gradient 1e-4 normwise
(exactly zero where the golden is zero); bf16 autocast loss within 1e-2 relative after one step.
"""
import json

import numpy as np
import pytest
from safetensors import safe_open

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

LOSS_TOL, LOGITS_TOL, GRAD_TOL = 1e-5, 1e-5, 1e-4


@pytest.fixture(scope="module")
def be():
    from ojas_b200 import CudaBackend
    backend = CudaBackend(0, 64 << 30)
    yield backend
    backend.close()


def load(path, prefix=""):
    f = safe_open(str(path), "np")
    return {k[len(prefix):]: f.get_tensor(k) for k in f.keys() if k.startswith(prefix)}, f.metadata()


def spec_pair(meta):
    from ojas_b200 import ModelSpec
    s = json.loads(meta["ojas.spec"])
    kw = dict(vocab=s["vocab"], n_embd=s["n_embd"], n_layer=s["n_layer"], n_head=s["n_head"], n_kv_head=s["n_kv_head"], head_dim=s["head_dim"],
              hidden=s["hidden"], max_seq=s["max_seq"], window=s.get("window"), rope_base=s["rope_base"], rms_eps=s["rms_eps"])
    return ModelSpec(**kw), orc.Spec(**kw)


def normwise(got, want):
    got, want = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    return np.linalg.norm(got - want) / np.linalg.norm(want)


def make_trainer(be, spec, params_by_name, batch, seq, **cfg):
    from ojas_b200 import TrainConfig, Trainer
    tr = Trainer(be, spec, TrainConfig(**cfg), batch, seq)
    tr.set_params([params_by_name[p.name] for p in tr.params])
    return tr


def check_grads(tr, want, no_grad, tol=GRAD_TOL):
    for i, p in enumerate(tr.params):
        if p.name in no_grad:
            assert not p.trains
            continue
        g, w = tr.get_grad(i), want[p.name]
        if not np.any(w):
            assert not np.any(g), p.name
        else:
            assert normwise(g, w) <= tol, (p.name, normwise(g, w))


def test_tiny_forward_and_gradients_match_the_torch_goldens(be, golden_dir):
    params, meta = load(golden_dir / "tiny/init.safetensors")
    spec, _ = spec_pair(meta)
    fwd, fmeta = load(golden_dir / "tiny/forward.safetensors")
    want_loss = float(np.uint32(json.loads(fmeta["ojas.oracle"])["loss_f32_bits"]).view(np.float32))
    for which in ("grads_init", "grads_step5"):
        want, gmeta = load(golden_dir / f"tiny/{which}.safetensors")
        gmeta = json.loads(gmeta["ojas.oracle"])
        p = params if which == "grads_init" else load(golden_dir / "tiny/trace_ns5_f32.safetensors")[0]
        tr = make_trainer(be, spec, p, 2, 32, loss_seed=gmeta["loss_seed"], grad_clip=0.0)
        if which == "grads_init":
            logits = tr.logits(fwd["x"])
            assert normwise(logits.reshape(2, 32, 256), fwd["logits"]) <= LOGITS_TOL
        loss = tr.gradients(fwd["x"], fwd["y"])
        assert abs(loss - gmeta["loss"]) / gmeta["loss"] <= LOSS_TOL
        if which == "grads_init":
            assert abs(loss - want_loss) / want_loss <= LOSS_TOL
        check_grads(tr, want, gmeta["no_grad"])
        tr.close()


@pytest.mark.parametrize("variant", ["gqa", "swa"])
def test_gqa_and_sliding_window_variants(be, golden_dir, variant):
    path = golden_dir / f"variants/{variant}.safetensors"
    params, meta = load(path, "param/")
    grads, _ = load(path, "grad/")
    rest, _ = load(path)
    spec, _ = spec_pair(meta)
    info = json.loads(meta["ojas.oracle"])
    tr = make_trainer(be, spec, params, 2, 32, loss_seed=info["loss_seed"], grad_clip=0.0)
    assert normwise(tr.logits(rest["x"]).reshape(rest["logits"].shape), rest["logits"]) <= LOGITS_TOL
    loss = tr.gradients(rest["x"], rest["y"])
    assert abs(loss - info["loss"]) / info["loss"] <= LOSS_TOL
    check_grads(tr, grads, info["no_grad"])
    tr.close()


def config1():
    """BASELINE config 1: 4 layers, d 256, 4 x 64 heads, hidden 1024, V 4096, T 256, B 8; weights N(0, 0.02) from seed 0
    (every matrix, o_proj and ffn.down included); ids uniform from SplitMix64(1), targets = inputs shifted by one."""
    kw = dict(vocab=4096, n_embd=256, n_layer=4, n_head=4, n_kv_head=4, head_dim=64, hidden=1024, max_seq=256)
    ospec = orc.Spec(**kw)
    params = orc.init_params(ospec, 0, normal_everywhere=True)
    rng = orc.SplitMix64(1)
    b, t = 8, 256
    draws = np.array([rng.below(4096) for _ in range(b * (t + 1))], np.uint32).reshape(b, t + 1)
    return kw, ospec, params, draws[:, :-1].copy(), draws[:, 1:].copy()


@pytest.fixture(scope="module")
def c1():
    kw, ospec, params, x, y = config1()
    loss, grads, _ = orc.forward_loss(ospec, params, x, y)
    table = orc.param_table(ospec)
    stepped = []
    for info, p, g in zip(table, params, grads):
        q, m, v = p.copy().ravel(), np.zeros(p.size, np.float32), np.zeros(p.size, np.float32)
        if info.trains:
            orc.adamw_step(q, g.ravel(), m, v, 0, 3e-4, weight_decay=0.1)
        stepped.append(q.reshape(p.shape))
    return kw, params, x, y, loss, grads, stepped


def test_config1_one_full_adamw_step_f32(be, c1):
    from ojas_b200 import ModelSpec
    kw, params, x, y, oloss, ograds, ostepped = c1
    tr = make_trainer(be, ModelSpec(**kw), {p.name: v for p, v in zip(orc.param_table(orc.Spec(**kw)), params)}, 8, 256, optimizer="adamw", adam_lr=3e-4,
                      adam_weight_decay=0.1, grad_clip=0.0)
    loss = tr.gradients(x, y)
    assert abs(loss - oloss) / oloss <= LOSS_TOL, (loss, oloss)
    for i, p in enumerate(tr.params):
        if p.trains:
            assert normwise(tr.get_grad(i), ograds[i]) <= GRAD_TOL, (p.name, normwise(tr.get_grad(i), ograds[i]))
    before = be.device_readbacks()
    rep = tr.step(x, y)
    assert be.device_readbacks() == before + 1  # one readback per step (Budget::device_readbacks, trainer gate G10)
    assert abs(rep.loss - oloss) / oloss <= LOSS_TOL and rep.step == 1 and rep.tokens == 8 * 256
    assert abs(rep.grad_norm - float(orc.grad_norm(ograds))) <= 1e-5 * float(orc.grad_norm(ograds))
    for i, p in enumerate(tr.params):
        if not np.any(ostepped[i]):
            assert not np.any(tr.get_param(i)), p.name
            continue
        assert normwise(tr.get_param(i), ostepped[i]) <= 1e-4, p.name  # TRACE_PARAM_NORMWISE_REL_TOL, ojas-oracle/src/parity.rs:41-43
    tr.close()


def test_config1_bf16_autocast_loss_within_one_percent(be, c1):
    from ojas_b200 import ModelSpec
    kw, params, x, y, oloss, ograds, _ = c1
    tr = make_trainer(be, ModelSpec(**kw), {p.name: v for p, v in zip(orc.param_table(orc.Spec(**kw)), params)}, 8, 256, autocast_bf16=True, optimizer="adamw",
                      adam_lr=3e-4, adam_weight_decay=0.1, grad_clip=0.0)
    rep = tr.step(x, y)
    assert abs(rep.loss - oloss) / oloss <= 1e-2, (rep.loss, oloss)
    rep2 = tr.step(x, y)
    assert rep2.loss < rep.loss  # the step went downhill on the same batch
    tr.close()
    tr = make_trainer(be, ModelSpec(**kw), {p.name: v for p, v in zip(orc.param_table(orc.Spec(**kw)), params)}, 8, 256, autocast_bf16=True, grad_clip=0.0)
    tr.gradients(x, y)
    worst = max(normwise(tr.get_grad(i), ograds[i]) for i, p in enumerate(tr.params) if p.trains and len(p.shape) == 2)
    assert worst <= 5e-2, worst  # bf16 operands: a few 1e-3 per matrix is expected; a wrong kernel is off by O(1)
    tr.close()


def test_bf16_autocast_loss_curve_tracks_the_f32_oracle_over_200_steps(be):
    """North-star gate for bf16 autocast: the loss curve stays within 2% of the CPU reference's over 200 optimizer steps
    (same seed, same weights, same batches). A small model so the strict-order oracle runs 200 steps in well under a minute."""
    from ojas_b200 import ModelSpec
    kw = dict(vocab=512, n_embd=128, n_layer=2, n_head=2, n_kv_head=2, head_dim=64, hidden=256, max_seq=64)
    ospec = orc.Spec(**kw)
    params = [p.copy() for p in orc.init_params(ospec, 0, normal_everywhere=True)]
    table = orc.param_table(ospec)
    rng = orc.SplitMix64(7)
    b, t, nbatch, steps, lr = 4, 64, 16, 200, 1e-3
    draws = np.array([rng.below(512) for _ in range(nbatch * b * (t + 1))], np.uint32).reshape(nbatch, b, t + 1)
    tr = make_trainer(be, ModelSpec(**kw), {info.name: v for info, v in zip(table, params)}, b, t, autocast_bf16=True, optimizer="adamw", adam_lr=lr,
                      adam_weight_decay=0.1, grad_clip=1.0)
    moments = [(np.zeros(p.size, np.float32), np.zeros(p.size, np.float32)) for p in params]
    worst, first, last = 0.0, None, None
    for step in range(steps):
        x, y = draws[step % nbatch, :, :-1].copy(), draws[step % nbatch, :, 1:].copy()
        oloss, grads, _ = orc.forward_loss(ospec, params, x, y)
        norm = float(orc.grad_norm(grads))
        scale = min(1.0, 1.0 / (norm + 1e-6))
        for info, p, g, (m, v) in zip(table, params, grads, moments):
            if info.trains:
                flat = p.reshape(-1)
                orc.adamw_step(flat, (g.ravel() * np.float32(scale)).astype(np.float32) if scale < 1.0 else g.ravel(), m, v, step, lr, weight_decay=0.1)
        rep = tr.step(x, y)
        worst = max(worst, abs(rep.loss - oloss) / oloss)
        first = oloss if first is None else first
        last = oloss
    tr.close()
    assert last < 0.5 * first, (first, last)   # the curve actually moves: 6.25 -> about 1.7 (the batches repeat every 16 steps)
    assert worst <= 2e-2, worst


def test_muon_hybrid_step_matches_the_oracle_grouping(be, golden_dir):
    """Trainer semantics: Muon NS5 on rank-2 hidden weights, AdamW without decay on the embedding and vectors, clip 1.0."""
    params, _ = load(golden_dir / "tiny/trace_ns5_f32.safetensors")
    spec, ospec = spec_pair(load(golden_dir / "tiny/init.safetensors")[1])
    fwd, _ = load(golden_dir / "tiny/forward.safetensors")
    table = orc.param_table(ospec)
    plist = [params[i.name] for i in table]
    _, grads, _ = orc.forward_loss(ospec, plist, fwd["x"], fwd["y"])
    clipped = [g.copy() for g in grads]
    orc.clip_grad_norm(clipped, 1.0)
    want = []
    for info, p, g in zip(table, plist, clipped):
        q = p.copy()
        if not info.trains:
            pass
        elif info.group == 1:
            mom = np.zeros_like(q)
            orc.muon_ns5_step(q, g, mom, lr=0.025, momentum=0.95, weight_decay=0.1)
        else:
            flat, m, v = q.ravel(), np.zeros(q.size, np.float32), np.zeros(q.size, np.float32)
            orc.adamw_step(flat, g.ravel(), m, v, 0, 6e-4, weight_decay=0.0)
        want.append(q)
    tr = make_trainer(be, spec, params, 2, 32, optimizer="muon", muon_momentum=0.95, grad_clip=1.0)
    tr.step(fwd["x"], fwd["y"])
    for i, p in enumerate(tr.params):
        assert normwise(tr.get_param(i) - plist[i] + 1e-30, want[i] - plist[i] + 1e-30) <= 2e-3 or not p.trains, p.name
    tr.close()


def test_muon_bf16_groups_run_as_batched_tensor_core_products(be):
    """ns5 in bf16 on a model whose matrices are wide enough for the tcgen05 kernels: the step driver steps each shape group
    (8 of 128x128, 4 of 256x128 tall, 2 of 128x256) with batched products. Checked against the oracle's bf16 NS5 per matrix;
    the momentum buffer, formed before any product, is compared through the second step's update."""
    from ojas_b200 import ModelSpec
    kw = dict(vocab=512, n_embd=128, n_layer=2, n_head=2, n_kv_head=2, head_dim=64, hidden=256, max_seq=64)
    ospec = orc.Spec(**kw)
    table = orc.param_table(ospec)
    params = orc.init_params(ospec, 3, normal_everywhere=True)
    rng = orc.SplitMix64(11)
    b, t = 4, 64
    draws = np.array([rng.below(512) for _ in range(b * (t + 1))], np.uint32).reshape(b, t + 1)
    x, y = draws[:, :-1].copy(), draws[:, 1:].copy()
    _, grads, _ = orc.forward_loss(ospec, params, x, y)
    clipped = [g.copy() for g in grads]
    orc.clip_grad_norm(clipped, 1.0)
    want = []
    for info, p, g in zip(table, params, clipped):
        q = p.copy()
        if info.trains and info.group == 1:
            orc.muon_ns5_step(q, g, np.zeros_like(q), lr=0.025, momentum=0.95, weight_decay=0.1, bf16=True)
        elif info.trains:
            orc.adamw_step(q.reshape(-1), g.ravel(), np.zeros(q.size, np.float32), np.zeros(q.size, np.float32), 0, 6e-4, weight_decay=0.0)
        want.append(q)
    tr = make_trainer(be, ModelSpec(**kw), {i.name: v for i, v in zip(table, params)}, b, t, optimizer="muon", muon_momentum=0.95, ns5_bf16=True, grad_clip=1.0)
    tr.step(x, y)
    worst = 0.0
    for i, (info, p) in enumerate(zip(table, tr.params)):
        if not p.trains:
            continue
        err = normwise(tr.get_param(i) - params[i] + 1e-30, want[i] - params[i] + 1e-30)
        worst = max(worst, err) if info.group == 1 else worst
        assert err <= (3e-2 if info.group == 1 else 2e-3), (p.name, err)   # bf16 products: tensor-core vs strict summation order
    assert worst > 0.0
    tr.close()


@pytest.mark.parametrize("clip", [1.0, 0.0])
def test_weight_gradients_on_the_side_stream_are_the_same_bits(be, c1, clip):
    """Under bf16 autocast the weight-gradient GEMMs run on a second stream beside the dX chain. Same kernels, same split
    counts, only the stream differs: every gradient, the loss and the stepped parameters must equal the one-stream run bit for bit.
    Without clipping (clip 0) a one-call AdamW step also updates each block on that stream while backward is still running."""
    from ojas_b200 import ModelSpec
    kw, params, x, y, _, _, _ = c1
    by_name = {p.name: v for p, v in zip(orc.param_table(orc.Spec(**kw)), params)}
    runs = []
    for lane in (False, True):
        tr = make_trainer(be, ModelSpec(**kw), by_name, 8, 256, autocast_bf16=True, optimizer="adamw", adam_lr=3e-4, adam_weight_decay=0.1, grad_clip=clip)
        tr.overlap_weight_grads(lane)
        loss = tr.gradients(x, y)
        grads = [tr.get_grad(i).copy() for i in range(len(tr.params))]
        for _ in range(3):
            tr.step(x, y)
        state = [tr.get_param(i).copy() for i in range(len(tr.params))]
        state += [tr.get_moment(i, s_).copy() for i, p in enumerate(tr.params) if p.trains for s_ in (0, 1)]
        runs.append((loss, grads, state))
        tr.close()
    (l0, g0, p0), (l1, g1, p1) = runs
    assert l0 == l1
    for a, b in zip(g0, g1):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    for a, b in zip(p0, p1):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_out_of_range_token_is_refused_before_any_launch(be):
    from ojas_b200 import ModelSpec, OjasError, TrainConfig, Trainer
    spec = ModelSpec(vocab=64, n_embd=32, n_layer=1, n_head=2, n_kv_head=2, head_dim=16, hidden=64, max_seq=8)
    tr = Trainer(be, spec, TrainConfig(), 1, 8)
    ids = np.arange(8, dtype=np.uint32)
    ids[3] = 64
    launches = be.kernel_launches()
    with pytest.raises(OjasError) as e:
        tr.gradients(ids, ids)
    assert e.value.kind == "OutOfRange" and be.kernel_launches() == launches
    tr.close()


@pytest.mark.parametrize("autocast", [False, True])
def test_activation_checkpointing_recomputes_the_same_bits_in_less_memory(be, golden_dir, autocast):
    """ActivationCheckpoint::Blocks (ojas-model/src/block.rs:323-336): only block inputs are kept and each block is recomputed in
    backward. The kernels are deterministic, so losses, gradients and the stepped parameters equal the plain run bit for bit."""
    from ojas_b200 import ModelSpec, TrainConfig, Trainer
    spec = ModelSpec(vocab=512, n_embd=128, n_layer=5, n_head=2, n_kv_head=1, head_dim=64, hidden=256, max_seq=128)
    ospec = orc.Spec(vocab=512, n_embd=128, n_layer=5, n_head=2, n_kv_head=1, head_dim=64, hidden=256, max_seq=128)
    weights = orc.init_params(ospec, 3, normal_everywhere=True)
    rng = np.random.default_rng(8)
    batches = [rng.integers(0, 512, (4, 129), dtype=np.uint32) for _ in range(3)]
    runs = []
    for ckpt in (False, True):
        live_before = be.budget()["live"]
        tr = Trainer(be, spec, TrainConfig(optimizer="muon", autocast_bf16=autocast, ns5_bf16=autocast, checkpoint_blocks=ckpt), 4, 128)
        held = be.budget()["live"] - live_before
        tr.set_params(weights)
        losses = []
        for i, b in enumerate(batches):
            if i == 0:
                losses.append(tr.gradients(b[:, :-1], b[:, 1:]))
                grads = [tr.get_grad(j) for j, p in enumerate(tr.params) if p.trains]
                tr.apply()
            else:
                losses.append(tr.step(b[:, :-1], b[:, 1:]).loss)
        runs.append((losses, grads, [tr.get_param(j) for j in range(len(tr.params))], held))
        tr.close()
    (l0, g0, p0, m0), (l1, g1, p1, m1) = runs
    assert l0 == l1
    assert all(a.tobytes() == b.tobytes() for a, b in zip(g0, g1)) and all(a.tobytes() == b.tobytes() for a, b in zip(p0, p1))
    assert m1 < 0.85 * m0, (m0, m1)      # five blocks of activations became two plus five block inputs (the rest is parameters, moments, gradients)
