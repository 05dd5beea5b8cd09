"""Parity at the shapes the benchmark runs, against the CPU oracle:

* nanolab GPT-124M (ModelSpec::nanolab_124m, ojas-model/src/spec.rs:76-91: 12 layers, d 768, 12 x 64 heads, hidden 2048, vocab
  50304) at T 1024 with enough rows (B 9 = 9216) that the fused tied-head cross-entropy walks more than one of its default 8192-row
  tiles over the ragged 50304-column vocabulary: one step's loss and every gradient, f32 tier (1e-5 / 1e-4, the f32 gates of
  ojas-oracle/src/parity.rs:29-35) and bf16 autocast (loss 1e-2 relative, matrices 5e-2 normwise);
* the attention backward the bf16 step uses (Dr = dO . O from the saved bf16 output) against the form the reference's autocast asks
  for (ojas-core/src/autocast.rs:1200-1254: recompute the output) at the step's own T 1024, 12 x 64 heads;
* causal SDPA forward + backward at [B 8, H 16, T 4096, D 128] bf16 drawn N(0, 1): six (b, h) planes against the strict-order
  oracle at 2e-2 relative, and every row's lse and output plus every gradient plane against this library's f32 tier (itself held
  to 1e-5 / 1e-4 of the oracle in test_gpu_ops.py).
"""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def rel(got, want):
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    denom = np.linalg.norm(want)
    return np.linalg.norm(got - want) / (denom if denom > 0 else 1.0)


@pytest.fixture(scope="module")
def be():
    from ojas_b200 import CudaBackend
    backend = CudaBackend(0, 100 << 30)
    yield backend
    backend.close()


KW_124M = dict(vocab=50304, n_embd=768, n_layer=12, n_head=12, n_kv_head=12, head_dim=64, hidden=2048, max_seq=1024)
B_124M, T_124M = 9, 1024


@pytest.fixture(scope="module")
def oracle_124m():
    ospec = orc.Spec(**KW_124M)
    params = orc.init_params(ospec, 0, normal_everywhere=True)
    rng = orc.SplitMix64(1)
    draws = np.array([rng.below(KW_124M["vocab"]) for _ in range(B_124M * (T_124M + 1))], np.uint32).reshape(B_124M, T_124M + 1)
    x, y = draws[:, :-1].copy(), draws[:, 1:].copy()
    loss, grads, _ = orc.forward_loss(ospec, params, x, y)
    return params, x, y, float(loss), grads


@pytest.mark.parametrize("autocast", [False, True])
def test_nanolab_124m_one_step_loss_and_gradients(be, oracle_124m, autocast):
    from ojas_b200 import ModelSpec, TrainConfig, Trainer
    params, x, y, oloss, ograds = oracle_124m
    tr = Trainer(be, ModelSpec(**KW_124M), TrainConfig(autocast_bf16=autocast, optimizer="adamw", adam_lr=3e-4, adam_weight_decay=0.1, grad_clip=0.0), B_124M, T_124M)
    tr.set_params(params)
    loss = tr.gradients(x, y)
    loss_tol, grad_tol = (1e-2, 5e-2) if autocast else (1e-5, 1e-4)
    assert abs(loss - oloss) <= loss_tol * abs(oloss), (loss, oloss)
    worst = ("", 0.0)
    for i, p in enumerate(tr.params):
        if not p.trains:
            continue
        err = rel(tr.get_grad(i), ograds[i])
        if p.name.endswith("vr_lambda"):
            # one scalar: s(1-s) times a sum of 9216 x 768 products of mixed sign. The oracle adds them one after the other in f32
            # (ojas-cpu/src/pointwise.rs:2031-2146), the device in a tree; at this length the two f32 sums differ by the rounding
            # error either one carries (measured 4e-3 of the result: a condition number near 1e5), which a normwise gate on a single
            # number cannot absorb; under autocast the operands' bf16 rounding (4e-3 each) moves such a sum by more than its size, so
            # there the scalar is only required to be finite (its kernels are held to the oracle on small models in test_gpu_ops.py)
            assert np.isfinite(tr.get_grad(i)).all() and (autocast or err <= 2e-2), (p.name, err)
            continue
        if autocast and len(p.shape) < 2:
            assert err <= 1e-1, (p.name, err)           # vectors gather many bf16-rounded terms; a wrong kernel is off by O(1)
            continue
        assert err <= grad_tol, (p.name, err)
        worst = max(worst, (p.name, err), key=lambda t: t[1])
    print(f"124M autocast={autocast}: loss {loss} vs {oloss}; worst matrix gradient {worst}")
    rep = tr.step(x, y)                                  # the one-call step the benchmark times (AdamW on the side lane under autocast)
    assert abs(rep.loss - oloss) <= loss_tol * abs(oloss) and rep.step == 1
    rep2 = tr.step(x, y)
    assert rep2.loss < rep.loss
    tr.close()


def test_attention_backward_from_the_saved_output_agrees_with_the_recompute_form(be):
    """The step's shortcut (Dr from the saved bf16 output) against ojc_causal_sdpa_backward_recompute at the 124M step's attention
    shape: the two differ only by the bf16 rounding of O inside Dr. Bound 1e-2 normwise per gradient, and both within 2e-2 of the
    oracle on the planes it computes."""
    from ojas_b200 import DType
    b, h, t, d = 2, 12, 1024, 64
    q, k, v, gy = (orc.round_bf16(orc.init_normal(n, 40 + i, 1.0, (b, h, t, d))) for i, n in enumerate(("q", "k", "v", "gy")))
    dq, dk, dv, dgy = (be.upload(a, DType.BF16) for a in (q, k, v, gy))
    y, lse = be.causal_sdpa_forward(dq, dk, dv)
    saved = [g.numpy() for g in be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy)]
    recomputed = [g.numpy() for g in be.causal_sdpa_backward_recompute(dq, dk, dv, dgy)]
    for name, a, r in zip(("dq", "dk", "dv"), saved, recomputed):
        assert rel(a, r) <= 1e-2, (name, rel(a, r))
    for bi, hi in ((0, 0), (1, 11)):
        sl = (slice(bi, bi + 1), slice(hi, hi + 1))
        oy, olse = orc.causal_sdpa_forward(q[sl], k[sl], v[sl])
        want = orc.causal_sdpa_backward(q[sl], k[sl], v[sl], oy, olse, gy[sl])
        for got_set in (saved, recomputed):
            assert max(rel(g[sl], w) for g, w in zip(got_set, want)) <= 2e-2


def test_causal_sdpa_at_the_standalone_benchmark_shape(be):
    from ojas_b200 import DType
    b, h, t, d = 8, 16, 4096, 128
    q, k, v, gy = (orc.round_bf16(orc.init_normal(n, 300 + i, 1.0, (b, h, t, d))) for i, n in enumerate(("q", "k", "v", "gy")))
    dq, dk, dv, dgy = (be.upload(a, DType.BF16) for a in (q, k, v, gy))
    y, lse = be.causal_sdpa_forward(dq, dk, dv)
    gq, gk, gv = be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy)
    got = [a.numpy() for a in (y, lse, gq, gk, gv)]
    del y, gq, gk, gv
    # strict-order oracle on six planes (first, last, and four inside)
    for bi, hi in ((0, 0), (0, 15), (3, 7), (5, 9), (7, 0), (7, 15)):
        sl = (slice(bi, bi + 1), slice(hi, hi + 1))
        oy, olse = orc.causal_sdpa_forward(q[sl], k[sl], v[sl])
        ogq, ogk, ogv = orc.causal_sdpa_backward(q[sl], k[sl], v[sl], oy, olse, gy[sl])
        assert rel(got[0][sl], oy) <= 2e-2 and np.abs(got[1][sl] - olse).max() <= 2e-3, (bi, hi)
        errs = [rel(g[sl], w) for g, w in zip(got[2:], (ogq, ogk, ogv))]
        assert max(errs) <= 2e-2, (bi, hi, errs)
    # every plane against the f32 tier (CUDA-core kernels, same inputs widened to f32)
    fq, fk, fv, fgy = (be.upload(a) for a in (q, k, v, gy))
    fy, flse = be.causal_sdpa_forward(fq, fk, fv)
    want_lse = flse.numpy()
    assert np.abs(got[1] - want_lse).max() <= 2e-3                      # all 8 x 16 x 4096 rows
    fgq, fgk, fgv = be.causal_sdpa_backward(fq, fk, fv, fy, flse, fgy)
    for name, g, w in zip(("out", "dq", "dk", "dv"), (got[0], got[2], got[3], got[4]), (fy, fgq, fgk, fgv)):
        w = w.numpy()
        worst = max(rel(g[bi, hi], w[bi, hi]) for bi in range(b) for hi in range(h))
        assert worst <= 2e-2, (name, worst)


def test_bf16_loss_curve_tracks_the_f32_tier_at_124m_over_200_steps(be):
    """The north star's 200-step curve gate at the model it is quoted on: 200 AdamW steps of nanolab-124M under bf16 autocast against the
    same 200 steps on this backend's f32 tier (which the tests above hold to the CPU oracle at these shapes; 200 strict-order CPU steps of
    this model would take hours), same weights, same batches. Every step's loss within 2%. The 200 batches are all different and their
    ids follow a skewed (exponential, mean 500) distribution, so the loss falls from ln V = 10.8 to the stream's unigram entropy near 7.2
    and stays there: a curve that moves without collapsing to zero, where a relative gap would mean nothing."""
    from ojas_b200 import ModelSpec, TrainConfig, Trainer
    from bench import init_weights
    b, t, steps = 2, 1024, 200
    rng = np.random.Generator(np.random.PCG64(3))
    draws = np.minimum(rng.exponential(500.0, size=(steps, b, t + 1)).astype(np.int64), KW_124M["vocab"] - 1).astype(np.uint32)
    curves = []
    for autocast in (False, True):
        tr = Trainer(be, ModelSpec(**KW_124M), TrainConfig(autocast_bf16=autocast, optimizer="adamw", adam_lr=3e-4, adam_weight_decay=0.1, grad_clip=1.0), b, t)
        tr.set_params(init_weights(tr.params, 0))
        curves.append([tr.step(np.ascontiguousarray(d[:, :-1]), np.ascontiguousarray(d[:, 1:])).loss for d in draws])
        tr.close()
    f32, bf16 = (np.array(c, np.float64) for c in curves)
    worst = np.max(np.abs(bf16 - f32) / f32)
    print(f"124M 200 steps: f32 {f32[0]:.4f} -> {f32[-1]:.4f}, bf16 {bf16[0]:.4f} -> {bf16[-1]:.4f}, worst relative gap {worst:.2e}")
    assert f32[-1] < 0.8 * f32[0] and f32[-1] > 3.0       # the curve moves, and stays a loss worth comparing
    assert worst <= 2e-2, worst
