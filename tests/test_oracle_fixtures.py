"""The CPU oracle against the reference's torch goldens (ojas-oracle/fixtures, copied to tests/golden).

Gates are the reference's own (ojas-oracle/src/parity.rs:29-45): forward loss 1e-5
relative, logits 1e-5 normwise, every gradient 1e-4 normwise and exactly zero
where torch's is zero.
"""
import json

import numpy as np
import pytest
from safetensors import safe_open

from oracle import oracle as orc

FORWARD_LOSS_REL_TOL = 1e-5
LOGITS_NORMWISE_REL_TOL = 1e-5
GRAD_NORMWISE_REL_TOL = 1e-4


def load(path, prefix=""):
    f = safe_open(str(path), "np")
    meta = f.metadata()
    tensors = {k[len(prefix):]: f.get_tensor(k) for k in f.keys() if k.startswith(prefix)}
    return tensors, meta


def spec_from(meta) -> orc.Spec:
    s = json.loads(meta["ojas.spec"])
    return orc.Spec(vocab=s["vocab"], n_embd=s["n_embd"], n_layer=s["n_layer"], n_head=s["n_head"], n_kv_head=s["n_kv_head"],
                    head_dim=s["head_dim"], hidden=s["hidden"], max_seq=s["max_seq"], window=s.get("window"),
                    rope_base=s["rope_base"], rms_eps=s["rms_eps"])


def normwise(got, want):
    got, want = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
    return np.linalg.norm(got - want) / np.linalg.norm(want)


def check_grads(spec, params, ids, targets, want, seed, no_grad):
    table = orc.param_table(spec)
    loss, grads, _ = orc.forward_loss(spec, [params[i.name] for i in table], ids, targets, seed=seed)
    for info, g in zip(table, grads):
        if info.name in no_grad:
            assert not info.trains
            continue
        w = want[info.name]
        if not np.any(w):
            assert not np.any(g), info.name
        else:
            assert normwise(g, w) <= GRAD_NORMWISE_REL_TOL, (info.name, normwise(g, w))
    return loss


@pytest.fixture(scope="module")
def tiny(golden_dir):
    params, meta = load(golden_dir / "tiny/init.safetensors")
    fwd, fmeta = load(golden_dir / "tiny/forward.safetensors")
    return spec_from(meta), params, fwd, json.loads(fmeta["ojas.oracle"])


def test_param_table_matches_the_init_fixture(tiny):
    spec, params, _, _ = tiny
    table = orc.param_table(spec)
    assert len(table) == 30 and {i.name for i in table} == set(params)
    for i in table:
        assert tuple(params[i.name].shape) == i.shape, i.name
    assert [i.name for i in table if not i.trains] == ["blocks.0.mixer.vr_lambda"]
    assert table[0].group == 0 and all(i.group == (1 if len(i.shape) == 2 else 0) for i in table[1:])


def test_forward_logits_and_loss(tiny):
    spec, params, fwd, meta = tiny
    table = orc.param_table(spec)
    loss, _, logits = orc.forward_loss(spec, [params[i.name] for i in table], fwd["x"], fwd["y"], want_grads=False, want_logits=True)
    want = np.uint32(meta["loss_f32_bits"]).view(np.float32)
    assert abs(float(loss) - float(want)) / abs(float(want)) <= FORWARD_LOSS_REL_TOL
    assert normwise(logits, fwd["logits"]) <= LOGITS_NORMWISE_REL_TOL


@pytest.mark.parametrize("which", ["grads_init", "grads_step5"])
def test_gradients(tiny, golden_dir, which):
    spec, params, fwd, _ = tiny
    want, meta = load(golden_dir / f"tiny/{which}.safetensors")
    meta = json.loads(meta["ojas.oracle"])
    if which == "grads_step5":
        params, _ = load(golden_dir / "tiny/trace_ns5_f32.safetensors")
    loss = check_grads(spec, params, fwd["x"], fwd["y"], want, meta["loss_seed"], meta["no_grad"])
    assert abs(float(loss) - meta["loss"]) / meta["loss"] <= FORWARD_LOSS_REL_TOL


@pytest.mark.parametrize("variant", ["gqa", "swa"])
def test_gqa_and_sliding_window_variants(golden_dir, variant):
    path = golden_dir / f"variants/{variant}.safetensors"
    params, meta = load(path, "param/")
    grads, _ = load(path, "grad/")
    rest, _ = load(path)
    spec = spec_from(meta)
    info = json.loads(meta["ojas.oracle"])
    assert (spec.n_kv_head, spec.window) == ((2, None) if variant == "gqa" else (4, 8))
    table = orc.param_table(spec)
    loss, _, logits = orc.forward_loss(spec, [params[i.name] for i in table], rest["x"], rest["y"], want_grads=False, want_logits=True)
    assert abs(float(loss) - info["loss"]) / info["loss"] <= FORWARD_LOSS_REL_TOL
    assert normwise(logits, rest["logits"]) <= LOGITS_NORMWISE_REL_TOL
    check_grads(spec, params, rest["x"], rest["y"], grads, info["loss_seed"], info["no_grad"])


def test_muon_bf16_step_matches_stock_nanolab(golden_dir):
    t, meta = load(golden_dir / "tiny/muon_step_bf16.safetensors")
    for i, case in enumerate(json.loads(meta["ojas.oracle"])["cases"]):
        p, m = t[f"c{i}.p"].copy(), t[f"c{i}.m"].copy()
        orc.muon_ns5_step(p, t[f"c{i}.g"], m, lr=case["lr"], momentum=case["momentum"], weight_decay=case["weight_decay"],
                          nesterov=case["nesterov"], bf16=True)
        assert np.array_equal(m.view(np.uint32), t[f"c{i}.m_after"].view(np.uint32)), i
        assert normwise(p, t[f"c{i}.p_after"]) <= 1e-6, (i, normwise(p, t[f"c{i}.p_after"]))


def test_one_head_step_against_torch_bits(golden_dir):
    """ojas-cpu/tests/torch_ref.rs:97-250: RMSNorm, QKV, RoPE, SDPA, CE, backward, AdamW; every error <= 1e-4."""
    d = json.loads((golden_dir / "torch_ref.json").read_text())
    f = lambda k, shape: np.array(d[k], np.uint32).view(np.float32).reshape(shape)
    b, t, dim, vocab = 1, 4, 16, 32
    x, norm_w = f("X", (b * t, dim)), f("NORM_W0", (dim,))
    wq, wk, wv, wo = f("WQ0", (dim, dim)), f("WK0", (dim, dim)), f("WV0", (dim, dim)), f("WO0", (vocab, dim))
    cos, sin = f("COS", (t, dim)), f("SIN", (t, dim))
    targets = np.array(d["TARGETS"], np.uint32)
    h = orc.rms_norm_forward(x, norm_w, 1e-6)
    q, k, v = orc.linear_forward(h, wq), orc.linear_forward(h, wk), orc.linear_forward(h, wv)
    qr = orc.rope(q.reshape(b, t, 1, dim), cos, sin).reshape(b, 1, t, dim)
    kr = orc.rope(k.reshape(b, t, 1, dim), cos, sin).reshape(b, 1, t, dim)
    va = v.reshape(b, 1, t, dim)
    attn, lse = orc.causal_sdpa_forward(qr, kr, va)
    y = attn.reshape(b * t, dim)
    logits = orc.linear_forward(y, wo)
    loss, g_logits = orc.cross_entropy_mean(logits, targets, want_grad=True)
    g_y, _ = orc.linear_backward(y, wo, g_logits)
    gq, gk, gv = orc.causal_sdpa_backward(qr, kr, va, attn, lse, g_y.reshape(b, 1, t, dim))
    gq_lin = orc.rope(gq.reshape(b, t, 1, dim), cos, sin, backward=True).reshape(b * t, dim)
    gk_lin = orc.rope(gk.reshape(b, t, 1, dim), cos, sin, backward=True).reshape(b * t, dim)
    gq_h, g_wq = orc.linear_backward(h, wq, gq_lin)
    gk_h, _ = orc.linear_backward(h, wk, gk_lin)
    gv_h, _ = orc.linear_backward(h, wv, gv.reshape(b * t, dim))
    g_h = (gq_h + gk_h + gv_h).astype(np.float32)
    _, g_norm = orc.rms_norm_backward(x, norm_w, g_h, 1e-6)
    lr = 6e-4 * float(np.array([d["COSINE_MULT_STEP8"]], np.uint64).view(np.float64)[0])
    wq2, m1, m2 = wq.copy(), np.zeros_like(wq), np.zeros_like(wq)
    orc.adamw_step(wq2, g_wq, m1, m2, 0, lr, weight_decay=0.1)
    nw, n1, n2 = norm_w.copy(), np.zeros_like(norm_w), np.zeros_like(norm_w)
    orc.adamw_step(nw, g_norm, n1, n2, 0, lr, weight_decay=0.0)
    errs = {
        "h": np.abs(h - f("H", h.shape)).max(), "attn": np.abs(y - f("ATTN", y.shape)).max(),
        "logits": np.abs(logits - f("LOGITS", logits.shape)).max(),
        "loss": abs(float(loss) - float(np.uint32(d["LOSS"]).view(np.float32))),
        "gwq": np.abs(g_wq - f("GWQ", g_wq.shape)).max(), "gnorm": np.abs(g_norm - f("GWN", g_norm.shape)).max(),
        "wq": np.abs(wq2 - f("WQ_AFTER", wq.shape)).max(), "norm": np.abs(nw - f("NORM_AFTER", nw.shape)).max(),
    }
    assert max(errs.values()) <= 1e-4, errs
