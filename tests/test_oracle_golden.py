"""Pins the CPU oracle to the reference's own golden vectors.

The fixtures and digest table repeat ojas-cpu/tests/exact_golden.rs:66-276: the
same SplitMix64 seeds, shapes and call order, and the FNV-1a digests of the output
bits recorded there. `ce_loss` takes libm's f32 ln and is checked only where it
was recorded (exact_golden.rs:199-202), so it is skipped here as it is there.
"""
import json

import numpy as np
import pytest

from oracle import oracle as orc

LINEAR = [(1, 1, 1), (3, 5, 9), (73, 11, 13), (127, 67, 131), (64, 128, 96), (70, 80, 100), (257, 129, 65),
          (65, 257, 129), (129, 65, 257), (97, 255, 95), (33, 1000, 17), (200, 300, 520)]


def digests():
    out = {}
    for i, (rows, kin, nout) in enumerate(LINEAR):
        rng = orc.SplitMix64(100 + i)
        x = rng.vec(rows * kin, 0.5).reshape(rows, kin)
        w = rng.vec(nout * kin, 0.5).reshape(nout, kin)
        gy = rng.vec(rows * nout, 0.5).reshape(rows, nout)
        y = orc.linear_forward(x, w)
        gx, gw = orc.linear_backward(x, w, gy)
        tag = f"{rows}x{kin}x{nout}"
        out[f"linear_fwd {tag}"], out[f"linear_gx {tag}"], out[f"linear_gw {tag}"] = orc.fnv(y), orc.fnv(gx), orc.fnv(gw)
    for i, (rows, cols) in enumerate([(64, 48), (48, 64), (130, 70), (97, 97)]):
        rng = orc.SplitMix64(200 + i)
        p = rng.vec(rows * cols, 0.1).reshape(rows, cols)
        g = rng.vec(rows * cols, 0.1).reshape(rows, cols)
        m = rng.vec(rows * cols, 0.01).reshape(rows, cols)
        orc.muon_ns5_step(p, g, m)  # MuonNs5Config::nanolab_default
        out[f"muon_p {rows}x{cols}"], out[f"muon_m {rows}x{cols}"] = orc.fnv(p), orc.fnv(m)
    for i, shape in enumerate([[2, 3, 33, 24], [1, 2, 300, 64], [2, 2, 64, 16]]):
        n = int(np.prod(shape))
        rng = orc.SplitMix64(300 + i)
        q, k, v, gy = (rng.vec(n, 0.5).reshape(shape) for _ in range(4))
        y, lse = orc.causal_sdpa_forward(q, k, v)
        gq, gk, gv = orc.causal_sdpa_backward(q, k, v, y, lse, gy)
        tag = str(shape)
        for name, val in (("fwd", y), ("lse", lse), ("gq", gq), ("gk", gk), ("gv", gv)):
            out[f"sdpa_{name} {tag}"] = orc.fnv(val)
    rows, dim = 300, 256
    rng = orc.SplitMix64(400)
    x = rng.vec(rows * dim, 1.0).reshape(rows, dim)
    w = (np.float32(1.0) + rng.vec(dim, 0.1)).astype(np.float32)
    gy = rng.vec(rows * dim, 1.0).reshape(rows, dim)
    out["rms_fwd"] = orc.fnv(orc.rms_norm_forward(x, w, 1e-6))
    gx, gw = orc.rms_norm_backward(x, w, gy, 1e-6)
    out["rms_gx"], out["rms_gw"] = orc.fnv(gx), orc.fnv(gw)
    b, t, h, d = 2, 64, 4, 32
    rng = orc.SplitMix64(500)
    x = rng.vec(b * t * h * d, 1.0).reshape(b, t, h, d)
    cos = rng.vec(t * d, 1.0).reshape(t, d)
    sin = rng.vec(t * d, 1.0).reshape(t, d)
    out["rope_fwd"] = orc.fnv(orc.rope(x, cos, sin))
    out["rope_bwd"] = orc.fnv(orc.rope(x, cos, sin, backward=True))
    rows, vocab = 257, 500
    rng = orc.SplitMix64(600)
    logits = rng.vec(rows * vocab, 4.0).reshape(rows, vocab)
    targets = np.array([7 if i % 11 == 3 else rng.below(vocab) for i in range(rows)], np.uint32)
    loss, grad = orc.cross_entropy_mean(logits, targets, ignore=7, want_grad=True)
    out["ce_loss"], out["ce_grad"] = orc.fnv(np.array([loss], np.float32)), orc.fnv(grad)
    n = 100_003
    rng = orc.SplitMix64(700)
    p, g, m1 = rng.vec(n, 1.0), rng.vec(n, 0.1), rng.vec(n, 0.01)
    m2 = np.abs(rng.vec(n, 0.01))
    orc.adamw_step(p, g, m1, m2, 9, 3e-3, weight_decay=0.1)  # AdamWConfig::nanolab(3e-3, 0.1)
    out["adamw_p"], out["adamw_m1"], out["adamw_m2"] = orc.fnv(p), orc.fnv(m1), orc.fnv(m2)
    return out


@pytest.fixture(scope="module")
def got():
    return digests()


def test_every_exact_golden_digest(got, golden_dir):
    want = json.loads((golden_dir / "exact_golden_digests.json").read_text())
    assert len(want) == 69 and set(want) == set(got)
    bad = {k: (f"{got[k]:016x}", want[k]) for k in want if k != "ce_loss" and f"{got[k]:016x}" != want[k]}
    assert not bad, bad


def test_digests_do_not_depend_on_thread_count(got):
    # exact_golden.rs:286-301 runs 1, 2, 3, 7, 16, 18 threads; OpenMP here never splits a reduction.
    import ctypes
    omp = ctypes.CDLL("libgomp.so.1")
    try:
        for threads in (1, 3, 7):
            omp.omp_set_num_threads(threads)
            assert digests() == got, threads
    finally:
        omp.omp_set_num_threads(omp.omp_get_num_procs())


def test_splitmix_and_fnv_reference_vectors():
    rng = orc.SplitMix64(0)  # ojas-kernels/src/rng.rs:57-60
    assert [rng.next_u64() for _ in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    assert orc.lib.orc_fnv1a_bytes(b"", 0) == 0xCBF29CE484222325


def test_exp_exact_pins(golden_dir):
    # ojas-core/src/exp_exact_pins.txt: every 2^20th f32 in [-104, 89], the near-boundary inputs, the range edges.
    pins = [l.split() for l in (golden_dir / "exp_exact_pins.txt").read_text().splitlines() if not l.startswith("#")]
    assert len(pins) > 2000
    xs = np.array([int(a, 16) for a, _ in pins], np.uint32).view(np.float32)
    want = np.array([int(b, 16) for _, b in pins], np.uint32)
    got = np.array([orc.exp_exact(float(x)) for x in xs], np.float32).view(np.uint32)
    assert np.array_equal(got, want)
    assert orc.exp_exact(0.0) == 1.0 and orc.exp_exact(float("inf")) == float("inf") and orc.exp_exact(-1e9) == 0.0
    assert np.isnan(orc.exp_exact(float("nan")))


def test_rms_norm_f64_fixture():
    """ojas-oracle/fixtures/rms_norm_f64.json: one row against the f64 formula x * w / sqrt(mean(x^2) + eps), eps 1e-6."""
    x = np.array([[0.5, -1.25, 0.75, 2.0]], np.float32)
    w = np.array([1.0, 0.5, -1.0, 1.5], np.float32)
    want = np.array([0.39605889293691887, -0.4950736161711486, -0.5940883394053783, 2.3763533576215132])
    got = orc.rms_norm_forward(x, w, 1e-6)
    assert np.abs(got[0].astype(np.float64) - want).max() <= 2e-7
    ref = x[0].astype(np.float64) * w / np.sqrt(np.mean(x[0].astype(np.float64) ** 2) + 1e-6)
    assert np.abs(ref - want).max() <= 1e-15
