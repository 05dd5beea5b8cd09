"""Per-op parity of the CUDA library against the CPU oracle, through the C ABI (f32 tier and bf16 tensor-core tier).

Shapes follow the reference's device-vs-CPU list (1, primes, both sides of 64 / 128 block edges; T = 1, 17, 257:
ojas-wgpu/tests/parity.rs:1-60). Bars: the f32 tier matches the strict-order oracle to 1e-5 (forward) / 1e-4
(gradients) normwise; index outputs are bit-exact; the bf16 tier is compared on bf16-exact inputs so only the f32
accumulation order differs.
"""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

FWD_TOL, GRAD_TOL = 1e-5, 1e-4


@pytest.fixture(scope="module")
def be():
    from ojas_b200 import CudaBackend
    backend = CudaBackend(0, 64 << 30)
    yield backend
    backend.sync()
    backend.close()


def rel(got, want):
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    denom = np.linalg.norm(want)
    return np.linalg.norm(got - want) / (denom if denom > 0 else 1.0)


def rnd(seed, shape, scale=1.0):
    return orc.SplitMix64(seed).vec(int(np.prod(shape)), scale).reshape(shape)


LINEAR = [(1, 1, 1), (3, 5, 9), (73, 11, 13), (127, 67, 131), (64, 128, 96), (257, 129, 65), (65, 257, 129), (33, 1000, 17), (200, 300, 520)]


@pytest.mark.parametrize("rows,kin,nout", LINEAR)
def test_linear_f32_tier(be, rows, kin, nout):
    x, w, gy = rnd(1, (rows, kin), 0.5), rnd(2, (nout, kin), 0.5), rnd(3, (rows, nout), 0.5)
    dx, dw, dgy = be.upload(x), be.upload(w), be.upload(gy)
    # the f32 tier adds a(i,k) b(k,j) for k ascending with a separate multiply and add, as the reference's Exact product does
    # (ojas-cpu/src/gemm.rs:11-16): the bits are the oracle's
    assert np.array_equal(be.linear_forward(dx, dw).numpy().view(np.uint32), orc.linear_forward(x, w).view(np.uint32))
    gx, gw = be.linear_backward(dx, dw, dgy)
    ogx, ogw = orc.linear_backward(x, w, gy)
    assert np.array_equal(gx.numpy().view(np.uint32), ogx.view(np.uint32)) and np.array_equal(gw.numpy().view(np.uint32), ogw.view(np.uint32))
    assert np.array_equal(be.linear_backward_input(dw, dgy).numpy().view(np.uint32), ogx.view(np.uint32))


# outputs of at least 256 x 256 take the two-SM kernel (CTA pairs), smaller ones the one-SM kernel; ragged edges on both
TC_SHAPES = [(128, 64, 256), (64, 64, 64), (200, 136, 520), (256, 768, 768), (1024, 768, 2048), (384, 2048, 768), (8, 8, 8), (130, 72, 264), (2048, 256, 4096),
             (300, 136, 520), (513, 72, 264), (640, 1024, 392)]


@pytest.mark.parametrize("rows,kin,nout", TC_SHAPES)
def test_linear_bf16_tensor_core_all_three_layouts(be, rows, kin, nout):
    """y = x W^T (both K-major), dX = g W (B MN-major), dW = g^T x (both MN-major) on the tcgen05 kernel."""
    from ojas_b200 import DType
    x, w, gy = orc.round_bf16(rnd(11, (rows, kin), 0.5)), orc.round_bf16(rnd(12, (nout, kin), 0.5)), orc.round_bf16(rnd(13, (rows, nout), 0.5))
    dx, dw, dgy = be.upload(x, DType.BF16), be.upload(w, DType.BF16), be.upload(gy, DType.BF16)
    y = be.linear_forward(dx, dw, out_dtype=DType.F32).numpy()
    assert rel(y, orc.linear_forward(x, w)) <= FWD_TOL
    gx, gw = be.linear_backward(dx, dw, dgy, out_dtype=DType.F32)
    ogx, ogw = orc.linear_backward(x, w, gy)
    assert rel(gx.numpy(), ogx) <= FWD_TOL
    assert rel(gw.numpy(), ogw) <= FWD_TOL
    yb = be.linear_forward(dx, dw).numpy()  # bf16 output: one rounding of the f32 accumulator
    assert rel(yb, orc.linear_forward(x, w)) <= 4e-3
    be.sync()


def test_linear_refusals(be):
    from ojas_b200 import OjasError
    x, w = be.upload(rnd(1, (4, 8))), be.upload(rnd(2, (3, 7)))
    with pytest.raises(OjasError) as e:
        be.linear_forward(x, w)
    assert e.value.kind == "Shape"
    ids = be.upload(np.zeros(4, np.uint32))
    with pytest.raises(OjasError) as e:
        be.linear_forward(ids, be.upload(rnd(2, (3, 1))))
    assert e.value.kind in ("Dtype", "Shape")


@pytest.mark.parametrize("rows,dim", [(1, 1), (7, 3), (300, 256), (33, 64), (65, 768), (129, 127), (5, 2048)])
def test_rms_norm(be, rows, dim):
    x, gy = rnd(400, (rows, dim)), rnd(401, (rows, dim))
    w = (1.0 + rnd(402, (dim,), 0.1)).astype(np.float32)
    dx, dw, dgy = be.upload(x), be.upload(w), be.upload(gy)
    assert rel(be.rms_norm_forward(dx, dw, 1e-6).numpy(), orc.rms_norm_forward(x, w, 1e-6)) <= FWD_TOL
    gx, gw = be.rms_norm_backward(dx, dw, dgy, 1e-6)
    ogx, ogw = orc.rms_norm_backward(x, w, gy, 1e-6)
    if dim > 1:  # with one column dX is pure cancellation noise on both sides
        assert rel(gx.numpy(), ogx) <= GRAD_TOL
    assert rel(gw.numpy(), ogw) <= GRAD_TOL


def test_rms_qk_norm_is_two_row_norms(be):
    q, k = rnd(1, (2, 9, 4, 16)), rnd(2, (2, 9, 2, 16))
    qw, kw = (1 + rnd(3, (16,), 0.1)).astype(np.float32), (1 + rnd(4, (16,), 0.1)).astype(np.float32)
    qo, ko = be.rms_qk_norm_forward(be.upload(q), be.upload(k), be.upload(qw), be.upload(kw), 1e-6)
    assert rel(qo.numpy(), orc.rms_norm_forward(q, qw, 1e-6)) <= FWD_TOL and rel(ko.numpy(), orc.rms_norm_forward(k, kw, 1e-6)) <= FWD_TOL
    gq, gk = rnd(5, q.shape), rnd(6, k.shape)
    a, b, c, d = be.rms_qk_norm_backward(be.upload(q), be.upload(k), be.upload(qw), be.upload(kw), be.upload(gq), be.upload(gk), 1e-6)
    oq, oqw = orc.rms_norm_backward(q, qw, gq, 1e-6)
    ok, okw = orc.rms_norm_backward(k, kw, gk, 1e-6)
    assert max(rel(a.numpy(), oq), rel(b.numpy(), ok), rel(c.numpy(), oqw), rel(d.numpy(), okw)) <= GRAD_TOL


@pytest.mark.parametrize("b,t,h,d", [(2, 64, 4, 32), (1, 1, 1, 2), (2, 17, 3, 64), (1, 257, 2, 16)])
def test_rope(be, b, t, h, d):
    x, cos, sin = rnd(500, (b, t, h, d)), rnd(501, (t, d)), rnd(502, (t, d))
    dx, dc, ds = be.upload(x), be.upload(cos), be.upload(sin)
    assert rel(be.rope_half_split_forward(dx, dc, ds).numpy(), orc.rope(x, cos, sin)) <= FWD_TOL
    assert rel(be.rope_half_split_backward(dx, dc, ds).numpy(), orc.rope(x, cos, sin, backward=True)) <= FWD_TOL


@pytest.mark.parametrize("shape,hkv,window", [((2, 3, 33, 24), 3, None), ((1, 2, 300, 64), 2, None), ((2, 2, 64, 16), 2, None), ((1, 4, 65, 32), 2, None),
                                              ((1, 2, 129, 64), 2, 8), ((1, 4, 40, 16), 1, 5), ((1, 1, 1, 8), 1, None), ((1, 2, 17, 128), 2, None),
                                              ((1, 1, 257, 64), 1, 1)])
def test_causal_sdpa_f32_tier(be, shape, hkv, window):
    b, h, t, d = shape
    q, gy = rnd(300, shape, 0.5), rnd(303, shape, 0.5)
    k, v = rnd(301, (b, hkv, t, d), 0.5), rnd(302, (b, hkv, t, d), 0.5)
    oy, olse = orc.causal_sdpa_forward(q, k, v, window)
    ogq, ogk, ogv = orc.causal_sdpa_backward(q, k, v, oy, olse, gy, window)
    dq, dk, dv, dgy = be.upload(q), be.upload(k), be.upload(v), be.upload(gy)
    y, lse = be.causal_sdpa_forward(dq, dk, dv, window)
    assert rel(y.numpy(), oy) <= FWD_TOL and rel(lse.numpy(), olse) <= FWD_TOL
    gq, gk, gv = be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy, window)
    assert max(rel(gq.numpy(), ogq), rel(gk.numpy(), ogk), rel(gv.numpy(), ogv)) <= GRAD_TOL
    rq, rk, rv = be.causal_sdpa_backward_recompute(dq, dk, dv, dgy, window)
    assert max(rel(rq.numpy(), ogq), rel(rk.numpy(), ogk), rel(rv.numpy(), ogv)) <= GRAD_TOL


@pytest.mark.parametrize("shape,hkv,window", [((1, 2, 300, 64), 2, None), ((2, 4, 128, 64), 2, None), ((1, 2, 129, 128), 2, None), ((1, 2, 200, 64), 1, 40),
                                              ((1, 1, 64, 64), 1, None), ((1, 2, 1, 64), 2, None), ((2, 3, 1024, 64), 3, None),
                                              ((1, 2, 256, 128), 2, None), ((2, 4, 384, 128), 2, None), ((1, 1, 132, 128), 1, None), ((1, 2, 640, 128), 1, None),
                                              ((1, 2, 64, 128), 1, None), ((2, 2, 100, 128), 2, None), ((1, 1, 4, 128), 1, None)])
def test_causal_sdpa_bf16_tensor_core_tier(be, shape, hkv, window):
    """bf16 q/k/v on the tensor-core kernels, against the f32 oracle on the same bf16-exact inputs: 2e-2 relative."""
    from ojas_b200 import DType
    b, h, t, d = shape
    q, gy = orc.round_bf16(rnd(300, shape, 1.0)), orc.round_bf16(rnd(303, shape, 1.0))
    k, v = orc.round_bf16(rnd(301, (b, hkv, t, d), 1.0)), orc.round_bf16(rnd(302, (b, hkv, t, d), 1.0))
    oy, olse = orc.causal_sdpa_forward(q, k, v, window)
    ogq, ogk, ogv = orc.causal_sdpa_backward(q, k, v, oy, olse, gy, window)
    dq, dk, dv, dgy = (be.upload(a, DType.BF16) for a in (q, k, v, gy))
    y, lse = be.causal_sdpa_forward(dq, dk, dv, window)
    assert rel(y.numpy(), oy) <= 2e-2 and rel(lse.numpy(), olse) <= 1e-4
    gq, gk, gv = be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy, window)
    assert max(rel(gq.numpy(), ogq), rel(gk.numpy(), ogk), rel(gv.numpy(), ogv)) <= 2e-2
    rq, rk, rv = be.causal_sdpa_backward_recompute(dq, dk, dv, dgy, window)
    assert max(rel(rq.numpy(), ogq), rel(rk.numpy(), ogk), rel(rv.numpy(), ogv)) <= 2e-2


@pytest.mark.parametrize("shape,hkv", [((2, 4, 384, 64), 2), ((1, 3, 300, 64), 3), ((3, 2, 640, 64), 1), ((2, 2, 516, 128), 2), ((1, 4, 1024, 128), 4)])
def test_persistent_attention_kernels_walk_several_tiles_per_cta(be, shape, hkv):
    """The persistent forward (head_dim 64) and backward kernels normally start once a launch has more tiles than the GPU has CTA slots;
    here they are forced onto three CTAs, so each walks several tiles (ragged ends, grouped-query heads, tile boundaries), and compared
    with the oracle at the tensor-core tier's 2e-2; the backward kernels must also reproduce the bits of the one-CTA-per-tile kernels."""
    import ctypes as C
    from ojas_b200 import DType
    from ojas_b200._lib import lib
    b, h, t, d = shape
    q, gy = orc.round_bf16(rnd(310, shape, 1.0)), orc.round_bf16(rnd(313, shape, 1.0))
    k, v = orc.round_bf16(rnd(311, (b, hkv, t, d), 1.0)), orc.round_bf16(rnd(312, (b, hkv, t, d), 1.0))
    oy, olse = orc.causal_sdpa_forward(q, k, v)
    want = orc.causal_sdpa_backward(q, k, v, oy, olse, gy)
    dq, dk, dv, dgy = (be.upload(a, DType.BF16) for a in (q, k, v, gy))
    try:
        lib.ojc_sdpa_forward_variant(C.c_int32(2))
        y, lse = be.causal_sdpa_forward(dq, dk, dv)
        got = [g.numpy() for g in be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy)]
        lib.ojc_sdpa_forward_variant(C.c_int32(1))
        one = [g.numpy() for g in be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy)]       # same output and lse in: the same arithmetic in the same order
        lib.ojc_sdpa_forward_variant(C.c_int32(3))
        wide = [g.numpy() for g in be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy)]      # the 128-wide kernels (the library's choice at head_dim 128) on three CTAs
        lib.ojc_sdpa_forward_variant(C.c_int32(5))
        full = [g.numpy() for g in be.causal_sdpa_backward(dq, dk, dv, y, lse, dgy)]      # and on a grid of their own choosing
    finally:
        lib.ojc_sdpa_forward_variant(C.c_int32(0))
    assert rel(y.numpy(), oy) <= 2e-2 and rel(lse.numpy(), olse) <= 1e-4
    assert max(rel(g, w) for g, w in zip(got, want)) <= 2e-2
    for a, c in zip(got, one):
        assert np.array_equal(a, c)
    # every product accumulates over the same operands in the same order of 16-wide steps: the wide kernels give the same bits too
    for a, c, e in zip(wide, one, full):
        assert max(rel(a, w) for a, w in zip(wide, want)) <= 2e-2
        assert np.array_equal(a, c) and np.array_equal(e, c)


def test_sdpa_reads_permuted_views_without_a_copy(be):
    """[B,T,H,dh] storage viewed as [B,H,T,dh] gives the same result as permute + contiguous attention."""
    b, t, h, d = 2, 33, 3, 16
    q, k, v = rnd(1, (b, t, h, d), 0.5), rnd(2, (b, t, h, d), 0.5), rnd(3, (b, t, h, d), 0.5)
    oy, olse = orc.causal_sdpa_forward(orc.permute_0213(q), orc.permute_0213(k), orc.permute_0213(v))
    dq, dk, dv = be.upload(q), be.upload(k), be.upload(v)
    from ojas_b200._lib import lib
    from ojas_b200.backend import _check, _p
    import ctypes as C
    out = be.empty((b, t, h, d))
    lse = be.empty((b, h, t))
    _check(lib.ojc_causal_sdpa_forward(be._handle, _p(dq.permuted((0, 2, 1, 3))), _p(dk.permuted((0, 2, 1, 3))), _p(dv.permuted((0, 2, 1, 3))), C.c_int64(-1),
                                       _p(out.permuted((0, 2, 1, 3))), _p(lse)))
    assert rel(orc.permute_0213(out.numpy()), oy) <= FWD_TOL and rel(lse.numpy(), olse) <= FWD_TOL
    assert np.array_equal(be.permute(dq, (0, 2, 1, 3)).numpy().view(np.uint32), orc.permute_0213(q).view(np.uint32))


def test_embedding_gather_is_bit_exact_and_scatter_matches(be):
    from ojas_b200 import OjasError
    vocab, dim, tokens = 257, 96, 1000
    table, grad = rnd(1, (vocab, dim)), rnd(2, (tokens, dim))
    rng = orc.SplitMix64(7)
    ids = np.array([rng.below(vocab) if i % 5 else 3 for i in range(tokens)], np.uint32)  # id 3 repeats: long runs
    dt, di = be.upload(table), be.upload(ids)
    out = be.embedding_forward(dt, di).numpy()
    assert np.array_equal(out.view(np.uint32), orc.embedding_forward(table, ids).view(np.uint32))
    g = be.embedding_backward(dt, di, be.upload(grad)).numpy()
    og = orc.embedding_backward(vocab, ids, grad)
    assert np.array_equal(g.view(np.uint32), og.view(np.uint32))  # ascending token order per row: same bits as the CPU
    for v2, d2 in ((5000, 96), (5000, 50)):     # mostly empty rows; 16-byte rows (one warp per row) and rows that are not (one block per row)
        ids2 = np.array([rng.below(v2) for _ in range(300)], np.uint32)
        grad2 = rnd(4, (300, d2))
        got = be.embedding_backward(be.empty((v2, d2)), be.upload(ids2), be.upload(grad2)).numpy()
        assert np.array_equal(got.view(np.uint32), orc.embedding_backward(v2, ids2, grad2).view(np.uint32))
    bad = ids.copy(); bad[17] = vocab
    be.embedding_forward(dt, be.upload(bad))
    with pytest.raises(OjasError) as e:
        be.sync()
    assert e.value.kind == "OutOfRange"


def test_pointwise_ops(be):
    n = 4099
    x, y, g = rnd(1, (n,), 4.0), rnd(2, (n,), 2.0), rnd(3, (n,))
    dx, dy, dg = be.upload(x), be.upload(y), be.upload(g)
    assert rel(be.silu_forward(dx).numpy(), orc.silu_forward(x)) <= FWD_TOL
    assert rel(be.silu_backward(dx, dg).numpy(), orc.silu_backward(x, g)) <= FWD_TOL
    assert np.array_equal(be.mul_forward(dx, dy).numpy(), x * y)
    ga, gb = be.mul_backward(dx, dy, dg)
    assert np.array_equal(ga.numpy(), g * y) and np.array_equal(gb.numpy(), g * x)
    assert np.array_equal(be.residual_add_forward(dx, dy).numpy(), x + y)
    a, b = be.residual_add_backward(dg)
    assert np.array_equal(a.numpy(), g) and np.array_equal(b.numpy(), g)
    acc = be.upload(x)
    be.accumulate_grad(acc, dy)
    assert np.array_equal(acc.numpy(), x + y)
    be.scale_grad(acc, 0.25)
    assert np.array_equal(acc.numpy(), (x + y) * np.float32(0.25))


def test_bf16_rounding_is_the_reference_integer_rule(be):
    from ojas_b200 import DType
    x = np.concatenate([rnd(1, (1000,), 3.0), np.array([0.0, -0.0, 1.0, 65504.0, 3.3895314e38, 1e-40, np.inf, -np.inf], np.float32),
                        np.array([0x3F808000, 0x3F818000, 0x3F80FFFF, 0x7F7FFFFF], np.uint32).view(np.float32)])
    want = orc.round_bf16(x)
    d = be.upload(x)
    assert np.array_equal(be.cast_bf16(d).numpy().view(np.uint32), want.view(np.uint32))
    assert np.array_equal(be.to_f32(be.to_bf16(d)).numpy().view(np.uint32), want.view(np.uint32))
    nan = np.array([0x7FC00001, 0xFF800001, 0x7F812345], np.uint32).view(np.float32)  # NaN keeps sign + payload, quiet bit set
    got = be.cast_bf16(be.upload(nan)).numpy().view(np.uint32)
    assert list(got) == [0x7FC00000, 0xFFC00000, 0x7FC10000]
    assert DType.BF16.size == 2


@pytest.mark.parametrize("rows,din,heads,dh", [(5, 7, 3, 4), (64, 64, 4, 16), (130, 96, 12, 8), (33, 768, 12, 64)])
def test_per_head_sigmoid_gate(be, rows, din, heads, dh):
    inp, w, b = rnd(1, (rows, din)), rnd(2, (heads, din), 0.2), rnd(3, (heads,), 0.5)
    attn, gy = rnd(4, (rows, heads, dh)), rnd(5, (rows, heads, dh))
    di, dw, db, da, dg = (be.upload(a) for a in (inp, w, b, attn, gy))
    oy, oscales = orc.gate_forward(inp, w, b, attn, want_scales=True)
    y, scales = be.per_head_sigmoid_gate_forward_saving(di, dw, db, da)
    assert rel(y.numpy(), oy) <= FWD_TOL and rel(scales.numpy(), oscales) <= FWD_TOL
    assert rel(be.per_head_sigmoid_gate_forward(di, dw, db, da).numpy(), oy) <= FWD_TOL
    ogx, ogw, ogb, oga = orc.gate_backward(inp, w, b, attn, gy)
    for saved in (None, scales):
        gx, gw, gb, ga = be.per_head_sigmoid_gate_backward(di, dw, db, da, dg, saved)
        assert max(rel(gx.numpy(), ogx), rel(gw.numpy(), ogw), rel(gb.numpy(), ogb), rel(ga.numpy(), oga)) <= GRAD_TOL


def test_value_residual_blend(be):
    n = 5003
    v, v0, gy = rnd(1, (n,)), rnd(2, (n,)), rnd(3, (n,))
    for lam in (0.0, 0.7, -2.5):
        dl = be.upload(np.array([lam], np.float32))
        assert rel(be.value_residual_blend_forward(be.upload(v), be.upload(v0), dl).numpy(), orc.vres_forward(v, v0, lam)) <= FWD_TOL
        gv, gv0, gl = be.value_residual_blend_backward(be.upload(v), be.upload(v0), dl, be.upload(gy))
        ogv, ogv0, ogl = orc.vres_backward(v, v0, gy, lam)
        assert rel(gv.numpy(), ogv) <= FWD_TOL and rel(gv0.numpy(), ogv0) <= FWD_TOL
        assert abs(float(gl.numpy()[0]) - float(ogl)) <= GRAD_TOL * max(1.0, abs(float(ogl)))


def test_cross_entropy_with_ignore_and_collapse(be):
    from ojas_b200 import OjasError
    rows, vocab = 257, 500
    rng = orc.SplitMix64(600)
    logits = rng.vec(rows * vocab, 4.0).reshape(rows, vocab)
    targets = np.array([7 if i % 11 == 3 else rng.below(vocab) for i in range(rows)], np.uint32)
    logits[5, :] = -30.0; logits[5, targets[5]] = 30.0  # a collapsed row: the softmax rounds to one-hot
    oloss, ograd = orc.cross_entropy_mean(logits, targets, ignore=7, want_grad=True)
    dl, dt = be.upload(logits), be.upload(targets)
    loss = be.cross_entropy_mean_forward(dl, dt, 7).numpy()[0]
    assert abs(loss - oloss) <= FWD_TOL * abs(oloss)
    g = be.cross_entropy_mean_backward(dl, dt, 7).numpy()
    assert rel(g, ograd) <= GRAD_TOL
    assert not np.any(g[targets == 7])  # ignored rows get a zero gradient
    assert g[5, targets[5]] < 0  # the collapse rule keeps a non-zero target gradient
    with pytest.raises(OjasError) as e:  # every target ignored: no mean exists
        be.cross_entropy_mean_forward(dl, be.upload(np.full(rows, 7, np.uint32)), 7)
        be.sync()
    assert e.value.kind == "NonFinite"


@pytest.mark.parametrize("rows,dim,vocab,chunk", [(64, 32, 256, 0), (100, 48, 500, 33), (257, 64, 1000, 64)])
def test_fused_linear_cross_entropy_f32_tier(be, rows, dim, vocab, chunk):
    x, w = rnd(1, (rows, dim)), rnd(2, (vocab, dim), 0.3)
    rng = orc.SplitMix64(3)
    targets = np.array([rng.below(vocab) for _ in range(rows)], np.uint32)
    oloss, ogx, ogw = orc.linear_cross_entropy_mean(x, w, targets)
    loss, gx, gw = be.linear_cross_entropy_mean(be.upload(x), be.upload(w), be.upload(targets), chunk=(chunk, 0))
    assert abs(loss.numpy()[0] - oloss) <= FWD_TOL * abs(oloss)
    assert rel(gx.numpy(), ogx) <= GRAD_TOL and rel(gw.numpy(), ogw) <= GRAD_TOL


def test_fused_linear_cross_entropy_bf16_tier(be):
    from ojas_b200 import DType
    rows, dim, vocab = 512, 128, 2048
    x, w = orc.round_bf16(rnd(1, (rows, dim))), orc.round_bf16(rnd(2, (vocab, dim), 0.3))
    rng = orc.SplitMix64(3)
    targets = np.array([rng.below(vocab) for _ in range(rows)], np.uint32)
    oloss, ogx, ogw = orc.linear_cross_entropy_mean(x, w, targets)
    loss, gx, gw = be.linear_cross_entropy_mean(be.upload(x, DType.BF16), be.upload(w, DType.BF16), be.upload(targets), chunk=(200, 0), grad_input_dtype=DType.F32)
    assert abs(loss.numpy()[0] - oloss) <= 5e-4 * abs(oloss)              # the logits tile is bf16 (one rounding of the f32 accumulator)
    assert rel(gx.numpy(), ogx) <= 1e-2 and rel(gw.numpy(), ogw) <= 1e-2  # d(logits) is rounded to bf16 before the two GEMMs


@pytest.mark.parametrize("vocab,rows,chunk", [(2048, 96, 40), (50304, 96, 40), (1000, 96, 40), (4096, 1000, 500), (50304, 700, 0)])
def test_fused_cross_entropy_row_kernels_give_the_same_bits(be, vocab, rows, chunk):
    """Under bf16 autocast the fused loss turns its bf16 logits tile into the gradient row by row. Rows that fit twice in an SM's shared
    memory (the 124M head's 50304 columns do) are worked on there: by persistent CTAs that stream rows through two buffers with bulk
    copies when a tile has at least two rows per SM (the last two cases; three or more rows per CTA, so buffers are reused), else by a
    CTA per row; wider rows are re-read from L2. Same arithmetic in the same order: the loss and both gradients must be equal bit for
    bit, also with ignored and collapsed rows and a width that is not a multiple of 8."""
    import ctypes as C
    from ojas_b200 import DType
    from ojas_b200._lib import lib
    dim = 64
    x, w = orc.round_bf16(rnd(11, (rows, dim))), orc.round_bf16(rnd(12, (vocab, dim), 0.3))
    x[5] *= 40.0                                         # a row whose softmax collapses onto one column
    x = orc.round_bf16(x)
    rng = orc.SplitMix64(13)
    targets = np.array([rng.below(vocab) for _ in range(rows)], np.uint32)
    targets[5] = int(np.argmax(x[5] @ w.T))
    targets[7] = 0xFFFFFFFF                              # ignored
    dx, dw, dt = be.upload(x, DType.BF16), be.upload(w, DType.BF16), be.upload(targets)
    out = []
    try:
        for variant in (0, 1, 2):
            assert lib.ojc_ce_rows_variant(C.c_int32(variant)) == 0
            launches = be.kernel_launches()
            loss, gx, gw = be.linear_cross_entropy_mean(dx, dw, dt, chunk=(chunk, 0), grad_input_dtype=DType.F32, ignore_index=0xFFFFFFFF)
            out.append((loss.numpy().copy(), gx.numpy().copy(), gw.numpy().copy(), be.kernel_launches() - launches))
    finally:
        lib.ojc_ce_rows_variant(C.c_int32(0))
    assert out[0][3] == out[1][3] == out[2][3]
    for other in out[1:]:
        for a, b_ in zip(out[0][:3], other[:3]):
            assert np.array_equal(a.view(np.uint32), b_.view(np.uint32)) and np.isfinite(a).all()


def test_argmax_rows_is_bit_exact_with_ties_to_the_lowest_column(be):
    x = rnd(1, (300, 517))
    x[3, 10] = x[3, 400] = 9.0
    x[4, :] = 1.0
    got = be.argmax_rows(be.upload(x)).numpy()
    assert np.array_equal(got, orc.argmax_rows(x)) and got[3] == 10 and got[4] == 0


def test_clip_grad_norm(be):
    parts = [rnd(1, (1000, 33)), rnd(2, (17,)), rnd(3, (50000,))]
    for max_norm in (1.0, 1e9):
        want = [p.copy() for p in parts]
        onorm = orc.clip_grad_norm(want, max_norm)
        dev = [be.upload(p) for p in parts]
        norm = be.clip_grad_norm(dev, max_norm)
        assert abs(norm - onorm) <= 1e-6 * onorm
        for d, w in zip(dev, want):
            assert rel(d.numpy(), w) <= 1e-6


def test_adamw_step(be):
    from ojas_b200 import AdamWConfig
    n = 100_003
    rng = orc.SplitMix64(700)
    p, g, m1 = rng.vec(n, 1.0), rng.vec(n, 0.1), rng.vec(n, 0.01)
    m2 = np.abs(rng.vec(n, 0.01))
    for wd in (0.1, 0.0):
        op, om1, om2 = p.copy(), m1.copy(), m2.copy()
        orc.adamw_step(op, g, om1, om2, 9, 3e-3, weight_decay=wd)
        dp, dm1, dm2 = be.upload(p), be.upload(m1), be.upload(m2)
        be.adamw_step(dp, be.upload(g), dm1, dm2, 9, AdamWConfig(3e-3, wd))
        assert rel(dp.numpy(), op) <= 1e-6 and rel(dm1.numpy(), om1) <= 1e-6 and rel(dm2.numpy(), om2) <= 1e-6


@pytest.mark.parametrize("rows,cols", [(64, 48), (48, 64), (130, 70), (97, 97)])
def test_muon_ns5_f32(be, rows, cols):
    from ojas_b200 import MuonNs5Config
    rng = orc.SplitMix64(200)
    p, g, m = (rng.vec(rows * cols, s).reshape(rows, cols) for s in (0.1, 0.1, 0.01))
    op, om = p.copy(), m.copy()
    orc.muon_ns5_step(op, g, om)
    dp, dm = be.upload(p), be.upload(m)
    be.muon_ns5_step(dp, be.upload(g), dm, MuonNs5Config())
    assert rel(dm.numpy(), om) <= 1e-6
    assert rel(dp.numpy(), op) <= 1e-4


@pytest.mark.parametrize("rows,cols", [(64, 64), (96, 32), (32, 96), (256, 768)])
def test_muon_ns5_bf16_on_tensor_cores(be, rows, cols):
    """bf16 Newton-Schulz is discontinuous in its input (ojas-oracle/src/parity.rs:47-58): held to the reference's 5e-2."""
    from ojas_b200 import MuonNs5Config
    rng = orc.SplitMix64(201)
    p, g, m = (rng.vec(rows * cols, s).reshape(rows, cols) for s in (0.1, 0.1, 0.01))
    op, om = p.copy(), m.copy()
    orc.muon_ns5_step(op, g, om, bf16=True)
    dp, dm = be.upload(p), be.upload(m)
    be.muon_ns5_step(dp, be.upload(g), dm, MuonNs5Config(ns5_bf16=True))
    assert rel(dm.numpy(), om) <= 1e-6
    assert rel(dp.numpy() - p, op - p) <= 5e-2


def test_budget_refuses_instead_of_clamping():
    from ojas_b200 import CudaBackend, OjasError
    small = CudaBackend(0, 1 << 20)
    t = small.empty((1000,))
    with pytest.raises(OjasError) as e:
        small.empty((1 << 20,))
    assert e.value.kind == "CapacityExceeded"
    b = small.budget()
    assert b["live"] == 4000 and b["cap"] == 1 << 20
    del t
    assert small.budget()["live"] == 0
    small.close()


# ---- decode / eval ops (the rows after the training step): top-k leaders, KV-cache ring, cached attention
def test_topk_rows_ranks_like_rank_logits_bit_for_bit(be):
    from ojas_b200 import OjasError
    rng = np.random.default_rng(5)
    x = rng.standard_normal((6, 50304)).astype(np.float32)
    x[0, :40] = 3.5                      # a run of ties at the top: lowest columns win, in column order
    x[1, 7] = x[1, 4000] = x[1, 123] = 9.0
    x[2, 100:300] = -np.inf              # masked logits rank after every finite value
    x[3] = 0.0
    x[3, ::2] = -0.0                     # +0.0 and -0.0 are one value: columns 0, 1, 2, ...; the value bits stay the row's own
    x[4] = -np.inf
    x[4, 9] = -1.0
    for k in (1, 5, 50, 64, 1000, 1024):
        values, ids = be.topk_rows(be.upload(x), k)
        want_v, want_i = orc.topk_rows(x, k)
        assert np.array_equal(ids.numpy(), want_i), k
        assert values.numpy().tobytes() == want_v.tobytes(), k
    small = rng.standard_normal((3, 17)).astype(np.float32)
    values, ids = be.topk_rows(be.upload(small), 17)            # k = cols: a full sort
    assert np.array_equal(ids.numpy(), orc.topk_rows(small, 17)[1])
    for bad_k in (0, 18, 2000):
        with pytest.raises(OjasError) as e:
            be.topk_rows(be.upload(small if bad_k < 100 else x), bad_k)
        assert e.value.kind == ("Unsupported" if bad_k == 2000 else "OutOfRange")
    bad = small.copy()
    bad[1, 3] = np.inf
    be.topk_rows(be.upload(bad), 2)
    with pytest.raises(OjasError) as e:
        be.sync()
    assert e.value.kind == "NonFinite"


def test_kv_cache_write_is_a_ring_and_refuses_what_the_validator_refuses(be):
    from ojas_b200 import OjasError
    rng = np.random.default_rng(6)
    cache = rng.standard_normal((2, 8, 3, 16)).astype(np.float32)
    dev = be.upload(cache)
    want = cache.copy()
    for at, tn in ((0, 5), (5, 6), (11, 1), (12, 8), (100, 3)):          # wraps, single positions, a full turn
        src = rng.standard_normal((2, tn, 3, 16)).astype(np.float32)
        be.kv_cache_write(dev, be.upload(src), at)
        orc.kv_cache_write(want, src, at)
        assert dev.numpy().tobytes() == want.tobytes(), (at, tn)
    odd = be.upload(rng.standard_normal((1, 4, 1, 3)).astype(np.float32))      # a 3-float step takes the scalar path
    src = rng.standard_normal((1, 2, 1, 3)).astype(np.float32)
    be.kv_cache_write(odd, be.upload(src), 3)
    assert np.array_equal(odd.numpy()[0, 3], src[0, 0]) and np.array_equal(odd.numpy()[0, 0], src[0, 1])
    with pytest.raises(OjasError) as e:
        be.kv_cache_write(dev, be.upload(np.zeros((2, 9, 3, 16), np.float32)), 0)
    assert e.value.kind == "OutOfRange"
    with pytest.raises(OjasError) as e:
        be.kv_cache_write(dev, be.upload(np.zeros((2, 2, 2, 16), np.float32)), 0)
    assert e.value.kind == "Shape"


@pytest.mark.parametrize("case", [
    dict(b=2, tq=1, h=4, hkv=4, d=64, cap=64, kv_len=37, window=None),      # one decode step on a prefix
    dict(b=1, tq=5, h=6, hkv=2, d=32, cap=48, kv_len=48, window=None),      # prefill onto a non-empty cache, GQA, full ring
    dict(b=2, tq=3, h=4, hkv=2, d=16, cap=16, kv_len=70, window=8),         # a ring that wrapped, sliding window
    dict(b=1, tq=4, h=2, hkv=1, d=128, cap=300, kv_len=4, window=None),     # kv_len == Tq: equals causal_sdpa_forward
    dict(b=1, tq=2, h=2, hkv=2, d=64, cap=1024, kv_len=900, window=1000),   # a window wider than the history is no window
])
def test_cached_attention_matches_the_per_row_kernel(be, case):
    c = case
    rng = np.random.default_rng(7)
    q = rng.standard_normal((c["b"], c["tq"], c["h"], c["d"])).astype(np.float32)
    kc = rng.standard_normal((c["b"], c["cap"], c["hkv"], c["d"])).astype(np.float32)
    vc = rng.standard_normal((c["b"], c["cap"], c["hkv"], c["d"])).astype(np.float32)
    if c["kv_len"] < c["cap"]:
        kc[:, c["kv_len"]:] = np.nan          # slots no query reads may hold anything (ojas-cpu/src/kv.rs:4-7)
        vc[:, c["kv_len"]:] = np.inf
    got = be.cached_attention_forward(be.upload(q), be.upload(kc), be.upload(vc), c["kv_len"], c["window"]).numpy()
    be.sync()
    want = orc.cached_attention_forward(q, np.nan_to_num(kc, nan=0.0, posinf=0.0), np.nan_to_num(vc, nan=0.0, posinf=0.0), c["kv_len"], c["window"])
    assert got.shape == want.shape and rel(got, want) <= 1e-5, rel(got, want)
    if c["kv_len"] == c["tq"]:           # the documented identity with causal_sdpa_forward after the layout permute
        k = np.ascontiguousarray(kc[:, :c["kv_len"]].transpose(0, 2, 1, 3)); v = np.ascontiguousarray(vc[:, :c["kv_len"]].transpose(0, 2, 1, 3))
        ref, _ = orc.causal_sdpa_forward(np.ascontiguousarray(q.transpose(0, 2, 1, 3)), k, v)
        assert np.array_equal(want, ref.transpose(0, 2, 1, 3))


def test_cached_attention_refusals(be):
    from ojas_b200 import OjasError
    q = be.upload(np.zeros((1, 2, 4, 16), np.float32))
    kc = be.upload(np.zeros((1, 8, 2, 16), np.float32))
    for kv_len, window, kind in ((1, None, "OutOfRange"), (9, None, "OutOfRange"), (20, 8, "OutOfRange"), (8, 0, "Shape")):
        with pytest.raises(OjasError) as e:
            be.cached_attention_forward(q, kc, kc, kv_len, window)
        assert e.value.kind == kind, (kv_len, window)
    assert be.cached_attention_forward(q, kc, kc, 20, 7).shape == (1, 2, 4, 16)      # span 2 + 7 - 1 = 8 positions fit the ring
    poisoned = np.zeros((1, 8, 2, 16), np.float32)
    poisoned[0, 3, 1, 2] = np.nan
    be.cached_attention_forward(q, be.upload(poisoned), kc, 8, None)
    with pytest.raises(OjasError) as e:
        be.sync()
    assert e.value.kind == "NonFinite"


@pytest.mark.parametrize("bf16", [False, True])
def test_fused_linear_cross_entropy_with_ignore_and_a_collapsed_row(be, bf16):
    """The fused tied-head loss with an ignore index and a row whose softmax rounds to one-hot (the target-excluded form of
    ojas-cpu/src/fused_ce.rs:22-29): loss, both gradients, zero gradient rows where the target is ignored; every target ignored
    has no mean (NonFinite at the next sync)."""
    from ojas_b200 import DType, OjasError
    rows, dim, vocab, ignore = 300, 64, 1000, 11
    x, w = rnd(1, (rows, dim)), rnd(2, (vocab, dim), 0.3)
    rng = orc.SplitMix64(3)
    targets = np.array([ignore if i % 7 == 2 else rng.below(vocab) for i in range(rows)], np.uint32)
    x[5] = 24.0 * w[targets[5]] / np.linalg.norm(w[targets[5]])     # one logit far above the rest: the row collapses
    if bf16:
        x, w = orc.round_bf16(x), orc.round_bf16(w)
    oloss, ogx, ogw = orc.linear_cross_entropy_mean(x, w, targets, ignore=ignore)
    dt = DType.BF16 if bf16 else DType.F32
    loss, gx, gw = be.linear_cross_entropy_mean(be.upload(x, dt), be.upload(w, dt), be.upload(targets), ignore_index=ignore, chunk=(128, 0), grad_input_dtype=DType.F32)
    assert abs(loss.numpy()[0] - oloss) <= (5e-4 if bf16 else FWD_TOL) * abs(oloss)
    tol = 1e-2 if bf16 else GRAD_TOL
    assert rel(gx.numpy(), ogx) <= tol and rel(gw.numpy(), ogw) <= tol
    assert not np.any(gx.numpy()[targets == ignore])
    with pytest.raises(OjasError) as e:
        be.linear_cross_entropy_mean(be.upload(x, dt), be.upload(w, dt), be.upload(np.full(rows, ignore, np.uint32)), ignore_index=ignore)
        be.sync()
    assert e.value.kind == "NonFinite"


def test_linear_backward_input_on_the_tensor_core_tier(be):
    from ojas_b200 import DType
    rows, kin, nout = 384, 768, 520
    w, gy = orc.round_bf16(rnd(12, (nout, kin), 0.5)), orc.round_bf16(rnd(13, (rows, nout), 0.5))
    ogx = orc.gemm(gy, w)
    gx = be.linear_backward_input(be.upload(w, DType.BF16), be.upload(gy, DType.BF16), out_dtype=DType.F32)
    assert rel(gx.numpy(), ogx) <= FWD_TOL


def test_accumulate_grad_refuses_a_non_finite_sum(be):
    """accumulate_grad never stores a sum that is not finite (ojas-cpu/src/accum.rs:33-115); on the device the refusal is the deferred
    fault the next sync reports, and the elements whose sums are finite are the ordinary sums."""
    from ojas_b200 import OjasError
    for n in (4096, 4099):                      # the 128-bit and the scalar forms
        a, g = rnd(1, (n,)), rnd(2, (n,))
        a[17], g[100], g[200] = 3.0e38, np.inf, np.nan
        g[17] = 3.0e38                           # finite operands, overflowing sum
        acc = be.upload(a)
        be.accumulate_grad(acc, be.upload(g))
        with pytest.raises(OjasError) as e:
            be.sync()
        assert e.value.kind == "NonFinite" and "accumulate_grad" in str(e.value)
        got, bad = acc.numpy(), np.array([17, 100, 200])
        assert np.array_equal(got[bad], a[bad])
        keep = np.ones(n, bool); keep[bad] = False
        assert np.array_equal(got[keep], (a + g)[keep])
    be.sync()                                    # reported once: the fault word is clear again


def test_optimizer_scratch_bytes_bounds_what_a_step_takes(be):
    """optimizer_scratch_bytes (ojas-core/src/backend.rs:953) is the preflight bound of Trainer::new (trainer.rs:401-426): AdamW takes
    none, a Muon step's peak above the live bytes stays within the bound for both Newton-Schulz precisions."""
    from ojas_b200 import MuonNs5Config
    assert be.optimizer_scratch_bytes("adamw", 768, 2048) == 0
    for rows, cols in ((768, 768), (2048, 768), (12, 768), (768, 2048)):
        bound = be.optimizer_scratch_bytes("muon", rows, cols)
        assert bound >= rows * cols * 4
        for bf in (False, True):
            p, g, m = be.upload(rnd(1, (rows, cols), 0.02)), be.upload(rnd(2, (rows, cols), 0.01)), be.zeros((rows, cols))
            be.sync()
            live = be.budget()["live"]
            import ctypes as C
            from ojas_b200._lib import lib
            lib.ojc_reset_peak(be._handle)
            be.muon_ns5_step(p, g, m, MuonNs5Config(0.025, 0.95, 0.1, True, bf))
            be.sync()
            assert be.budget()["peak"] - live <= bound, (rows, cols, bf)


def test_a_host_wait_that_runs_out_is_a_retryable_wait_timeout(be):
    """Every host wait is bounded (RuntimeConfig::sync_timeout, ojas-cuda/src/runtime.rs:76): with a zero budget a sync behind queued
    work reports WaitTimeout, nothing is lost, and the next sync with the default budget succeeds."""
    from ojas_b200 import DType, OjasError
    x, w = be.upload(orc.round_bf16(rnd(1, (8192, 4096))), DType.BF16), be.upload(orc.round_bf16(rnd(2, (4096, 4096))), DType.BF16)
    be.sync()
    be.set_sync_timeout_ms(0)
    try:
        ys = [be.linear_forward(x, w) for _ in range(40)]          # about 10 ms of queued GEMMs
        with pytest.raises(OjasError) as e:
            be.sync()
        assert e.value.kind == "WaitTimeout" and e.value.retryable
    finally:
        be.set_sync_timeout_ms(60000)
    be.sync()
    want = orc.linear_forward(orc.round_bf16(rnd(1, (8192, 4096)))[:4], orc.round_bf16(rnd(2, (4096, 4096))))
    assert rel(ys[-1].numpy()[:4], want) <= 4e-3


def test_a_device_wait_that_runs_out_ends_the_kernel_in_order(be):
    """The bounded mbarrier wait of the tensor-pipeline kernels on a barrier nothing arrives on, with a one-millisecond limit: every
    thread gives up, the kernel returns, the next sync reports WaitTimeout, and the backend goes on working."""
    import ctypes as C
    from ojas_b200 import OjasError
    from ojas_b200._lib import lib
    from ojas_b200.backend import _check
    gave_up = C.c_int32(-1)
    with pytest.raises(OjasError) as e:
        _check(lib.ojc_selftest_bounded_wait(be._handle, C.c_uint64(2_000_000), C.byref(gave_up)))
    assert e.value.kind == "WaitTimeout" and gave_up.value == 64
    be.sync()
    a = be.upload(rnd(3, (64, 64)))
    assert np.array_equal(be.residual_add_forward(a, a).numpy(), rnd(3, (64, 64)) * 2)
