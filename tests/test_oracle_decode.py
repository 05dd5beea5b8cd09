"""The oracle's restatements of the decode ops, checked on the CPU against independent f64 arithmetic and the rules the
reference documents (ojas-core/src/backend.rs:186-195 rank_logits, :2521-2565; ojas-cpu/src/kv.rs:1-19)."""
import numpy as np
import pytest

from oracle import oracle as orc


def test_topk_rows_order_is_value_descending_then_column_ascending():
    x = np.array([[1.0, 3.0, 3.0, -np.inf, 0.0, -0.0, 2.0], [-0.0, 0.0, -1.0, -np.inf, -np.inf, 5.0, 0.0]], np.float32)
    values, ids = orc.topk_rows(x, 7)
    assert ids.tolist() == [[1, 2, 6, 0, 4, 5, 3], [5, 0, 1, 6, 2, 3, 4]]
    assert values.tobytes() == np.take_along_axis(x, ids.astype(np.int64), 1).tobytes()      # -0.0 keeps its own bits
    assert orc.topk_rows(x, 2)[1].tolist() == [[1, 2], [5, 0]]
    for bad in (np.nan, np.inf):
        y = x.copy()
        y[0, 0] = bad
        with pytest.raises(orc.OracleError):
            orc.topk_rows(y, 1)


def test_kv_cache_write_wraps_the_ring():
    cache = np.zeros((1, 4, 1, 2), np.float32)
    src = np.arange(12, dtype=np.float32).reshape(1, 3, 1, 4)[..., :2].copy()
    orc.kv_cache_write(cache, src, 3)                      # positions 3, 4, 5 -> slots 3, 0, 1
    assert cache[0, 3, 0].tolist() == src[0, 0, 0].tolist() and cache[0, 0, 0].tolist() == src[0, 1, 0].tolist() and cache[0, 1, 0].tolist() == src[0, 2, 0].tolist()
    assert not cache[0, 2].any()


@pytest.mark.parametrize("b,tq,h,hkv,d,cap,kv_len,window", [(2, 3, 4, 2, 16, 16, 70, 8), (1, 5, 6, 2, 32, 48, 48, None), (2, 1, 4, 4, 64, 64, 37, None), (1, 2, 2, 1, 8, 8, 2, 5)])
def test_cached_attention_equals_plain_softmax_attention_over_the_visible_positions(b, tq, h, hkv, d, cap, kv_len, window):
    rng = np.random.default_rng(1)
    q = rng.standard_normal((b, tq, h, d)).astype(np.float32)
    kc, vc = (rng.standard_normal((b, cap, hkv, d)).astype(np.float32) for _ in range(2))
    got = orc.cached_attention_forward(q, kc, vc, kv_len, window)
    want = np.zeros(q.shape, np.float64)
    for bb in range(b):
        for i in range(tq):
            p = kv_len - tq + i
            lo = max(0, p + 1 - window) if window else 0
            js = np.arange(lo, p + 1) % cap
            for hh in range(h):
                k, v = kc[bb, js, hh // (h // hkv)].astype(np.float64), vc[bb, js, hh // (h // hkv)].astype(np.float64)
                s = k @ q[bb, i, hh].astype(np.float64) / np.sqrt(d)
                pr = np.exp(s - s.max())
                want[bb, i, hh] = (pr / pr.sum()) @ v
    assert np.abs(got - want).max() <= 2e-6
