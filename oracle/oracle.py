"""ctypes/numpy face of the CPU oracle (libojas_oracle.so). TEST INFRASTRUCTURE ONLY.

Importable from tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs;
nothing under ojas_b200/ may import it. Each function restates one Backend
method of ojas's CPU reference under Numerics::Exact; the C++ side cites the
reference file:line it follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libojas_oracle.so"


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside this file."""
    if force or not _LIB_PATH.exists():
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _LIB_PATH


def _load() -> C.CDLL:
    build()
    lib = C.CDLL(str(_LIB_PATH))
    lib.orc_splitmix_next.restype = C.c_uint64
    lib.orc_splitmix_below.restype = C.c_uint64
    lib.orc_fnv1a_bytes.restype = C.c_uint64
    lib.orc_fnv1a_f32.restype = C.c_uint64
    lib.orc_param_count.restype = C.c_int64
    for name in ("orc_exp_exact", "orc_log_sum_exp_exact", "orc_log1p_exact", "orc_sigmoid_exact",
                 "orc_round_bf16", "orc_sdpa_scale"):
        getattr(lib, name).restype = C.c_float
    return lib


lib = _load()

STATUS = {0: "ok", 1: "Shape", 2: "NonFinite", 3: "OutOfRange"}


class OracleError(RuntimeError):
    def __init__(self, op: str, status: int):
        super().__init__(f"{op}: {STATUS.get(status, status)}")
        self.status = status
        self.kind = STATUS.get(status, str(status))


def _chk(op: str, st: int) -> None:
    if st != 0:
        raise OracleError(op, st)


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def _p(a: np.ndarray | None):
    return C.c_void_p(a.ctypes.data) if a is not None else C.c_void_p(0)


i64 = C.c_int64
f32 = C.c_float
f64 = C.c_double


# ------------------------------------------------------------------ generators
class SplitMix64:
    """ojas-test-support/src/rng.rs:15-45."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def next_u64(self) -> int:
        return lib.orc_splitmix_next(C.byref(self.state))

    def below(self, n: int) -> int:
        return lib.orc_splitmix_below(C.byref(self.state), C.c_uint64(n))

    def vec(self, n: int, scale: float) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib.orc_splitmix_vec(C.byref(self.state), i64(n), f32(scale), _p(out))
        return out


def fnv(values) -> int:
    v = _f(values).ravel()
    return lib.orc_fnv1a_f32(_p(v), i64(v.size))


def init_normal(name: str, seed: int, std: float, shape) -> np.ndarray:
    out = np.empty(int(np.prod(shape)), np.float32)
    lib.orc_init_normal(name.encode(), C.c_uint64(seed), f64(float(np.float32(std))), i64(out.size), _p(out))
    return out.reshape(shape)


def rope_tables(base: float, start: int, length: int, dim: int):
    cos = np.empty((length, dim), np.float32)
    sin = np.empty((length, dim), np.float32)
    lib.orc_rope_tables(f64(base), i64(start), i64(length), i64(dim), _p(cos), _p(sin))
    return cos, sin


def exp_exact(x: float) -> float:
    return lib.orc_exp_exact(f32(x))


def round_bf16(x) -> np.ndarray:
    x = _f(x)
    out = np.empty_like(x)
    lib.orc_round_bf16_vec(_p(x), i64(x.size), _p(out))
    return out


# ------------------------------------------------------------------ ops
def linear_forward(x, w):
    x, w = _f(x), _f(w)
    rows, kin, nout = x.size // x.shape[-1], x.shape[-1], w.shape[0]
    y = np.empty(x.shape[:-1] + (nout,), np.float32)
    _chk("linear_forward", lib.orc_linear_forward(_p(x), _p(w), i64(rows), i64(kin), i64(nout), _p(y)))
    return y


def linear_backward(x, w, gy):
    x, w, gy = _f(x), _f(w), _f(gy)
    rows, kin, nout = x.size // x.shape[-1], x.shape[-1], w.shape[0]
    gx, gw = np.empty_like(x), np.empty_like(w)
    _chk("linear_backward", lib.orc_linear_backward(_p(x), _p(w), _p(gy), i64(rows), i64(kin), i64(nout), _p(gx), _p(gw)))
    return gx, gw


def gemm(a, b):
    a, b = _f(a), _f(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    _chk("gemm", lib.orc_gemm(_p(a), i64(k), i64(1), _p(b), i64(n), i64(1), _p(c), i64(m), i64(k), i64(n), C.c_int(0)))
    return c


def rms_norm_forward(x, w, eps):
    x, w = _f(x), _f(w)
    dim = w.size
    y = np.empty_like(x)
    _chk("rms_norm_forward", lib.orc_rms_norm_forward(_p(x), _p(w), i64(x.size // dim), i64(dim), f32(eps), _p(y)))
    return y


def rms_norm_backward(x, w, gy, eps):
    x, w, gy = _f(x), _f(w), _f(gy)
    dim = w.size
    gx, gw = np.empty_like(x), np.empty_like(w)
    _chk("rms_norm_backward", lib.orc_rms_norm_backward(_p(x), _p(w), _p(gy), i64(x.size // dim), i64(dim), f32(eps), _p(gx), _p(gw)))
    return gx, gw


def rope(x, cos, sin, backward=False):
    """x [B,T,H,dh]; tables [T,dh] (RopeLayout::TimeDim)."""
    x, cos, sin = _f(x), _f(cos), _f(sin)
    b, t, h, dh = x.shape
    y = np.empty_like(x)
    _chk("rope", lib.orc_rope(_p(x), _p(cos), _p(sin), i64(b * t * h), i64(dh), i64(t), i64(h), C.c_int(int(backward)), _p(y)))
    return y


def causal_sdpa_forward(q, k, v, window=None):
    q, k, v = _f(q), _f(k), _f(v)
    b, h, t, d = q.shape
    hkv = k.shape[1]
    out = np.empty_like(q)
    lse = np.empty((b, h, t), np.float32)
    _chk("causal_sdpa_forward", lib.orc_causal_sdpa_forward(
        _p(q), _p(k), _p(v), i64(b), i64(h), i64(hkv), i64(t), i64(d), i64(-1 if window is None else window), _p(out), _p(lse)))
    return out, lse


def causal_sdpa_backward(q, k, v, out, lse, gy, window=None):
    q, k, v, out, lse, gy = map(_f, (q, k, v, out, lse, gy))
    b, h, t, d = q.shape
    hkv = k.shape[1]
    gq, gk, gv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    _chk("causal_sdpa_backward", lib.orc_causal_sdpa_backward(
        _p(q), _p(k), _p(v), _p(out), _p(lse), _p(gy), i64(b), i64(h), i64(hkv), i64(t), i64(d),
        i64(-1 if window is None else window), _p(gq), _p(gk), _p(gv)))
    return gq, gk, gv


def embedding_forward(table, ids):
    table, ids = _f(table), _u(ids)
    vocab, dim = table.shape
    out = np.empty(ids.shape + (dim,), np.float32)
    _chk("embedding_forward", lib.orc_embedding_forward(_p(table), _p(ids), i64(ids.size), i64(vocab), i64(dim), _p(out)))
    return out


def embedding_backward(vocab, ids, grad):
    ids, grad = _u(ids), _f(grad)
    dim = grad.shape[-1]
    out = np.empty((vocab, dim), np.float32)
    _chk("embedding_backward", lib.orc_embedding_backward(_p(ids), _p(grad), i64(ids.size), i64(vocab), i64(dim), _p(out)))
    return out


def silu_forward(x):
    x = _f(x)
    y = np.empty_like(x)
    lib.orc_silu_forward(_p(x), i64(x.size), _p(y))
    return y


def silu_backward(x, gy):
    x, gy = _f(x), _f(gy)
    gx = np.empty_like(x)
    lib.orc_silu_backward(_p(x), _p(gy), i64(x.size), _p(gx))
    return gx


def mul_forward(a, b):
    return (_f(a) * _f(b)).astype(np.float32)


def mul_backward(a, b, gy):
    return (_f(gy) * _f(b)).astype(np.float32), (_f(gy) * _f(a)).astype(np.float32)


def residual_add(a, b):
    return (_f(a) + _f(b)).astype(np.float32)


def permute_0213(x):
    return np.ascontiguousarray(np.transpose(_f(x), (0, 2, 1, 3)))


def gate_forward(inp, weight, bias, attn, want_scales=False):
    inp, weight, bias, attn = map(_f, (inp, weight, bias, attn))
    heads, din = weight.shape
    rows = inp.size // din
    dh = attn.size // (rows * heads)
    y = np.empty_like(attn)
    scales = np.empty((rows, heads), np.float32)
    _chk("gate_forward", lib.orc_gate_forward(_p(inp), _p(weight), _p(bias), _p(attn), i64(rows), i64(din), i64(heads), i64(dh), _p(y), _p(scales)))
    return (y, scales) if want_scales else y


def gate_backward(inp, weight, bias, attn, gy):
    inp, weight, bias, attn, gy = map(_f, (inp, weight, bias, attn, gy))
    heads, din = weight.shape
    rows = inp.size // din
    dh = attn.size // (rows * heads)
    gx, gw, gb, ga = np.empty_like(inp), np.empty_like(weight), np.empty_like(bias), np.empty_like(attn)
    _chk("gate_backward", lib.orc_gate_backward(_p(inp), _p(weight), _p(bias), _p(attn), _p(gy), i64(rows), i64(din), i64(heads), i64(dh), _p(gx), _p(gw), _p(gb), _p(ga)))
    return gx, gw, gb, ga


def vres_forward(v, v0, lam):
    v, v0 = _f(v), _f(v0)
    y = np.empty_like(v)
    lib.orc_vres_forward(_p(v), _p(v0), f32(lam), i64(v.size), _p(y))
    return y


def vres_backward(v, v0, gy, lam):
    v, v0, gy = _f(v), _f(v0), _f(gy)
    gv, gv0 = np.empty_like(v), np.empty_like(v)
    gl = C.c_float(0)
    lib.orc_vres_backward(_p(v), _p(v0), _p(gy), f32(lam), i64(v.size), _p(gv), _p(gv0), C.byref(gl))
    return gv, gv0, np.float32(gl.value)


def cross_entropy_mean(logits, targets, ignore=None, want_grad=False):
    logits, targets = _f(logits), _u(targets)
    rows, vocab = logits.shape
    loss = C.c_float(0)
    grad = np.empty_like(logits) if want_grad else None
    _chk("cross_entropy_mean", lib.orc_cross_entropy_mean(
        _p(logits), _p(targets), i64(rows), i64(vocab), C.c_int(ignore is not None), C.c_uint32(ignore or 0), C.byref(loss), _p(grad)))
    return (np.float32(loss.value), grad) if want_grad else np.float32(loss.value)


def linear_cross_entropy_mean(x, w, targets, ignore=None, want_grads=True):
    x, w, targets = _f(x), _f(w), _u(targets)
    rows, dim = x.shape
    vocab = w.shape[0]
    loss = C.c_float(0)
    gx = np.empty_like(x) if want_grads else None
    gw = np.empty_like(w) if want_grads else None
    _chk("linear_cross_entropy_mean", lib.orc_linear_cross_entropy_mean(
        _p(x), _p(w), _p(targets), i64(rows), i64(dim), i64(vocab), C.c_int(ignore is not None), C.c_uint32(ignore or 0),
        C.byref(loss), _p(gx), _p(gw)))
    return np.float32(loss.value), gx, gw


def argmax_rows(x):
    x = _f(x)
    rows, cols = x.shape
    out = np.empty(rows, np.uint32)
    _chk("argmax_rows", lib.orc_argmax_rows(_p(x), i64(rows), i64(cols), _p(out)))
    return out


def topk_rows(x, k):
    """ojas-core/src/backend.rs:1571-1612 with rank_logits (:186-195): value descending, +0.0 and -0.0 one value, -inf after
    every finite value, then column ascending. NaN or +inf in a row is refused."""
    x = _f(x)
    if np.isnan(x).any() or np.isposinf(x).any():
        raise OracleError("topk_rows", 2)
    rows, cols = x.shape
    key = np.where(x == 0.0, np.float32(0.0), x)
    # a stable sort of the negated key keeps equal values in column order
    order = np.argsort(-key.astype(np.float64), axis=1, kind="stable")[:, :k]
    return np.take_along_axis(x, order, axis=1), order.astype(np.uint32)


def kv_cache_write(cache, src, at):
    """ojas-cpu/src/kv.rs (kv_cache_write): position at + t of src [B, Tn, Hkv, D] goes to slot (at + t) % Tcap, in place."""
    cap = cache.shape[1]
    for t in range(src.shape[1]):
        cache[:, (at + t) % cap] = src[:, t]
    return cache


def cached_attention_forward(q, k_cache, v_cache, kv_len, window=None):
    """ojas-cpu/src/kv.rs:107-200: each query row runs the per-row kernel of causal_sdpa_forward over its visible positions,
    oldest first. Restated through that kernel: the ring is unrolled into positions first .. kv_len - 1, the new queries are
    the last Tq rows of a causal problem over them (earlier rows get zero queries and are dropped), under the same window."""
    q, k_cache, v_cache = _f(q), _f(k_cache), _f(v_cache)
    b, tq, h, d = q.shape
    cap, hkv = k_cache.shape[1], k_cache.shape[2]
    w = window if (window is not None and window < kv_len) else None
    first = max(0, kv_len - tq + 1 - w) if w else 0          # the oldest position any query reads
    pos = np.arange(first, kv_len)
    k = np.ascontiguousarray(k_cache[:, pos % cap].transpose(0, 2, 1, 3))      # [B, Hkv, n, D]
    v = np.ascontiguousarray(v_cache[:, pos % cap].transpose(0, 2, 1, 3))
    n = len(pos)
    qf = np.zeros((b, h, n, d), np.float32)
    qf[:, :, n - tq:] = q.transpose(0, 2, 1, 3)
    out, _ = causal_sdpa_forward(qf, k, v, window=w)
    return np.ascontiguousarray(out[:, :, n - tq:].transpose(0, 2, 1, 3))


def _ptr_array(arrs):
    return (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])


def clip_grad_norm(grads, max_norm):
    """In place on the float32 arrays of `grads`; returns the f32 norm before clipping."""
    for g in grads:
        assert g.dtype == np.float32 and g.flags.c_contiguous
    lens = (C.c_int64 * len(grads))(*[g.size for g in grads])
    norm = C.c_float(0)
    _chk("clip_grad_norm", lib.orc_clip_grad_norm(_ptr_array(grads), lens, i64(len(grads)), f32(max_norm), C.byref(norm)))
    return np.float32(norm.value)


def grad_norm(grads):
    grads = [_f(g) for g in grads]
    lens = (C.c_int64 * len(grads))(*[g.size for g in grads])
    norm = C.c_float(0)
    _chk("grad_norm", lib.orc_grad_norm(_ptr_array(grads), lens, i64(len(grads)), C.byref(norm)))
    return np.float32(norm.value)


def adamw_step(p, g, m, v, step_before, lr, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0):
    """In place on p, m, v (float32, contiguous)."""
    g = _f(g)
    _chk("adamw_step", lib.orc_adamw_step(_p(p), _p(g), _p(m), _p(v), i64(p.size), C.c_uint64(step_before),
                                           f64(lr), f64(beta1), f64(beta2), f64(eps), f64(weight_decay)))


def muon_ns5_step(p, g, mom, lr=0.025, momentum=0.99, weight_decay=0.1, nesterov=True, bf16=False):
    """In place on p and mom (float32 [rows, cols])."""
    g = _f(g)
    rows, cols = p.shape
    _chk("muon_ns5_step", lib.orc_muon_ns5_step(_p(p), _p(g), _p(mom), i64(rows), i64(cols), f64(lr), f64(momentum),
                                                 f64(weight_decay), C.c_int(int(nesterov)), C.c_int(int(bf16))))


def newton_schulz5(update, bf16=False):
    u = _f(update).copy()
    _chk("newton_schulz5", lib.orc_newton_schulz5(_p(u), i64(u.shape[0]), i64(u.shape[1]), C.c_int(int(bf16))))
    return u


# ------------------------------------------------------------------ model
class _Spec(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("vocab", "n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "hidden", "max_seq", "window")] + [
        ("rope_base", C.c_double), ("rms_eps", C.c_float)]


@dataclass
class Spec:
    """ojas-model/src/spec.rs:45 (ModelSpec); window=None is full causal attention."""
    vocab: int
    n_embd: int
    n_layer: int
    n_head: int
    n_kv_head: int
    head_dim: int
    hidden: int
    max_seq: int
    window: int | None = None
    rope_base: float = 10000.0
    rms_eps: float = 1e-6

    def c(self) -> _Spec:
        return _Spec(self.vocab, self.n_embd, self.n_layer, self.n_head, self.n_kv_head, self.head_dim, self.hidden,
                     self.max_seq, -1 if self.window is None else self.window, self.rope_base, self.rms_eps)


@dataclass
class ParamInfo:
    name: str
    shape: tuple
    init: int  # 0 zeros, 1 ones, 2 normal
    group: int  # 0 AdamW, 1 Muon
    trains: bool


def param_table(spec: Spec) -> list[ParamInfo]:
    cs = spec.c()
    out = []
    for i in range(lib.orc_param_count(C.byref(cs))):
        name = C.create_string_buffer(128)
        rank, shape = C.c_int64(0), (C.c_int64 * 2)()
        init, group, trains = C.c_int(0), C.c_int(0), C.c_int(0)
        _chk("param_info", lib.orc_param_info(C.byref(cs), i64(i), name, i64(128), C.byref(rank), shape, C.byref(init), C.byref(group), C.byref(trains)))
        out.append(ParamInfo(name.value.decode(), tuple(shape[: rank.value]), init.value, group.value, bool(trains.value)))
    return out


def init_params(spec: Spec, seed: int, normal_everywhere: bool = False) -> list[np.ndarray]:
    """ojas-model/src/init.rs:73-110. normal_everywhere also draws o_proj / ffn.down from N(0, 0.02)."""
    out = []
    for info in param_table(spec):
        kind = info.init
        if normal_everywhere and len(info.shape) == 2:
            kind = 2
        if kind == 2:
            out.append(init_normal(info.name, seed, 0.02, info.shape))
        else:
            out.append(np.full(info.shape, float(kind), np.float32))
    return out


def forward_loss(spec: Spec, params, ids, targets, ignore=None, seed=1.0, want_grads=True, want_logits=False):
    """Loss, gradients (param_table order) and optionally logits [B*T, V]."""
    params = [_f(p) for p in params]
    ids, targets = _u(ids), _u(targets)
    b, t = ids.shape
    cs = spec.c()
    grads = [np.zeros_like(p) for p in params] if want_grads else None
    logits = np.empty((b * t, spec.vocab), np.float32) if want_logits else None
    loss = C.c_float(0)
    _chk("forward_loss", lib.orc_forward_loss(
        C.byref(cs), _ptr_array(params), _p(ids), _p(targets), i64(b), i64(t), C.c_int(ignore is not None), C.c_uint32(ignore or 0),
        f32(seed), C.byref(loss), _ptr_array(grads) if want_grads else C.c_void_p(0), _p(logits)))
    return np.float32(loss.value), grads, logits


def set_threads(n: int) -> int:
    """Run every later parallel region on n threads (CpuBackend::with_threads), whatever OMP_NUM_THREADS said at start-up
    (torch.distributed.run sets it to 1 for its children). Returns the count in force."""
    return int(lib.orc_set_threads(C.c_int(n)))


def max_threads() -> int:
    return int(lib.orc_max_threads())


def set_fast(on: bool) -> None:
    """Numerics::Fast for the timed CPU baseline (fused multiply-add products, f32 AdamW). Parity checks never switch it on."""
    lib.orc_set_fast(C.c_int(int(on)))


# ------------------------------------------------------------------ trainer (host logic of one optimizer step)
COSINE_FLOOR_FRAC = 0.1          # ojas-cpu/src/schedule.rs:27
MUON_MOMENTUM, MUON_WEIGHT_DECAY, ADAM_HYBRID_WEIGHT_DECAY = 0.99, 0.1, 0.0   # ojas-cpu/src/train.rs:31-37
MAX_CONSECUTIVE_SKIPS = 8        # ojas-model/src/trainer.rs:81


def lr_multiplier(schedule: str, warmup: int, total: int, step: int, decay_frac: float = 0.2) -> float:
    """LrSchedule::multiplier (ojas-cpu/src/schedule.rs:66-90 cosine, 163-199 wsd): every line an f64 operation in the
    reference's order. A step past `total` is refused by wsd and clamped by cosine."""
    import math
    if step < warmup:
        return (float(step) + 1.0) / float(warmup)
    if schedule == "cosine":
        span = float(total) - float(warmup)
        denom = 1.0 if span < 1.0 else span
        t = min(max((float(step) - float(warmup)) / denom, 0.0), 1.0)
        return COSINE_FLOOR_FRAC + (1.0 - COSINE_FLOOR_FRAC) * 0.5 * (1.0 + math.cos(math.pi * t))
    if schedule == "wsd":
        if step > total:
            raise OracleError("wsd_schedule", 3)
        decay_steps = int(decay_frac * float(total))
        decay_start = total - decay_steps
        if step < decay_start:
            return 1.0
        frac = float(step - decay_start) / float(max(decay_steps, 1))
        return COSINE_FLOOR_FRAC + (1.0 - COSINE_FLOOR_FRAC) * (1.0 - frac)
    raise ValueError(schedule)


def micro_weights(counts):
    """MicroWeights::new (ojas-model/src/trainer.rs:1083-1119): (f32 weights, uniform, run). No valid target at all is NonFinite."""
    total = sum(counts)
    live = [n for n in counts if n > 0]
    if not live:
        raise OracleError("Trainer::step", 4)
    run, first = len(live), live[0]
    uniform = all(n == 0 or n == first for n in counts)
    weights = [np.float32(0.0) if n == 0 else (np.float32(1.0) / np.float32(run) if uniform else np.float32(float(n) / float(total))) for n in counts]
    return weights, uniform, run


class TrainerOracle:
    """Trainer::run (ojas-model/src/trainer.rs:754-1046) on the CPU oracle: K micro-batches seeded by MicroWeights, gradients
    summed in f32 in micro-batch order, global-norm clip, then per slot Muon NS5 (rank-2 hidden weights) or AdamW without decay
    (embedding, vectors) at the schedule's learning rates; a non-finite norm leaves everything unchanged."""

    def __init__(self, spec: Spec, params, schedule=("cosine", 0, 1), matrix_lr=0.025, adam_lr=6e-4, grad_clip=1.0, ns5_bf16=False,
                 muon_momentum=MUON_MOMENTUM, ignore=None):
        self.spec, self.table = spec, param_table(spec)
        self.params = [np.array(p, np.float32, copy=True) for p in params]
        self.schedule, self.matrix_lr, self.adam_lr, self.grad_clip = schedule, matrix_lr, adam_lr, grad_clip
        self.ns5_bf16, self.muon_momentum, self.ignore = ns5_bf16, muon_momentum, ignore
        self.m = [np.zeros_like(p) for p in self.params]
        self.v = [np.zeros_like(p) for p in self.params]
        self.step = 0

    def run(self, batches):
        """batches: [(x [B, T], y [B, T])]; returns (loss, grad_norm, lr_multiplier)."""
        kind, warmup, total = self.schedule[:3]
        mult = lr_multiplier(kind, warmup, total, self.step, *self.schedule[3:])
        counts = [int(np.count_nonzero(_u(y) != self.ignore)) if self.ignore is not None else int(np.asarray(y).size) for _, y in batches]
        weights, uniform, run = micro_weights(counts)
        acc, loss_sum = None, None
        for (x, y), w in zip(batches, weights):
            if w == 0.0:
                continue
            loss, grads, _ = forward_loss(self.spec, self.params, x, y, ignore=self.ignore, seed=float(w))
            acc = grads if acc is None else [(a + g).astype(np.float32) for a, g in zip(acc, grads)]
            lv = np.float32(loss) if uniform or w == 1.0 else np.float32(np.float32(loss) * w)
            loss_sum = lv if loss_sum is None else np.float32(loss_sum + lv)
        train = [i for i, info in enumerate(self.table) if info.trains]
        flat = [np.ascontiguousarray(acc[i]) for i in train]
        norm = clip_grad_norm(flat, self.grad_clip)
        if not np.isfinite(norm):
            raise OracleError("clip_grad_norm", 4)
        for i, g in zip(train, flat):
            info, p = self.table[i], self.params[i]
            if info.group == 1:
                muon_ns5_step(p, g.reshape(p.shape), self.m[i], lr=self.matrix_lr * mult, momentum=self.muon_momentum, weight_decay=MUON_WEIGHT_DECAY,
                              bf16=self.ns5_bf16)
            else:
                adamw_step(p.reshape(-1), g.ravel(), self.m[i].reshape(-1), self.v[i].reshape(-1), self.step, self.adam_lr * mult, weight_decay=ADAM_HYBRID_WEIGHT_DECAY)
        self.step += 1
        loss = np.float32(loss_sum / np.float32(run)) if uniform else loss_sum
        return float(loss), float(norm), mult
