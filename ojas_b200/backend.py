"""Host-side mirror of the reference's operator interface for the training-step path.

`CudaBackend` carries one method per `ojas_core::Backend` method the step exercises (same
names and argument meaning as ojas-core/src/backend.rs:889-2634); each forwards to the C ABI of
libojas_cuda.so. Errors surface as `OjasError` with the reference's variant names
(ojas-core/src/error.rs:18-118). Nothing here computes: a backend that cannot open raises.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from enum import IntEnum

import numpy as np

from . import _lib
from ._lib import CTensor, lib

STATUS_NAMES = ["Ok", "Shape", "Dtype", "OutOfRange", "NonFinite", "UnsupportedHeadDim", "CapacityExceeded", "Poisoned",
                "DeviceLost", "WaitTimeout", "Backend", "Unsupported", "Placement", "NoDevice"]


class OjasError(RuntimeError):
    """`kind` is the OjasError variant name; `retryable` follows error.rs:47-95 (WaitTimeout only)."""

    def __init__(self, status: int, detail: str):
        self.status = status
        self.kind = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else f"Status{status}"
        self.detail = detail
        self.retryable = self.kind == "WaitTimeout"
        super().__init__(f"{self.kind}: {detail}")


def _check(status: int) -> None:
    if status != 0:
        raise OjasError(status, lib.ojc_last_error().decode(errors="replace"))


class DType(IntEnum):
    F32 = 0
    BF16 = 1
    F16 = 2
    U32 = 3

    @property
    def size(self) -> int:
        return 2 if self in (DType.BF16, DType.F16) else 4


def _contig_strides(shape):
    strides, acc = [], 1
    for d in reversed(shape):
        strides.append(acc)
        acc *= d
    return tuple(reversed(strides))


class Tensor:
    """Shape + dtype + a device buffer owned by the backend (ojas-core/src/tensor.rs:20-55). Views share storage."""

    def __init__(self, backend: "CudaBackend", ptr: int, shape, dtype: DType, strides=None, owner: "Tensor | None" = None):
        self.backend, self.ptr, self.shape, self.dtype = backend, ptr, tuple(int(s) for s in shape), DType(dtype)
        self.strides = tuple(strides) if strides is not None else _contig_strides(self.shape)
        self._owner = owner  # keeps the storage alive for views
        self._owns = owner is None

    def __del__(self):
        if getattr(self, "_owns", False) and self.ptr and self.backend is not None and self.backend._handle:
            lib.ojc_free(self.backend._handle, C.c_void_p(self.ptr))
            self.ptr = 0

    @property
    def numel(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    def c(self) -> CTensor:
        t = CTensor()
        t.data, t.dtype, t.rank = self.ptr, int(self.dtype), len(self.shape)
        for i, (s, st) in enumerate(zip(self.shape, self.strides)):
            t.shape[i], t.stride[i] = s, st
        return t

    def reshape(self, shape) -> "Tensor":
        shape = tuple(int(s) for s in shape)
        assert int(np.prod(shape)) == self.numel and self.strides == _contig_strides(self.shape)
        return Tensor(self.backend, self.ptr, shape, self.dtype, owner=self._owner or self)

    def permuted(self, dims) -> "Tensor":
        """A strided view (no copy); only the attention family accepts it."""
        return Tensor(self.backend, self.ptr, [self.shape[d] for d in dims], self.dtype, [self.strides[d] for d in dims], owner=self._owner or self)

    def numpy(self) -> np.ndarray:
        return self.backend.download(self)


def _dt(choice, default):
    return default if choice is None else choice


def _p(t: "Tensor | None"):
    return C.byref(t.c()) if t is not None else None


@dataclass
class AdamWConfig:
    """AdamWConfig::nanolab (ojas-core/src/backend.rs:494-546)."""
    lr: float
    weight_decay: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8

    def c(self):
        return _lib.AdamWConfig(self.lr, self.beta1, self.beta2, self.eps, self.weight_decay)


@dataclass
class MuonNs5Config:
    """MuonNs5Config::nanolab_default (ojas-core/src/backend.rs:548-570)."""
    lr: float = 0.025
    momentum: float = 0.99
    weight_decay: float = 0.1
    nesterov: bool = True
    ns5_bf16: bool = False

    def c(self):
        return _lib.MuonConfig(self.lr, self.momentum, self.weight_decay, int(self.nesterov), int(self.ns5_bf16))


class CudaBackend:
    """`impl Backend for CudaBackend` on B200. Opening refuses anything but an sm_100 device; there is no host path."""

    def __init__(self, device: int = 0, budget_bytes: int = 160 << 30):
        self._handle = None
        h = C.c_void_p()
        _check(lib.ojc_open(C.c_int32(device), C.c_uint64(budget_bytes), C.byref(h)))
        self._handle = h

    @classmethod
    def _adopt(cls, handle) -> "CudaBackend":
        """A view of a backend some other owner opens and closes (a Session's owner thread)."""
        be = cls.__new__(cls)
        be._handle, be._borrowed = C.c_void_p(handle), True
        return be

    def close(self):
        if self._handle:
            if not getattr(self, "_borrowed", False):
                lib.ojc_close(self._handle)
            self._handle = None

    def __del__(self):
        self.close()

    # ---- BackendCore
    def id(self) -> str:
        return "cuda"

    def numerics(self) -> str:
        return "Fast"

    def bf16_operands(self) -> bool:
        return True

    def budget(self) -> dict:
        cap, live, peak = C.c_uint64(), C.c_uint64(), C.c_uint64()
        _check(lib.ojc_budget(self._handle, C.byref(cap), C.byref(live), C.byref(peak)))
        return {"cap": cap.value, "live": live.value, "peak": peak.value}

    def device_readbacks(self) -> int:
        n = C.c_uint64()
        lib.ojc_readbacks(self._handle, C.byref(n))
        return n.value

    def kernel_launches(self) -> int:
        return int(lib.ojc_kernel_launches(self._handle))

    def stream(self) -> int:
        return int(lib.ojc_stream(self._handle) or 0)

    def profile_gemm(self, enable: bool):
        _check(lib.ojc_profile_gemm(self._handle, C.c_int32(int(enable))))

    def profile_gemm_read(self):
        """(device milliseconds, 2mnk flops, launches) of the tensor-core GEMMs since the last read."""
        ms, fl, n = C.c_double(), C.c_double(), C.c_uint64()
        _check(lib.ojc_profile_gemm_read(self._handle, C.byref(ms), C.byref(fl), C.byref(n)))
        return ms.value, fl.value, n.value

    def profile_gemm_read_split(self):
        """The same in two parts: ((ms, flops, launches) of the plain products, the same of the launches with SwiGLU in their epilogue)."""
        v = [C.c_double(), C.c_double(), C.c_uint64(), C.c_double(), C.c_double(), C.c_uint64()]
        _check(lib.ojc_profile_gemm_read_split(self._handle, *(C.byref(x) for x in v)))
        return (v[0].value, v[1].value, v[2].value), (v[3].value, v[4].value, v[5].value)

    def stream_wait_event(self, stream_ptr: int, event_ptr: int):
        _check(lib.ojc_stream_wait_event(self._handle, C.c_void_p(stream_ptr), C.c_void_p(event_ptr)))

    def set_sync_timeout_ms(self, ms: int):
        lib.ojc_set_sync_timeout_ms(self._handle, C.c_uint64(ms))

    def empty(self, shape, dtype: DType = DType.F32) -> Tensor:
        shape = tuple(int(s) for s in shape)
        n = int(np.prod(shape)) if shape else 1
        ptr = C.c_void_p()
        _check(lib.ojc_alloc(self._handle, C.c_uint64(max(n, 1) * DType(dtype).size), C.byref(ptr)))
        return Tensor(self, ptr.value, shape, dtype)

    def zeros(self, shape, dtype: DType = DType.F32) -> Tensor:
        t = self.empty(shape, dtype)
        _check(lib.ojc_fill_zero(self._handle, C.c_void_p(t.ptr), C.c_uint64(t.numel * t.dtype.size)))
        return t

    def upload(self, array: np.ndarray, dtype: DType | None = None) -> Tensor:
        """Host array -> device tensor. float32 -> F32 (or BF16 when asked, rounded on the device), uint32 -> U32."""
        array = np.ascontiguousarray(array)
        if array.dtype == np.uint32 or array.dtype == np.int64 or array.dtype == np.int32:
            array = array.astype(np.uint32)
            t = self.empty(array.shape, DType.U32)
        else:
            array = array.astype(np.float32, copy=False)
            t = self.empty(array.shape, DType.F32)
        _check(lib.ojc_upload(self._handle, C.c_void_p(t.ptr), C.c_void_p(array.ctypes.data), C.c_uint64(array.nbytes)))
        if dtype == DType.BF16:
            return self.to_bf16(t)
        return t

    def upload_ptr(self, t: Tensor, host_ptr: int, nbytes: int):
        """Copy from a caller-owned (for example pinned) host buffer given by address into an existing tensor."""
        _check(lib.ojc_upload(self._handle, C.c_void_p(t.ptr), C.c_void_p(host_ptr), C.c_uint64(nbytes)))

    def download(self, t: Tensor) -> np.ndarray:
        assert t.strides == _contig_strides(t.shape), "download wants a contiguous tensor"
        if t.dtype == DType.BF16:
            t = self.to_f32(t)
        out = np.empty(t.shape, np.uint32 if t.dtype == DType.U32 else np.float32)
        _check(lib.ojc_download(self._handle, C.c_void_p(out.ctypes.data), C.c_void_p(t.ptr), C.c_uint64(out.nbytes)))
        return out

    def sync(self):
        _check(lib.ojc_sync(self._handle))

    def cast_bf16(self, x: Tensor) -> Tensor:
        y = self.empty(x.shape, DType.F32)
        _check(lib.ojc_cast_bf16(self._handle, _p(x), _p(y)))
        return y

    def to_bf16(self, x: Tensor) -> Tensor:
        y = self.empty(x.shape, DType.BF16)
        _check(lib.ojc_to_bf16(self._handle, _p(x), _p(y)))
        return y

    def to_f32(self, x: Tensor) -> Tensor:
        y = self.empty(x.shape, DType.F32)
        _check(lib.ojc_to_f32(self._handle, _p(x), _p(y)))
        return y

    # ---- BackendModule
    def embedding_forward(self, table: Tensor, ids: Tensor, out_dtype: DType | None = None) -> Tensor:
        out = self.empty(ids.shape + (table.shape[1],), _dt(out_dtype, table.dtype))
        _check(lib.ojc_embedding_forward(self._handle, _p(table), _p(ids), _p(out)))
        return out

    def embedding_backward(self, table: Tensor, ids: Tensor, grad_out: Tensor) -> Tensor:
        g = self.empty(table.shape, DType.F32)
        _check(lib.ojc_embedding_backward(self._handle, _p(table), _p(ids), _p(grad_out), _p(g)))
        return g

    def linear_forward(self, x: Tensor, weight: Tensor, out_dtype: DType | None = None) -> Tensor:
        y = self.empty(x.shape[:-1] + (weight.shape[0],), _dt(out_dtype, x.dtype))
        _check(lib.ojc_linear_forward(self._handle, _p(x), _p(weight), _p(y)))
        return y

    def linear_backward(self, x: Tensor, weight: Tensor, grad_y: Tensor, out_dtype: DType | None = None):
        gx, gw = self.empty(x.shape, _dt(out_dtype, x.dtype)), self.empty(weight.shape, DType.F32)
        _check(lib.ojc_linear_backward(self._handle, _p(x), _p(weight), _p(grad_y), _p(gx), _p(gw)))
        return gx, gw

    def linear_backward_input(self, weight: Tensor, grad_y: Tensor, out_dtype: DType | None = None) -> Tensor:
        gx = self.empty(grad_y.shape[:-1] + (weight.shape[1],), _dt(out_dtype, grad_y.dtype))
        _check(lib.ojc_linear_backward_input(self._handle, _p(weight), _p(grad_y), _p(gx)))
        return gx

    def rms_norm_forward(self, x: Tensor, weight: Tensor, eps: float, out_dtype: DType | None = None) -> Tensor:
        y = self.empty(x.shape, _dt(out_dtype, x.dtype))
        _check(lib.ojc_rms_norm_forward(self._handle, _p(x), _p(weight), C.c_float(eps), _p(y)))
        return y

    def rms_norm_backward(self, x: Tensor, weight: Tensor, grad_y: Tensor, eps: float):
        gx, gw = self.empty(x.shape, x.dtype), self.empty(weight.shape, DType.F32)
        _check(lib.ojc_rms_norm_backward(self._handle, _p(x), _p(weight), _p(grad_y), C.c_float(eps), _p(gx), _p(gw)))
        return gx, gw

    def rms_qk_norm_forward(self, q, k, q_weight, k_weight, eps):
        qo, ko = self.empty(q.shape, q.dtype), self.empty(k.shape, k.dtype)
        _check(lib.ojc_rms_qk_norm_forward(self._handle, _p(q), _p(k), _p(q_weight), _p(k_weight), C.c_float(eps), _p(qo), _p(ko)))
        return qo, ko

    def rms_qk_norm_backward(self, q, k, q_weight, k_weight, grad_q, grad_k, eps):
        gq, gk = self.empty(q.shape, q.dtype), self.empty(k.shape, k.dtype)
        gqw, gkw = self.empty(q_weight.shape), self.empty(k_weight.shape)
        _check(lib.ojc_rms_qk_norm_backward(self._handle, _p(q), _p(k), _p(q_weight), _p(k_weight), _p(grad_q), _p(grad_k), C.c_float(eps),
                                            _p(gq), _p(gk), _p(gqw), _p(gkw)))
        return gq, gk, gqw, gkw

    def rope_half_split_forward(self, x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        y = self.empty(x.shape, x.dtype)
        _check(lib.ojc_rope_half_split_forward(self._handle, _p(x), _p(cos), _p(sin), _p(y)))
        return y

    def rope_half_split_backward(self, grad_y: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
        gx = self.empty(grad_y.shape, grad_y.dtype)
        _check(lib.ojc_rope_half_split_backward(self._handle, _p(grad_y), _p(cos), _p(sin), _p(gx)))
        return gx

    def value_residual_blend_forward(self, v: Tensor, v0: Tensor, lam: Tensor) -> Tensor:
        y = self.empty(v.shape, v.dtype)
        _check(lib.ojc_value_residual_blend_forward(self._handle, _p(v), _p(v0), _p(lam), _p(y)))
        return y

    def value_residual_blend_backward(self, v: Tensor, v0: Tensor, lam: Tensor, grad_y: Tensor):
        gv, gv0, gl = self.empty(v.shape, grad_y.dtype), self.empty(v.shape, grad_y.dtype), self.empty((1,))
        _check(lib.ojc_value_residual_blend_backward(self._handle, _p(v), _p(v0), _p(lam), _p(grad_y), _p(gv), _p(gv0), _p(gl)))
        return gv, gv0, gl

    def permute(self, x: Tensor, dims) -> Tensor:
        y = self.empty([x.shape[d] for d in dims], x.dtype)
        arr = (C.c_int32 * len(dims))(*dims)
        _check(lib.ojc_permute(self._handle, _p(x), arr, C.c_int32(len(dims)), _p(y)))
        return y

    @staticmethod
    def _window(window):
        return C.c_int64(-1 if window is None else int(window))

    def causal_sdpa_forward(self, q: Tensor, k: Tensor, v: Tensor, window=None):
        out = self.empty(q.shape, q.dtype)
        lse = self.empty(q.shape[:3], DType.F32)
        _check(lib.ojc_causal_sdpa_forward(self._handle, _p(q), _p(k), _p(v), self._window(window), _p(out), _p(lse)))
        return out, lse

    def causal_sdpa_backward(self, q, k, v, output, lse, grad_output, window=None):
        gq, gk, gv = self.empty(q.shape, q.dtype), self.empty(k.shape, k.dtype), self.empty(v.shape, v.dtype)
        _check(lib.ojc_causal_sdpa_backward(self._handle, _p(q), _p(k), _p(v), _p(output), _p(lse), _p(grad_output), self._window(window), _p(gq), _p(gk), _p(gv)))
        return gq, gk, gv

    def causal_sdpa_backward_recompute(self, q, k, v, grad_output, window=None):
        gq, gk, gv = self.empty(q.shape, q.dtype), self.empty(k.shape, k.dtype), self.empty(v.shape, v.dtype)
        _check(lib.ojc_causal_sdpa_backward_recompute(self._handle, _p(q), _p(k), _p(v), _p(grad_output), self._window(window), _p(gq), _p(gk), _p(gv)))
        return gq, gk, gv

    def per_head_sigmoid_gate_forward(self, inp, weight, bias, attn) -> Tensor:
        out = self.empty(attn.shape, attn.dtype)
        _check(lib.ojc_per_head_sigmoid_gate_forward(self._handle, _p(inp), _p(weight), _p(bias), _p(attn), _p(out), None))
        return out

    def per_head_sigmoid_gate_forward_saving(self, inp, weight, bias, attn):
        out = self.empty(attn.shape, attn.dtype)
        rows = inp.numel // weight.shape[1]
        scales = self.empty((rows, weight.shape[0]), DType.F32)
        _check(lib.ojc_per_head_sigmoid_gate_forward(self._handle, _p(inp), _p(weight), _p(bias), _p(attn), _p(out), _p(scales)))
        return out, scales

    def per_head_sigmoid_gate_backward(self, inp, weight, bias, attn, grad_out, saved_scales=None, grad_input_dtype=None):
        gi, gw, gb, ga = self.empty(inp.shape, _dt(grad_input_dtype, inp.dtype)), self.empty(weight.shape), self.empty(bias.shape), self.empty(attn.shape, attn.dtype)
        _check(lib.ojc_per_head_sigmoid_gate_backward(self._handle, _p(inp), _p(weight), _p(bias), _p(attn), _p(grad_out), _p(saved_scales), _p(gi), _p(gw), _p(gb), _p(ga)))
        return gi, gw, gb, ga

    per_head_sigmoid_gate_backward_saved = per_head_sigmoid_gate_backward

    def _unary(self, fn, x, out_dtype=None):
        y = self.empty(x.shape, _dt(out_dtype, x.dtype))
        _check(fn(self._handle, _p(x), _p(y)))
        return y

    def silu_forward(self, x):
        return self._unary(lib.ojc_silu_forward, x)

    def silu_backward(self, x, grad_y):
        gx = self.empty(x.shape, x.dtype)
        _check(lib.ojc_silu_backward(self._handle, _p(x), _p(grad_y), _p(gx)))
        return gx

    def mul_forward(self, a, b):
        y = self.empty(a.shape, a.dtype)
        _check(lib.ojc_mul_forward(self._handle, _p(a), _p(b), _p(y)))
        return y

    def mul_backward(self, a, b, grad_y):
        ga, gb = self.empty(a.shape, a.dtype), self.empty(b.shape, b.dtype)
        _check(lib.ojc_mul_backward(self._handle, _p(a), _p(b), _p(grad_y), _p(ga), _p(gb)))
        return ga, gb

    def residual_add_forward(self, x, y):
        out = self.empty(x.shape, x.dtype)
        _check(lib.ojc_residual_add_forward(self._handle, _p(x), _p(y), _p(out)))
        return out

    def residual_add_backward(self, grad_out):
        gx, gy = self.empty(grad_out.shape, grad_out.dtype), self.empty(grad_out.shape, grad_out.dtype)
        _check(lib.ojc_residual_add_backward(self._handle, _p(grad_out), _p(gx), _p(gy)))
        return gx, gy

    def linear_cross_entropy_mean(self, x, weight, targets, ignore_index=None, chunk=(0, 0), grads=(True, True), grad_input_dtype=None):
        """LinearCe {loss, grad_input, grad_weight} (ojas-core/src/backend.rs:2513, CeChunk/CeGrads 3081-3136)."""
        loss = self.empty((1,), DType.F32)
        gx = self.empty(x.shape, _dt(grad_input_dtype, x.dtype)) if grads[0] else None
        gw = self.empty(weight.shape, DType.F32) if grads[1] else None
        _check(lib.ojc_linear_cross_entropy_mean(self._handle, _p(x), _p(weight), _p(targets), C.c_int32(ignore_index is not None), C.c_uint32(ignore_index or 0),
                                                 C.c_int64(chunk[0]), C.c_int64(chunk[1]), _p(loss), _p(gx), _p(gw)))
        return loss, gx, gw

    def cross_entropy_mean_forward(self, logits, targets, ignore_index=None):
        loss = self.empty((1,), DType.F32)
        _check(lib.ojc_cross_entropy_mean_forward(self._handle, _p(logits), _p(targets), C.c_int32(ignore_index is not None), C.c_uint32(ignore_index or 0), _p(loss)))
        return loss

    def cross_entropy_mean_backward(self, logits, targets, ignore_index=None):
        g = self.empty(logits.shape, logits.dtype)
        _check(lib.ojc_cross_entropy_mean_backward(self._handle, _p(logits), _p(targets), C.c_int32(ignore_index is not None), C.c_uint32(ignore_index or 0), _p(g)))
        return g

    def argmax_rows(self, x):
        out = self.empty((x.shape[0],), DType.U32)
        _check(lib.ojc_argmax_rows(self._handle, _p(x), _p(out)))
        return out

    # ---- decode / eval ops
    def topk_rows(self, x, k: int):
        """(values F32 [rows, k], ids U32 [rows, k]) ranked as rank_logits ranks (value descending, then column ascending)."""
        values, ids = self.empty((x.shape[0], k), DType.F32), self.empty((x.shape[0], k), DType.U32)
        _check(lib.ojc_topk_rows(self._handle, _p(x), C.c_int64(k), _p(values), _p(ids)))
        return values, ids

    def kv_cache_write(self, cache: Tensor, src: Tensor, at: int):
        _check(lib.ojc_kv_cache_write(self._handle, _p(cache), _p(src), C.c_uint64(at)))

    def cached_attention_forward(self, q, k_cache, v_cache, kv_len: int, window: int | None = None):
        out = self.empty(q.shape, DType.F32)
        _check(lib.ojc_cached_attention_forward(self._handle, _p(q), _p(k_cache), _p(v_cache), C.c_uint64(kv_len), C.c_int64(-1 if window is None else window), _p(out)))
        return out

    # ---- in-place gradient plumbing and optimizers
    def accumulate_grad(self, acc: Tensor, grad: Tensor):
        _check(lib.ojc_accumulate_grad(self._handle, _p(acc), _p(grad)))

    def scale_grad(self, grad: Tensor, scale: float):
        _check(lib.ojc_scale_grad(self._handle, _p(grad), C.c_float(scale)))

    def clip_grad_norm(self, grads, max_norm: float) -> float:
        cts = [g.c() for g in grads]
        arr = (C.POINTER(CTensor) * len(cts))(*[C.pointer(c) for c in cts])
        norm = C.c_float()
        _check(lib.ojc_clip_grad_norm(self._handle, arr, C.c_int64(len(cts)), C.c_float(max_norm), C.byref(norm)))
        return norm.value

    def adamw_step(self, param, grad, m, v, step: int, config: AdamWConfig, bf16_mirror=None):
        cfg = config.c()
        _check(lib.ojc_adamw_step(self._handle, _p(param), _p(grad), _p(m), _p(v), C.c_uint64(step), C.byref(cfg), _p(bf16_mirror)))

    def muon_ns5_step(self, param, grad, momentum, config: MuonNs5Config, bf16_mirror=None):
        cfg = config.c()
        _check(lib.ojc_muon_ns5_step(self._handle, _p(param), _p(grad), _p(momentum), C.byref(cfg), _p(bf16_mirror)))

    def optimizer_scratch_bytes(self, kind: str, rows: int, cols: int) -> int:
        out = C.c_uint64()
        _check(lib.ojc_optimizer_scratch_bytes(self._handle, C.c_int32(0 if kind == "adamw" else 1), C.c_int64(rows), C.c_int64(cols), C.byref(out)))
        return out.value


@dataclass
class ModelSpec:
    """ojas-model/src/spec.rs:45. nanolab_124m is spec.rs:76-91."""
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

    @staticmethod
    def nanolab_124m(hidden: int = 2048) -> "ModelSpec":
        return ModelSpec(vocab=50304, n_embd=768, n_layer=12, n_head=12, n_kv_head=12, head_dim=64, hidden=hidden, max_seq=1024)

    def c(self):
        return _lib.ModelSpec(self.vocab, self.n_embd, self.n_layer, self.n_head, self.n_kv_head, self.head_dim, self.hidden, self.max_seq,
                              -1 if self.window is None else self.window, self.rope_base, self.rms_eps)

    def matmul_params(self) -> int:
        """N_mm = L (d q + 2 d kv + q d + H d + 3 F d) + V d."""
        d, q, kv = self.n_embd, self.n_head * self.head_dim, self.n_kv_head * self.head_dim
        return self.n_layer * (d * q + 2 * d * kv + q * d + self.n_head * d + 3 * self.hidden * d) + self.vocab * d

    def flops_per_token(self, seq: int) -> float:
        """6 N_mm + 6 L T q (causal-halved attention; recompute is not counted)."""
        return 6.0 * self.matmul_params() + 6.0 * self.n_layer * seq * self.n_head * self.head_dim


@dataclass
class TrainConfig:
    """TrainConfig (ojas-model/src/trainer.rs:100-172). optimizer 'adamw' steps every tensor with AdamW;
    'muon' is the Trainer's own grouping (Muon NS5 on rank-2 hidden weights, AdamW without decay elsewhere)."""
    autocast_bf16: bool = False
    optimizer: str = "muon"
    adam_lr: float = 6e-4
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    adam_weight_decay: float = 0.0
    matrix_lr: float = 0.025
    muon_momentum: float = 0.99
    muon_weight_decay: float = 0.1
    ns5_bf16: bool = False
    grad_clip: float = 1.0
    ignore_index: int | None = None
    ce_chunk_rows: int = 0
    loss_seed: float = 1.0
    checkpoint_blocks: bool = False      # ActivationCheckpoint::Blocks: recompute each block in backward from its saved input
    schedule: str = "none"               # LrSchedule (ojas-cpu/src/schedule.rs:205-226): "none" (multiplier 1), "cosine" or "wsd"
    warmup_steps: int = 0
    total_steps: int = 0
    decay_frac: float = 0.2              # WSD_DECAY_FRAC
    on_nonfinite: str = "abort"          # NonFinitePolicy (trainer.rs:85-91): "abort" or "skip_batch"

    def c(self):
        return _lib.TrainConfig(int(self.autocast_bf16), 0 if self.optimizer == "adamw" else 1, self.adam_lr, self.adam_beta1, self.adam_beta2, self.adam_eps,
                                self.adam_weight_decay, self.matrix_lr, self.muon_momentum, self.muon_weight_decay, int(self.ns5_bf16), self.grad_clip,
                                int(self.ignore_index is not None), self.ignore_index or 0, self.ce_chunk_rows, self.loss_seed, int(self.checkpoint_blocks),
                                {"none": 0, "cosine": 1, "wsd": 2}[self.schedule], self.warmup_steps, self.total_steps, self.decay_frac,
                                {"abort": 0, "skip_batch": 1}[self.on_nonfinite])

    def lr_multiplier(self, step: int) -> float:
        """LrSchedule::multiplier at a 0-based step, computed by the library (f64, nanolab's order of operations)."""
        out, cc = C.c_double(), self.c()
        _check(lib.ojc_lr_multiplier(C.byref(cc), C.c_uint64(step), C.byref(out)))
        return out.value


@dataclass
class ParamInfo:
    name: str
    shape: tuple
    group: str
    trains: bool


@dataclass
class StepReport:
    loss: float
    grad_norm: float
    step: int
    tokens: int
    lr_multiplier: float = 1.0


class Trainer:
    """One optimizer step per call, the sequence of ojas-model's Trainer::step (trainer.rs:672-1046) run by the C++ driver."""

    def __init__(self, backend: CudaBackend, spec: ModelSpec, config: TrainConfig, batch: int, seq: int):
        self.backend, self.spec, self.config, self.batch, self.seq = backend, spec, config, batch, seq
        self._h = None
        h = C.c_void_p()
        cs, cc = spec.c(), config.c()
        _check(lib.ojc_trainer_open(backend._handle, C.byref(cs), C.byref(cc), C.c_int64(batch), C.c_int64(seq), C.byref(h)))
        self._h = h
        self.params: list[ParamInfo] = []
        for i in range(lib.ojc_trainer_param_count(h)):
            name = C.create_string_buffer(128)
            rank, shape, group, trains = C.c_int32(), (C.c_int64 * 2)(), C.c_int32(), C.c_int32()
            _check(lib.ojc_trainer_param_info(h, C.c_int64(i), name, C.c_int64(128), C.byref(rank), shape, C.byref(group), C.byref(trains)))
            self.params.append(ParamInfo(name.value.decode(), tuple(shape[: rank.value]), "muon" if group.value else "adamw", bool(trains.value)))

    def close(self):
        if self._h:
            if self.backend._handle:  # a closed backend already released everything the trainer owned
                lib.ojc_trainer_close(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def set_param(self, index: int, values: np.ndarray):
        v = np.ascontiguousarray(values, np.float32)
        _check(lib.ojc_trainer_set_param(self._h, C.c_int64(index), C.c_void_p(v.ctypes.data), C.c_uint64(v.size)))

    def set_params(self, values):
        for i, v in enumerate(values):
            self.set_param(i, v)

    def get_param(self, index: int) -> np.ndarray:
        out = np.empty(self.params[index].shape, np.float32)
        _check(lib.ojc_trainer_get_param(self._h, C.c_int64(index), C.c_void_p(out.ctypes.data), C.c_uint64(out.size)))
        return out

    def get_grad(self, index: int) -> np.ndarray:
        out = np.empty(self.params[index].shape, np.float32)
        _check(lib.ojc_trainer_get_grad(self._h, C.c_int64(index), C.c_void_p(out.ctypes.data), C.c_uint64(out.size)))
        return out

    def get_moment(self, index: int, slot: int) -> np.ndarray:
        """Optimizer state of one parameter: slot 0 is the Muon momentum or the AdamW first moment, slot 1 the AdamW second."""
        out = np.empty(self.params[index].shape, np.float32)
        _check(lib.ojc_trainer_get_moment(self._h, C.c_int64(index), C.c_int32(slot), C.c_void_p(out.ctypes.data), C.c_uint64(out.size)))
        return out

    def set_moment(self, index: int, slot: int, values: np.ndarray):
        v = np.ascontiguousarray(values, np.float32)
        _check(lib.ojc_trainer_set_moment(self._h, C.c_int64(index), C.c_int32(slot), C.c_void_p(v.ctypes.data), C.c_uint64(v.size)))

    @property
    def steps_done(self) -> int:
        return int(lib.ojc_trainer_steps_done(self._h))

    @steps_done.setter
    def steps_done(self, step: int):
        _check(lib.ojc_trainer_set_steps_done(self._h, C.c_uint64(step)))

    @staticmethod
    def _ids(a) -> np.ndarray:
        return np.ascontiguousarray(a, np.uint32)

    def gradients(self, ids, targets) -> float:
        ids, targets = self._ids(ids), self._ids(targets)
        assert ids.size == self.batch * self.seq == targets.size
        loss = C.c_float()
        _check(lib.ojc_trainer_gradients(self._h, C.c_void_p(ids.ctypes.data), C.c_void_p(targets.ctypes.data), C.byref(loss)))
        return loss.value

    def apply(self, read_norm: bool = True):
        """Clip + optimizer. With read_norm the gradient norm is read back (a sync); without, nothing is."""
        norm = C.c_float()
        _check(lib.ojc_trainer_apply(self._h, C.byref(norm) if read_norm else None))
        return norm.value if read_norm else None

    def overlap_weight_grads(self, enable: bool) -> None:
        """Run (default) or do not run the weight-gradient GEMMs on the second stream; results are the same bits either way."""
        _check(lib.ojc_trainer_overlap_weight_grads(self._h, C.c_int32(int(enable))))

    def finish(self) -> StepReport:
        rep = _lib.StepReport()
        _check(lib.ojc_trainer_finish(self._h, C.byref(rep)))
        return StepReport(rep.loss, rep.grad_norm, rep.step, rep.tokens, rep.lr_multiplier)

    def step(self, ids, targets) -> StepReport:
        ids, targets = self._ids(ids), self._ids(targets)
        assert ids.size == self.batch * self.seq == targets.size
        rep = _lib.StepReport()
        _check(lib.ojc_trainer_step(self._h, C.c_void_p(ids.ctypes.data), C.c_void_p(targets.ctypes.data), C.byref(rep)))
        return StepReport(rep.loss, rep.grad_norm, rep.step, rep.tokens, rep.lr_multiplier)

    def _batch_ptrs(self, batches):
        xs = [self._ids(x) for x, _ in batches]
        ys = [self._ids(y) for _, y in batches]
        for a in xs + ys:
            assert a.size == self.batch * self.seq
        px = (C.c_void_p * len(xs))(*[a.ctypes.data for a in xs])
        py = (C.c_void_p * len(ys))(*[a.ctypes.data for a in ys])
        return xs, ys, px, py

    def run(self, batches) -> StepReport:
        """Trainer::step_tokens (trainer.rs:713-720): one optimizer step over K micro-batches [(ids, targets)], each [batch, seq]."""
        keep = self._batch_ptrs(batches)
        rep = _lib.StepReport()
        _check(lib.ojc_trainer_run(self._h, keep[2], keep[3], C.c_int64(len(batches)), C.byref(rep)))
        return StepReport(rep.loss, rep.grad_norm, rep.step, rep.tokens, rep.lr_multiplier)

    def run_gradients(self, batches) -> None:
        """The gradient half of run(): K forward/backward passes summed into the gradient buckets; apply() and finish() complete the step."""
        keep = self._batch_ptrs(batches)
        _check(lib.ojc_trainer_run_gradients(self._h, keep[2], keep[3], C.c_int64(len(batches))))

    def step_sampled(self, sampler, bin_, accum: int = 1) -> StepReport:
        """Trainer::step (trainer.rs:672-711): draw `accum` micro-batches from the sampler, run them, and move the sampler's cursor
        past them on success, or on a NonFinite step under NonFinitePolicy::SkipBatch (at most 8 in a row); any other failure
        leaves the cursor where it was."""
        saved = (sampler.epoch, sampler.ordinal)
        batches = [sampler.next_batch(bin_) for _ in range(accum)]
        try:
            return self.run(batches)
        except OjasError as err:
            advance = C.c_int32(0)
            final = lib.ojc_trainer_resolve_failure(self._h, C.c_int32(err.status), C.byref(advance))
            if not advance.value:
                sampler.epoch, sampler.ordinal = saved
            if final != err.status:
                _check(final)
            raise

    @property
    def state(self) -> str:
        """TrainState (trainer.rs:93-98)."""
        return "Poisoned" if lib.ojc_trainer_state(self._h) else "Ready"

    def inject_failure(self, where: str) -> None:
        """Host-made failure for tests: 'gradients' fails the next gradient pass after its forward, 'optimizer' the next optimizer phase
        after its first update kernel."""
        _check(lib.ojc_trainer_inject_failure(self._h, C.c_int32({"none": 0, "gradients": 1, "optimizer": 2}[where])))

    def set_comm(self, comm, shard_muon: bool = False) -> None:
        """Attach a dp.Communicator (or None): step / step_device / run then sum the gradient buckets across ranks between backward and
        the optimizer. shard_muon splits the Muon phase: each rank orthogonalises every world-th matrix of a shape group and the new
        parameters are broadcast from their owners."""
        _check(lib.ojc_trainer_set_comm(self._h, comm._h if comm is not None else None, C.c_int32(int(shard_muon))))
        self._comm = comm          # keeps the communicator alive as long as the trainer uses it

    def sync_moments(self) -> None:
        """Under shard_muon a matrix's momentum lives on its owner rank: broadcast every momentum from its owner (before a checkpoint)."""
        _check(lib.ojc_trainer_sync_moments(self._h))

    def exposed_exchange_ms(self) -> float:
        """Device time the library's stream waited for the gradient exchange in the last finished step."""
        out = C.c_float()
        _check(lib.ojc_trainer_exposed_exchange_ms(self._h, C.byref(out)))
        return out.value

    def param_checksum(self) -> int:
        """FNV-1a over every parameter's f32 bytes in table order: equal on every rank of a healthy data-parallel job."""
        out = C.c_uint64()
        _check(lib.ojc_trainer_param_checksum(self._h, C.byref(out)))
        return out.value

    def step_host_ptrs(self, ids_ptr: int, targets_ptr: int) -> StepReport:
        """Same as step() for caller-owned (for example pinned) host buffers given by address."""
        rep = _lib.StepReport()
        _check(lib.ojc_trainer_step(self._h, C.c_void_p(ids_ptr), C.c_void_p(targets_ptr), C.byref(rep)))
        return StepReport(rep.loss, rep.grad_norm, rep.step, rep.tokens, rep.lr_multiplier)

    def step_device(self, ids: Tensor, targets: Tensor) -> StepReport:
        rep = _lib.StepReport()
        _check(lib.ojc_trainer_step_device(self._h, C.c_void_p(ids.ptr), C.c_void_p(targets.ptr), C.byref(rep)))
        return StepReport(rep.loss, rep.grad_norm, rep.step, rep.tokens, rep.lr_multiplier)

    def gradients_device(self, ids: Tensor, targets: Tensor):
        _check(lib.ojc_trainer_gradients_device(self._h, C.c_void_p(ids.ptr), C.c_void_p(targets.ptr)))

    def logits(self, ids) -> np.ndarray:
        ids = self._ids(ids)
        out = np.empty((self.batch * self.seq, self.spec.vocab), np.float32)
        _check(lib.ojc_trainer_logits(self._h, C.c_void_p(ids.ctypes.data), C.c_void_p(out.ctypes.data)))
        return out

    def buckets(self):
        out = []
        for i in range(lib.ojc_trainer_bucket_count(self._h)):
            ptr, n, ev = C.c_void_p(), C.c_uint64(), C.c_void_p()
            _check(lib.ojc_trainer_bucket(self._h, C.c_int64(i), C.byref(ptr), C.byref(n)))
            _check(lib.ojc_trainer_bucket_ready_event(self._h, C.c_int64(i), C.byref(ev)))
            out.append((ptr.value, n.value, ev.value))
        return out


_SESSION_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_void_p)


class Session:
    """An owner-thread session (ojc_session_*): the library starts a thread that opens the backend and is the only one ever to touch
    it, which is how ojas-capi holds a backend whose handle is single-owner-thread (ojas-capi/src/owner.rs). `run(fn)` executes
    `fn(backend)` on that thread and returns its value, from whichever thread calls it; calls from several threads queue up."""

    def __init__(self, device: int = 0, budget_bytes: int = 160 << 30, open_timeout_ms: int = 120_000):
        self._h = None
        h = C.c_void_p()
        _check(lib.ojc_session_open(C.c_int32(device), C.c_uint64(budget_bytes), C.c_uint64(open_timeout_ms), C.byref(h)))
        self._h = h

    def run(self, fn):
        box = {}

        def thunk(be_ptr, _arg):
            try:
                box["value"] = fn(CudaBackend._adopt(be_ptr))
                return 0
            except OjasError as e:
                box["error"] = e
                return e.status
            except BaseException as e:      # a Python error on the owner thread is re-raised on the caller's
                box["error"] = e
                return 10
        st = lib.ojc_session_call(self._h, _SESSION_FN(thunk), None)
        if "error" in box:
            raise box["error"]
        _check(st)
        return box.get("value")

    def close(self):
        if self._h:
            lib.ojc_session_close(self._h)
            self._h = None

    def __del__(self):
        self.close()
