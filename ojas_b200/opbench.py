"""Single-op timing through the C ABI, for profiling one kernel at a time.

    python -m ojas_b200.opbench gemm ROWS IN OUT [bf16|f32] [--reps N]     y = x W^T on BF16 operands (tcgen05 kernels)
    python -m ojas_b200.opbench sdpa BATCH HEADS TIME HEAD_DIM [--reps N] [--one-tile]  causal attention forward and backward (BF16)

Prints microseconds per call (CUDA events on the library's stream) and TFLOP/s. The operands are uninitialised device
memory for gemm (timing does not depend on values) and seeded normal draws for sdpa (the softmax needs finite rows).
"""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np


def _timed(be, fn, reps: int) -> float:
    import torch
    stream = torch.cuda.ExternalStream(be.stream())
    for _ in range(3):
        fn()
    be.sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(reps):
        fn()
    b.record(stream)
    be.sync()
    return a.elapsed_time(b) / reps * 1000.0


def gemm(args) -> None:
    from . import CudaBackend, DType
    be = CudaBackend(0, 16 << 30)
    x, w = be.empty((args.rows, args.kin), DType.BF16), be.empty((args.nout, args.kin), DType.BF16)
    out_dt = DType.F32 if args.out == "f32" else DType.BF16
    us = _timed(be, lambda: be.linear_forward(x, w, out_dtype=out_dt), args.reps)
    flops = 2.0 * args.rows * args.kin * args.nout
    print(f"linear_forward {args.rows}x{args.kin}->{args.nout} {args.out}: {us:.1f} us  {flops / us / 1e6:.1f} TFLOP/s")
    be.close()


def sdpa(args) -> None:
    from . import CudaBackend, DType
    from ._lib import lib
    from .backend import _check, _p
    B, H, T, D = args.batch, args.heads, args.time, args.dim
    be = CudaBackend(0, 16 << 30)
    _check(lib.ojc_sdpa_forward_variant(C.c_int32(args.variant if args.variant else int(args.one_tile))))   # 1: one CTA per tile, forward and backward

    def draw(seed):  # [B,T,H,D] storage viewed as [B,H,T,D], the layout the step driver uses
        return be.upload(np.random.default_rng(seed).standard_normal((B, T, H, D), dtype=np.float32), DType.BF16).permuted((0, 2, 1, 3))

    q, k, v, g = draw(0), draw(1), draw(2), draw(3)
    out = be.empty((B, T, H, D), DType.BF16).permuted((0, 2, 1, 3))
    lse = be.empty((B, H, T))
    gq, gk, gv = (be.empty((B, T, H, D), DType.BF16).permuted((0, 2, 1, 3)) for _ in range(3))
    fwd = lambda: _check(lib.ojc_causal_sdpa_forward(be._handle, _p(q), _p(k), _p(v), C.c_int64(-1), _p(out), _p(lse)))
    bwd = lambda: _check(lib.ojc_causal_sdpa_backward(be._handle, _p(q), _p(k), _p(v), _p(out), _p(lse), _p(g), C.c_int64(-1), _p(gq), _p(gk), _p(gv)))
    flops = 4.0 * B * H * T * T * D / 2
    for name, fn, mult in (("causal_sdpa_forward", fwd, 1.0), ("causal_sdpa_backward", bwd, 2.5)):
        us = _timed(be, fn, args.reps)
        print(f"{name} B{B} H{H} T{T} D{D}: {us:.1f} us  {flops * mult / us / 1e6:.1f} TFLOP/s")
    be.close()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("rows", type=int); g.add_argument("kin", type=int); g.add_argument("nout", type=int)
    g.add_argument("out", nargs="?", default="bf16", choices=["bf16", "f32"])
    g.add_argument("--reps", type=int, default=10)
    g.set_defaults(fn=gemm)
    s = sub.add_parser("sdpa")
    s.add_argument("batch", type=int); s.add_argument("heads", type=int); s.add_argument("time", type=int); s.add_argument("dim", type=int)
    s.add_argument("--reps", type=int, default=10)
    s.add_argument("--one-tile", action="store_true", help="time the one-CTA-per-tile kernels (forward and backward) instead of the library's choice")
    s.add_argument("--variant", type=int, default=0, help="kernel selection as ojc_sdpa_forward_variant takes it (4: the 64-wide backward kernels by their own rule, 5: the 128-wide ones always)")
    s.set_defaults(fn=sdpa)
    args = ap.parse_args()
    args.fn(args)


if __name__ == "__main__":
    main()
