#!/usr/bin/env python
"""Benchmark of the one hot path: the nanolab GPT-124M bf16 training step on B200.

    python bench.py --gpus N --steps K --warmup W            this library (one process per GPU; torchrun for N > 1)
    python bench.py --impl reference --gpus N --steps K ...  the CPU restatement of the reference's path on the host cores

A step is one optimizer step (forward, fused tied-head cross-entropy, backward, AdamW on every tensor) over one batch
of synthetic token ids: ModelSpec::nanolab_124m (hidden 2048), B 32 x T 1024 per GPU, bf16 autocast. Rank 0 prints one
JSON line. `value` is tokens/s with the batch already in HBM; `e2e` is the same step through Trainer.step with pinned
host ids/targets copied in and the loss read back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BATCH, SEQ = 32, 1024
# The workloads BASELINE.json names: "124m" is the headline (configs 2 and 3: ModelSpec::nanolab_124m, hidden 2048, B 32 x T 1024 per GPU);
# "1p7b" is its 1.3B-class data-parallel case (config 5: 24 layers, d 2048, 16 x 128 heads, hidden 8192, B 8 x T 2048 per GPU; 1,714,528,664
# parameters with this model's three-matrix SwiGLU and gate).
CONFIGS = {
    "124m": dict(spec=dict(vocab=50304, n_embd=768, n_layer=12, n_head=12, n_kv_head=12, head_dim=64, hidden=2048, max_seq=1024), batch=32, seq=1024,
                 name="nanolab GPT-124M train step (ModelSpec::nanolab_124m, hidden 2048): 12 layers, d 768, 12x64 heads, vocab 50304, seq 1024, micro-batch 32 per GPU"),
    "1p7b": dict(spec=dict(vocab=50304, n_embd=2048, n_layer=24, n_head=16, n_kv_head=16, head_dim=128, hidden=8192, max_seq=2048), batch=8, seq=2048,
                 name="nanolab GPT 1.3B-class train step (1,714,528,664 parameters): 24 layers, d 2048, 16x128 heads, hidden 8192, vocab 50304, seq 2048, micro-batch 8 per GPU"),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one full-size GEMM launch of the step, the q/k/v projection
# [32768 x 768] x [768 x 2304] -> bf16, from one ncu capture of `python -m ojas_b200.opbench gemm 32768 768 2304`:
# 53.9 MB read + 96.7 MB written against 205.0 MB of algorithmic bytes (the tail of the output is still in L2 when the kernel ends).
GEMM_TRAFFIC_BYTES_PER_LAUNCH = 150_663_424
GEMM_TRAFFIC_LAUNCH = "q/k/v projection 32768x768x2304 bf16: algorithmic 205.0 MB per launch"


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def spec_kwargs(config: str = "124m") -> dict:
    return dict(CONFIGS[config]["spec"])


def init_weights(param_infos, seed: int):
    """Random-init weights of the architecture: N(0, 0.02) on every matrix, ones on norm weights, zeros on bias / lambda."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = []
    for p in param_infos:
        if len(p.shape) == 2:
            out.append((rng.standard_normal(p.shape, dtype=np.float32) * np.float32(0.02)).astype(np.float32))
        elif p.name.endswith("norm.weight") or ".norm1." in p.name or ".norm2." in p.name or p.name == "norm_f.weight":
            out.append(np.ones(p.shape, np.float32))
        else:
            out.append(np.zeros(p.shape, np.float32))
    return out


def token_batches(count: int, batch: int, seq: int, vocab: int, seed: int):
    rng = np.random.Generator(np.random.PCG64(seed))
    out = []
    for _ in range(count):
        draws = rng.integers(0, vocab, size=(batch, seq + 1), dtype=np.uint32)
        out.append((np.ascontiguousarray(draws[:, :-1]), np.ascontiguousarray(draws[:, 1:])))
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 100 ms; the lines that arrive while the timed region runs are the ones reported."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.lines, self.proc = device, [], None
        self.t0 = self.t1 = None

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.device)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()  # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        # The sampler is started before the warm-up steps (nvidia-smi takes longer to produce its first line than a short timed region
        # lasts); only lines that arrived between mark_start and mark_end count.
        inside = [line for ts, line in self.lines if self.t0 is None or (self.t0 <= ts <= (self.t1 if self.t1 is not None else ts))]
        for line in inside:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU arm
def host_threads() -> int:
    """The host threads this process may use (its affinity mask, not the machine's core count)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_step_rate(budget_s: float, steps: int, warmup: int, fast: bool):
    """Times the CPU restatement of the reference's step (oracle/) on a bounded sample of the workload: the 124M model, B = 1,
    T chosen so (steps + warmup) steps fit the budget. fast selects Numerics::Fast (the reference's default tier: fused
    multiply-add products, f32 AdamW) instead of the strict-order Exact tier. The thread count is set explicitly (a launcher
    may have exported OMP_NUM_THREADS=1) and the count actually in force is what is reported.
    Returns (tokens/s, threads, sample text, ms/step, seq)."""
    from oracle import oracle as orc
    threads = orc.set_threads(host_threads())
    orc.set_fast(fast)
    try:
        spec = orc.Spec(**spec_kwargs())
        table = orc.param_table(spec)
        params = init_weights(table, 0)
        m1 = [np.zeros(p.size, np.float32) for p in params]
        m2 = [np.zeros(p.size, np.float32) for p in params]

        def one_step(ids, targets, step_before):
            loss, grads, _ = orc.forward_loss(spec, params, ids, targets)
            for info, p, g, a, b in zip(table, params, grads, m1, m2):
                if info.trains:
                    orc.adamw_step(p.reshape(-1), g.reshape(-1), a, b, step_before, 3e-4, weight_decay=0.1)
            return float(loss)

        probe_t = 64
        (px, py), = token_batches(1, 1, probe_t, spec.vocab, 7)
        one_step(px, py, 0)
        t1 = time.perf_counter()
        one_step(px, py, 1)
        probe = time.perf_counter() - t1
        seq = 64
        for cand in (1024, 512, 256, 128):
            if probe * (cand / probe_t) * (steps + warmup) <= budget_s:
                seq = cand
                break
        batches = token_batches(steps + warmup, 1, seq, spec.vocab, 11)
        for i in range(warmup):
            one_step(*batches[i], 2 + i)
        t0 = time.perf_counter()
        for i in range(steps):
            one_step(*batches[warmup + i], 2 + warmup + i)
        elapsed = time.perf_counter() - t0
    finally:
        orc.set_fast(False)
    tier = "Numerics::Fast (fused multiply-add products, f32 AdamW)" if fast else "Numerics::Exact (strict-order f32, f64 AdamW)"
    sample = f"nanolab-124M step (fwd + fused CE + bwd + AdamW) in {tier}, B=1 T={seq}, {steps} steps after {warmup} warm-up, {threads} OpenMP threads"
    return steps * seq / elapsed, threads, sample, 1000.0 * elapsed / steps, seq


def cpu_baseline_object(budget_s: float, steps: int, warmup: int) -> tuple[dict, float, int]:
    """The reported CPU baseline: the reference's default tier (Fast) as `value`, the strict-order Exact tier beside it."""
    rate, threads, sample, ms, seq = cpu_step_rate(budget_s * 0.7, steps, warmup, fast=True)
    erate, _, esample, _, _ = cpu_step_rate(budget_s * 0.3, 1, 0, fast=False)
    return ({"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "tier": "fast", "sample": sample,
             "exact_tier": {"value": erate, "unit": "tokens/s", "sample": esample}}, ms, seq)


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    base, ms, seq = cpu_baseline_object(200.0, args.steps, args.warmup)
    config = workload_config(args.gpus)
    config["cpu_sample"] = f"timed on B=1 T={seq} of the workload above, f32 on the host cores (no GPU); tokens/s = sampled tokens / elapsed"
    line = {
        "impl": "reference", "metric": "nanolab_gpt_124m_train_tokens_per_s", "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


MUON_RECIPE = "Muon NS5 bf16 (lr 0.025, momentum 0.95, wd 0.1, Nesterov) on 2-D hidden weights + AdamW(lr 6e-4, wd 0) on embedding and vectors, clip 1.0"


def workload_config(n_gpus: int, optimizer: str = "adamw", config: str = "124m") -> dict:
    opt = "AdamW(lr 3e-4, betas 0.9/0.95, eps 1e-8, wd 0.1) on every tensor" if optimizer == "adamw" else MUON_RECIPE
    c = CONFIGS[config]
    return {"workload": c["name"] + ", bf16 autocast, " + opt,
            "global_batch": c["batch"] * n_gpus, "seq_len": c["seq"], "parallelism": f"dp{n_gpus}",
            "l2": "inputs larger than L2: one step streams many GB of activations, weights and optimizer state"}


# ------------------------------------------------------------------------------------------------ GPU arm
def train_config(optimizer: str, world: int):
    from ojas_b200 import TrainConfig
    if optimizer == "muon":   # BASELINE's data-parallel recipe
        return TrainConfig(autocast_bf16=True, optimizer="muon", adam_lr=6e-4, adam_weight_decay=0.0, matrix_lr=0.025, muon_momentum=0.95, muon_weight_decay=0.1,
                           ns5_bf16=True, grad_clip=1.0, loss_seed=1.0 / world)
    return TrainConfig(autocast_bf16=True, optimizer="adamw", adam_lr=3e-4, adam_weight_decay=0.1, grad_clip=0.0, loss_seed=1.0 / world)


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch
    from ojas_b200 import CudaBackend, ModelSpec, Trainer
    from ojas_b200.dp import Communicator

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))   # barriers and the max over ranks; the step's exchange is the library's own
    be = CudaBackend(local_rank, 170 << 30)
    if args.kernel_variants:
        import ctypes
        from ojas_b200._lib import lib
        switches = {"ce_rows": lib.ojc_ce_rows_variant, "mlp_epilogue": lib.ojc_mlp_epilogue_variant, "sdpa": lib.ojc_sdpa_forward_variant}
        for item in args.kernel_variants.split(","):
            name, _, value = item.partition("=")
            switches[name.strip()](ctypes.c_int32(int(value)))
    conf = CONFIGS[args.config]
    spec = ModelSpec(**conf["spec"])
    seq = conf["seq"]
    batch = args.batch if args.batch else conf["batch"]   # the workload's; smaller only for profiler captures, and the line then says so
    comm = Communicator.over_torch_distributed(be) if world > 1 else None
    main = torch.cuda.ExternalStream(be.stream(), device=torch.device("cuda", local_rank))
    n_batches = 4
    batches = token_batches(n_batches, batch, seq, spec.vocab, 1 + rank)  # a distinct id stream per rank
    dev = [(be.upload(x), be.upload(y)) for x, y in batches]
    pinned = []
    for x, y in batches:
        px, py = torch.empty(x.size, dtype=torch.int32).pin_memory(), torch.empty(y.size, dtype=torch.int32).pin_memory()
        px.numpy().view(np.uint32)[:] = x.ravel(); py.numpy().view(np.uint32)[:] = y.ravel()
        pinned.append((px, py))

    def timed(step_fn, steps):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(main)
        rep = None
        for i in range(steps):
            rep = step_fn(i)
        stop.record(main)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=f"cuda:{local_rank}")
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), rep

    def open_trainer(optimizer):
        tr = Trainer(be, spec, train_config(optimizer, world), batch, seq)
        tr.set_params(init_weights(tr.params, 0))  # identical weights on every rank
        if comm is not None:
            tr.set_comm(comm, shard_muon=optimizer == "muon")   # the Muon phase is split across the ranks
        return tr

    def ranks_identical(tr):
        if dist is None:
            return None
        mine = torch.tensor([tr.param_checksum() & 0x7FFFFFFFFFFFFFFF], dtype=torch.int64, device=f"cuda:{local_rank}")
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool(lo.item() == hi.item())

    warm = max(args.warmup, 3)
    tokens = batch * seq * world
    pk, pk_kind = peaks()
    fpt = spec.flops_per_token(seq)

    # ---- the other optimizer recipe first (its trainer is closed before the headline's opens): a short measurement of its own
    other = "muon" if args.optimizer == "adamw" else "adamw"
    other_obj = None
    if not args.no_second_recipe:
        tr = open_trainer(other)
        step = lambda i: tr.step_device(*dev[i % n_batches])
        for i in range(warm):
            step(i)
        oms, orep = timed(step, args.steps)
        exposed = [tr.exposed_exchange_ms()] if comm is not None else None
        other_obj = {"optimizer": MUON_RECIPE if other == "muon" else "AdamW on every tensor, no clipping", "value": tokens * args.steps / (oms / 1000.0), "unit": "tokens/s",
                     "ms_per_step": oms / args.steps, "mfu": tokens * args.steps / (oms / 1000.0) * fpt / (world * pk["bf16_tflops"] * 1e12),
                     "final_loss": orep.loss if orep else None, "muon_split_across_ranks": bool(comm is not None and other == "muon"),
                     "exposed_allreduce_ms": exposed[0] if exposed else None, "ranks_bit_identical": ranks_identical(tr)}
        tr.set_comm(None) if comm is not None else None
        tr.close()

    tr = open_trainer(args.optimizer)

    def step_resident(i):
        return tr.step_device(*dev[i % n_batches])

    def step_e2e(i):
        px, py = pinned[i % n_batches]
        return tr.step_host_ptrs(px.data_ptr(), py.data_ptr())

    with ClockSampler(local_rank) as clocks:
        for i in range(warm):
            step_resident(i)
        launches0 = be.kernel_launches()
        clocks.mark_start()
        ms, rep = timed(step_resident, args.steps)
        clocks.mark_end()
    launches = be.kernel_launches() - launches0
    exposed_ms = tr.exposed_exchange_ms() if comm is not None else None
    # Roofline pass: the same K steps again with the weight-gradient GEMMs folded back into the one stream, so every GEMM launch
    # is bracketed by CUDA events with the GPU to itself (in the timed region above they share the SMs with the dX chain).
    tr.overlap_weight_grads(False)
    be.profile_gemm(True)
    roof_ms, _ = timed(step_resident, args.steps)
    (gemm_ms, gemm_flops, gemm_launches), (epi_ms, epi_flops, epi_launches) = be.profile_gemm_read_split()
    be.profile_gemm(False)
    tr.overlap_weight_grads(True)
    e2e_ms = None
    if not args.no_e2e:
        step_e2e(0)
        e2e_ms, _ = timed(step_e2e, args.steps)

    value = tokens * args.steps / (ms / 1000.0)
    line = {
        "metric": "nanolab_gpt_124m_train_tokens_per_s" if args.config == "124m" else "nanolab_gpt_1p7b_train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(world, args.optimizer, args.config) if batch == conf["batch"] and not args.kernel_variants else
                  {"workload": f"PROFILER CASE, not the benchmark workload: micro-batch {batch}, kernel variants '{args.kernel_variants}'"},
        "mfu": value * fpt / (world * pk["bf16_tflops"] * 1e12), "mfu_vs_sustained": value * fpt / (world * pk["bf16_tflops_sustained"] * 1e12),
        "flops_per_token": fpt, "final_loss": rep.loss if rep else None,
        "e2e": {"value": tokens * args.steps / (e2e_ms / 1000.0) if e2e_ms else None, "unit": "tokens/s", "h2d_bytes_per_step": 2 * batch * seq * 4,
                "d2h_bytes_per_step": 20 + 8},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
    }
    if comm is not None:
        line["exchange"] = {"how": "ojc_allreduce_start / _wait: one NCCL all-reduce per ~25 MB gradient bucket on the communicator's stream, behind the bucket's ready event",
                            "exposed_allreduce_ms": exposed_ms, "ranks_bit_identical": ranks_identical(tr)}
    if other_obj is not None:
        line["muon_hybrid" if other == "muon" else "adamw_only"] = other_obj
    if gemm_ms > 0:
        achieved = gemm_flops / (gemm_ms / 1000.0) / 1e12
        line["roofline"] = {"kernel": "gemm_tc2_kernel / gemm_tc_kernel (tcgen05 bf16 GEMM, two-SM and one-SM tiles; every plain launch of the timed steps)", "bound": "tensor",
                            "achieved": achieved,
                            "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / pk["bf16_tflops_sustained"],
                            "peak_source": f"bf16_tflops_sustained, of {pk_kind}", "launches": int(gemm_launches), "share_of_step_time": (gemm_ms + epi_ms) / roof_ms,
                            "with_swiglu_epilogue": {"launches": int(epi_launches), "achieved": epi_flops / (epi_ms / 1000.0) / 1e12 if epi_ms > 0 else None, "unit": "TFLOP/s",
                                                     "note": "the gate/up product that also stores m = silu(a) u and the down projection's input-gradient product that stores SwiGLU's "
                                                             "backward instead of its result: 2-3x the bytes of the plain product for the same 2mnk, counted in share_of_step_time, kept out of frac"},
                            "pass": f"second pass of the same {args.steps} steps on one stream ({roof_ms / args.steps:.2f} ms per step)",
                            "traffic": GEMM_TRAFFIC_BYTES_PER_LAUNCH if args.config == "124m" else None,
                            "traffic_launch": GEMM_TRAFFIC_LAUNCH if args.config == "124m" else None}
    if rank == 0 and world == 1 and not args.no_sdpa:
        line["sdpa_standalone"] = sdpa_standalone(be, main, pk["bf16_tflops"])
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.config == "124m":
        line["cpu_baseline"], _, _ = cpu_baseline_object(30.0, 1, 0)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if comm is not None:
        tr.set_comm(None)
    tr.close()
    if comm is not None:
        comm.close()
    be.close()
    if dist is not None:
        dist.destroy_process_group()


def sdpa_standalone(be, main_stream, peak_tflops: float) -> dict:
    """BASELINE's standalone attention case: causal SDPA forward + backward on bf16 [B 8, H 16, T 4096, D 128], N(0,1) inputs
    (seeded numpy draws), timed with CUDA events on the library's stream. FLOPs: forward 4 B H T^2 D / 2 (causal half),
    backward 2.5x (the recompute of S is counted once, as in the step's MFU)."""
    import ctypes as C
    import torch
    from ojas_b200 import DType
    from ojas_b200._lib import lib
    from ojas_b200.backend import _check, _p
    B, H, T, D = 8, 16, 4096, 128
    rng = np.random.default_rng(4)

    def draw():
        return be.upload(rng.standard_normal((B, T, H, D), dtype=np.float32), DType.BF16).permuted((0, 2, 1, 3))

    q, k, v, g = draw(), draw(), draw(), draw()
    out = be.empty((B, T, H, D), DType.BF16).permuted((0, 2, 1, 3))
    lse = be.empty((B, H, T))
    gq, gk, gv = (be.empty((B, T, H, D), DType.BF16).permuted((0, 2, 1, 3)) for _ in range(3))
    fwd = lambda: _check(lib.ojc_causal_sdpa_forward(be._handle, _p(q), _p(k), _p(v), C.c_int64(-1), _p(out), _p(lse)))
    bwd = lambda: _check(lib.ojc_causal_sdpa_backward(be._handle, _p(q), _p(k), _p(v), _p(out), _p(lse), _p(g), C.c_int64(-1), _p(gq), _p(gk), _p(gv)))
    flops = 4.0 * B * H * T * T * D / 2
    res = {"shape": [B, H, T, D], "dtype": "bf16"}
    for name, fn, mult in (("fwd", fwd, 1.0), ("bwd", bwd, 2.5)):
        for _ in range(3):
            fn()
        be.sync()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(main_stream)
        for _ in range(5):
            fn()
        b_.record(main_stream)
        be.sync()
        ms = a.elapsed_time(b_) / 5
        res[name + "_ms"] = ms
        res[name + "_tflops"] = flops * mult / ms / 1e9
    res["fwd_bwd_tflops"] = flops * 3.5 / (res["fwd_ms"] + res["bwd_ms"]) / 1e9
    res["frac_of_peak"] = res["fwd_bwd_tflops"] / peak_tflops
    return res


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the bounded CPU sample (the default run reports it)")
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "muon"], help="adamw: the headline workload; muon: the Muon NS5 + AdamW recipe of the data-parallel configs")
    ap.add_argument("--batch", type=int, default=0, help="micro-batch per GPU; anything but the workload's own is a reduced case for profiler captures only")
    ap.add_argument("--config", default="124m", choices=sorted(CONFIGS), help="124m: the headline workload; 1p7b: BASELINE's 1.3B-class data-parallel case")
    ap.add_argument("--no-second-recipe", action="store_true", help="skip the short measurement of the other optimizer recipe (Muon hybrid beside an AdamW headline)")
    ap.add_argument("--no-sdpa", action="store_true", help="skip the standalone attention case [8,16,4096,128]")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (used for profiler captures)")
    ap.add_argument("--kernel-variants", default="", help="profiler captures only: comma-separated name=value pairs passed to the library's kernel-selection "
                    "switches (ce_rows, mlp_epilogue, sdpa), e.g. ce_rows=1 to capture the cross-entropy row kernel that re-reads its row from L2; such a line names itself")
    args = ap.parse_args()
    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
