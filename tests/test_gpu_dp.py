"""Data parallelism on real GPUs (NCCL, one process per GPU): needs at least two devices, skipped otherwise.

Two ranks run the step driver on their own micro-batches with the backward seeded by 1/world, exchange the gradient
buckets (ojas_b200/dp.py) and apply the optimizer. Checked: the reduced gradients equal the CPU oracle's sum of the two
seeded micro-batch gradients (the reference's K = 2 accumulation, ojas-model/src/trainer.rs:892-1001) at the f32 gate,
and after two steps both ranks hold the same parameter bits. Under bf16 autocast the weight gradients are written on the
driver's second stream, so this also covers the ordering of that stream against the bucket-ready events.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]

WORKER = r"""
import json, os, sys
import numpy as np
import torch, torch.distributed as dist
from safetensors import safe_open
sys.path.insert(0, os.environ["OJAS_ROOT"])
from ojas_b200 import CudaBackend, TrainConfig, Trainer, checkpoint as ck
from ojas_b200.dp import BucketAllReduce

rank, world, out = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), os.environ["OJAS_OUT"]
autocast = os.environ["OJAS_AUTOCAST"] == "1"
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
f = safe_open(os.path.join(os.environ["OJAS_ROOT"], "tests", "golden", "tiny", "init.safetensors"), "np")
spec = ck.spec_from_json(f.metadata()["ojas.spec"])
be = CudaBackend(rank, 8 << 30)
tr = Trainer(be, spec, TrainConfig(optimizer="muon", autocast_bf16=autocast, ns5_bf16=autocast, loss_seed=1.0 / world), 2, 32)
tr.set_params([f.get_tensor(p.name) for p in tr.params])
reducer = BucketAllReduce(be, tr, torch.device("cuda", rank))
rng = np.random.default_rng(100 + rank)
result = {}
for step in range(2):
    b = rng.integers(0, spec.vocab, (2, 33), dtype=np.uint32)
    ids, tg = be.upload(np.ascontiguousarray(b[:, :-1])), be.upload(np.ascontiguousarray(b[:, 1:]))
    tr.gradients_device(ids, tg)
    reducer.exchange()
    be.sync()
    if step == 0:
        result.update({"g." + p.name: tr.get_grad(i) for i, p in enumerate(tr.params) if p.trains})
        result["batch"] = b
    tr.apply(read_norm=False)
    tr.finish()
result.update({"p." + p.name: tr.get_param(i) for i, p in enumerate(tr.params)})
np.savez(os.path.join(out, f"rank{rank}.npz"), **result)
dist.barrier()
tr.close(); be.close()
dist.destroy_process_group()
"""


@pytest.mark.parametrize("autocast", [False, True])
def test_two_ranks_reduce_to_the_accumulated_gradient_and_stay_bit_identical(tmp_path, golden_dir, autocast):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from safetensors import safe_open
    from oracle import oracle as orc
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OJAS_ROOT=str(ROOT), OJAS_OUT=str(tmp_path), OJAS_AUTOCAST="1" if autocast else "0", NCCL_NVLS_ENABLE="0")
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29533" if autocast else "29532", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    names = [k for k in r0.files if k.startswith("p.")]
    assert names and all(r0[k].tobytes() == r1[k].tobytes() for k in names), "ranks diverged"
    grads = [k for k in r0.files if k.startswith("g.")]
    assert all(r0[k].tobytes() == r1[k].tobytes() for k in grads), "ranks hold different reduced gradients"

    f = safe_open(str(golden_dir / "tiny" / "init.safetensors"), "np")
    s = json.loads(f.metadata()["ojas.spec"])
    spec = orc.Spec(vocab=s["vocab"], n_embd=s["n_embd"], n_layer=s["n_layer"], n_head=s["n_head"], n_kv_head=s["n_kv_head"], head_dim=s["head_dim"],
                    hidden=s["hidden"], max_seq=s["max_seq"], window=s.get("window"), rope_base=s["rope_base"], rms_eps=s["rms_eps"])
    table = [p.name for p in orc.param_table(spec)]
    params = [f.get_tensor(name) for name in table]
    total = None
    for r in (r0, r1):
        b = r["batch"]
        _, g, _ = orc.forward_loss(spec, params, b[:, :-1], b[:, 1:], seed=0.5)
        total = [a.copy() for a in g] if total is None else [a + c for a, c in zip(total, g)]
    total = dict(zip(table, total))
    tol = 3e-2 if autocast else 1e-4
    for k in grads:
        want, got = total[k[2:]].astype(np.float64).ravel(), r0[k].astype(np.float64).ravel()
        if not np.any(want):
            assert not np.any(got), k
        else:
            assert np.linalg.norm(got - want) / np.linalg.norm(want) <= tol, (k, np.linalg.norm(got - want) / np.linalg.norm(want))


COMM_WORKER = r"""
import os, sys
import numpy as np
import torch.distributed as dist
from safetensors import safe_open
sys.path.insert(0, os.environ["OJAS_ROOT"])
from ojas_b200 import CudaBackend, TrainConfig, Trainer, checkpoint as ck
from ojas_b200.dp import Communicator

rank, world, out = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), os.environ["OJAS_OUT"]
dist.init_process_group("gloo")                      # carries the communicator's 128-byte id and nothing else
f = safe_open(os.path.join(os.environ["OJAS_ROOT"], "tests", "golden", "tiny", "init.safetensors"), "np")
spec = ck.spec_from_json(f.metadata()["ojas.spec"])
be = CudaBackend(rank, 8 << 30)
comm = Communicator.over_torch_distributed(be)
rng = np.random.default_rng(7)
batches = [rng.integers(0, spec.vocab, (2, 33), dtype=np.uint32) for _ in range(2 * 2 * world)]   # 2 steps x K 2 x world ranks
result = {"batches": np.stack(batches)}
for shard in (0, 1):
    tr = Trainer(be, spec, TrainConfig(optimizer="muon", loss_seed=1.0 / world, schedule="cosine", warmup_steps=1, total_steps=4), 2, 32)
    tr.set_params([f.get_tensor(p.name) for p in tr.params])
    tr.set_comm(comm, shard_muon=bool(shard))
    for step in range(2):
        mine = [batches[step * 2 * world + rank * 2 + k] for k in range(2)]
        rep = tr.run([(b[:, :-1], b[:, 1:]) for b in mine])
        result[f"loss{shard}.{step}"] = np.float32(rep.loss)
        result[f"norm{shard}.{step}"] = np.float32(rep.grad_norm)
    result[f"exposed{shard}"] = np.float32(tr.exposed_exchange_ms())
    result[f"sum{shard}"] = np.uint64(tr.param_checksum())
    tr.sync_moments()
    result.update({f"p{shard}." + p.name: tr.get_param(i) for i, p in enumerate(tr.params)})
    result.update({f"m{shard}." + p.name: tr.get_moment(i, 0) for i, p in enumerate(tr.params) if p.trains})
    tr.set_comm(None)
    tr.close()
np.savez(os.path.join(out, f"comm{rank}.npz"), **result)
dist.barrier()
comm.close(); be.close()
dist.destroy_process_group()
"""


def test_the_library_communicator_runs_the_data_parallel_step_and_splits_muon(tmp_path, golden_dir):
    """The exchange behind the C ABI (ojc_comm_*, NCCL by dlopen) with K = 2 micro-batches per rank on two ranks: parameters after two
    steps equal the CPU oracle's Trainer::run over the four micro-batches of each step (the K = world x 2 accumulation the exchange
    stands for) at the f32 gates, both ranks hold the same bits, and splitting the Muon phase across the ranks changes no bit."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from safetensors import safe_open
    from oracle import oracle as orc
    script = tmp_path / "comm_worker.py"
    script.write_text(COMM_WORKER)
    env = dict(os.environ, OJAS_ROOT=str(ROOT), OJAS_OUT=str(tmp_path), NCCL_NVLS_ENABLE="0")
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29534", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    r0, r1 = np.load(tmp_path / "comm0.npz"), np.load(tmp_path / "comm1.npz")
    for shard in (0, 1):
        keys = [k for k in r0.files if k.startswith((f"p{shard}.", f"m{shard}."))]
        assert keys and all(r0[k].tobytes() == r1[k].tobytes() for k in keys), "ranks diverged"
        assert r0[f"sum{shard}"] == r1[f"sum{shard}"] and r0[f"exposed{shard}"] >= 0.0
    for k in [k for k in r0.files if k.startswith("p0.")]:
        assert r0[k].tobytes() == r0["p1." + k[3:]].tobytes(), ("splitting Muon across ranks changed", k)
    for k in [k for k in r0.files if k.startswith("m0.")]:
        assert r0[k].tobytes() == r0["m1." + k[3:]].tobytes(), ("momentum after sync_moments differs", k)

    f = safe_open(str(golden_dir / "tiny" / "init.safetensors"), "np")
    s = json.loads(f.metadata()["ojas.spec"])
    spec = orc.Spec(**{k: s[k] for k in ("vocab", "n_embd", "n_layer", "n_head", "n_kv_head", "head_dim", "hidden", "max_seq", "rope_base", "rms_eps")})
    table = orc.param_table(spec)
    otr = orc.TrainerOracle(spec, [f.get_tensor(i.name) for i in table], schedule=("cosine", 1, 4))
    batches = r0["batches"]
    for step in range(2):
        loss, norm, _ = otr.run([(b[:, :-1], b[:, 1:]) for b in batches[step * 4:(step + 1) * 4]])
        mean = 0.5 * (float(r0[f"loss0.{step}"]) + float(r1[f"loss0.{step}"]))      # each rank reports the mean of its own micro-batches
        assert abs(mean - loss) <= 1e-5 * abs(loss) and abs(float(r0[f"norm0.{step}"]) - norm) <= 1e-4 * norm
    for i, info in enumerate(table):
        want, got = otr.params[i].astype(np.float64).ravel(), r0["p0." + info.name].astype(np.float64).ravel()
        assert np.linalg.norm(got - want) <= 1e-4 * max(np.linalg.norm(want), 1e-30), info.name


def test_two_backends_on_two_devices_in_one_process():
    """Function attributes (dynamic shared-memory limits, cluster occupancy) are per device: a second backend on another GPU must set its
    own, or its first tensor-core launch fails. One process, two devices, the kernels that need more than 48 KB of shared memory."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import oracle as orc
    from ojas_b200 import CudaBackend, DType
    x, w = orc.round_bf16(orc.SplitMix64(1).vec(512 * 256, 0.5).reshape(512, 256)), orc.round_bf16(orc.SplitMix64(2).vec(768 * 256, 0.5).reshape(768, 256))
    q = orc.round_bf16(orc.init_normal("q", 5, 1.0, (1, 2, 384, 128)))
    want_y = orc.linear_forward(x, w)
    want_o, _ = orc.causal_sdpa_forward(q, q, q)
    for device in (0, 1):
        be = CudaBackend(device, 4 << 30)
        try:
            y = be.linear_forward(be.upload(x, DType.BF16), be.upload(w, DType.BF16), out_dtype=DType.F32).numpy()      # two-SM tcgen05 GEMM
            assert np.linalg.norm(y - want_y) <= 1e-5 * np.linalg.norm(want_y), device
            dq = be.upload(q, DType.BF16)
            o, lse = be.causal_sdpa_forward(dq, dq, dq)                                                                 # tcgen05 attention, head_dim 128
            gq, gk, gv = be.causal_sdpa_backward(dq, dq, dq, o, lse, dq)
            assert np.linalg.norm(o.numpy() - want_o) <= 2e-2 * np.linalg.norm(want_o), device
            assert np.isfinite(gq.numpy()).all() and np.isfinite(gk.numpy()).all() and np.isfinite(gv.numpy()).all()
            be.sync()
        finally:
            be.close()
