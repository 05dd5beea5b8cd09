"""Data parallelism on CPU ranks (gloo, world_size 2): summing per-rank gradients seeded with 1/world equals the
reference's gradient accumulation over K = world micro-batches (ojas-model/src/trainer.rs:892-1001), and every rank
ends with the same bits."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
KW = dict(vocab=64, n_embd=32, n_layer=2, n_head=2, n_kv_head=1, head_dim=16, hidden=48, max_seq=16)


def _batches():
    from oracle import oracle as orc
    rng = orc.SplitMix64(5)
    draws = np.array([rng.below(64) for _ in range(2 * 2 * 17)], np.uint32).reshape(2, 2, 17)
    return [(draws[r, :, :-1].copy(), draws[r, :, 1:].copy()) for r in range(2)]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc
    from ojas_b200.dp import allreduce_sum_
    spec = orc.Spec(**KW)
    params = orc.init_params(spec, 0, normal_everywhere=True)
    x, y = _batches()[rank]
    loss, grads, _ = orc.forward_loss(spec, params, x, y, seed=1.0 / world)
    tensors = [torch.from_numpy(g) for g in grads]
    allreduce_sum_(tensors)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), *[t.numpy() for t in tensors], loss=np.float32(loss))
    dist.destroy_process_group()


def test_two_rank_sum_equals_two_micro_batch_accumulation(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    from oracle import oracle as orc
    spec = orc.Spec(**KW)
    params = orc.init_params(spec, 0, normal_everywhere=True)
    acc = None
    for x, y in _batches():
        _, grads, _ = orc.forward_loss(spec, params, x, y, seed=0.5)
        if acc is None:
            acc = [g.copy() for g in grads]
        else:
            for a, g in zip(acc, grads):
                orc.lib.orc_accumulate_grad(a.ctypes.data_as(__import__("ctypes").c_void_p), g.ctypes.data_as(__import__("ctypes").c_void_p),
                                            __import__("ctypes").c_int64(a.size))
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for i, want in enumerate(acc):
        a, b = r0[f"arr_{i}"], r1[f"arr_{i}"]
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))  # ranks agree bit for bit
        assert np.array_equal(a.view(np.uint32), want.view(np.uint32))  # two-term sums: the same bits as accumulation
