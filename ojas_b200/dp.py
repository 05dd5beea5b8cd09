"""Data-parallel gradient exchange for the training step (new: the reference has no distributed code).

Each rank runs the identical forward/backward on its own micro-batch with the backward seeded by 1/world, exactly the
reference's K-micro-batch weighting (MicroWeights, ojas-model/src/trainer.rs:1083-1119); gradients are then summed across
ranks bucket by bucket, after which every rank runs the same clip and optimizer and stays bit-identical to its peers.
`torch.distributed` (NCCL on GPUs, gloo in the CPU tests) carries the collectives; no kernel here reads a peer's memory.
"""
from __future__ import annotations


def allreduce_sum_(tensors, group=None, async_op: bool = False):
    """Sum every tensor in place across the group; returns the work handles when async_op."""
    import torch.distributed as dist
    works = [dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group, async_op=async_op) for t in tensors]
    return works if async_op else None


class DevPtr:
    """Lets torch view library-owned device memory without a copy (CUDA array interface)."""

    def __init__(self, ptr: int, n: int):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 3}


class BucketAllReduce:
    """One all-reduce per ~25 MB gradient bucket, issued on a side stream as soon as the bucket's ready event (recorded by
    the step driver during backward) fires, so the exchange overlaps the rest of backward. The library's own stream then
    waits for every bucket before clip + optimizer run."""

    def __init__(self, backend, trainer, device):
        import torch
        self.torch, self.backend = torch, backend
        self.comm_stream = torch.cuda.Stream(device=device)
        self.main_stream = torch.cuda.ExternalStream(backend.stream(), device=device)
        self.buckets = [(torch.as_tensor(DevPtr(ptr, n), device=device), ev) for ptr, n, ev in trainer.buckets()]

    def exchange(self):
        torch = self.torch
        works = []
        for tensor, event in self.buckets:
            self.backend.stream_wait_event(self.comm_stream.cuda_stream, event)
            with torch.cuda.stream(self.comm_stream):
                works.extend(allreduce_sum_([tensor], async_op=True))
        with torch.cuda.stream(self.main_stream):
            for w in works:
                w.wait()
