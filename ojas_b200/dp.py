"""Data-parallel gradient exchange for the training step (new: the reference has no distributed code).

Each rank runs the identical forward/backward on its own micro-batch with the backward seeded by 1/world, exactly the
reference's K-micro-batch weighting (MicroWeights, ojas-model/src/trainer.rs:1083-1119); gradients are then summed across
ranks bucket by bucket, after which every rank runs the same clip and optimizer and stays bit-identical to its peers.
The exchange itself lives behind the C ABI (ojc_comm_*, ojc_allreduce_start / _wait: NCCL reached with dlopen, include/ojas_cuda.h);
`Communicator` is its ctypes face and needs only some way to hand rank 0's 128-byte id to the other ranks. `BucketAllReduce` is the
same exchange carried by `torch.distributed` instead (gloo in the CPU tests). No kernel here reads a peer's memory.
"""
from __future__ import annotations

import ctypes as C


class Communicator:
    """ojc_comm: one NCCL communicator for a CudaBackend. `share_id(id_bytes_or_None) -> id_bytes` must return rank 0's id on every
    rank (rank 0 passes its fresh id in, the others pass None): a torch.distributed broadcast, a file, a socket."""

    def __init__(self, backend, rank: int, world: int, share_id):
        from ._lib import lib
        from .backend import _check
        self._h = None
        self.backend, self.rank, self.world = backend, rank, world
        buf = (C.c_uint8 * 128)()
        if rank == 0:
            _check(lib.ojc_comm_unique_id(buf))
        ident = share_id(bytes(buf) if rank == 0 else None)
        assert len(ident) == 128
        buf = (C.c_uint8 * 128).from_buffer_copy(ident)
        h = C.c_void_p()
        _check(lib.ojc_comm_init(backend._handle, C.c_int32(rank), C.c_int32(world), buf, C.byref(h)))
        self._h = h

    @staticmethod
    def over_torch_distributed(backend, group=None) -> "Communicator":
        """Rendezvous through an initialised torch.distributed process group of any backend (used for the id only)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)

        def share(ident):
            box = [ident]
            dist.broadcast_object_list(box, src=0, group=group)
            return box[0]
        return Communicator(backend, rank, world, share)

    def allreduce_sum_f32(self, tensor) -> None:
        """In place on a library tensor (F32), on the backend's stream."""
        from ._lib import lib
        from .backend import _check
        _check(lib.ojc_comm_allreduce(self._h, C.c_void_p(tensor.ptr), C.c_uint64(tensor.numel), C.c_int32(0), C.c_int32(0)))

    def check(self) -> None:
        from ._lib import lib
        from .backend import _check
        _check(lib.ojc_comm_check(self._h))

    def close(self) -> None:
        if self._h:
            from ._lib import lib
            if self.backend._handle:
                lib.ojc_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


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
