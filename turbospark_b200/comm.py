"""The exchange object of a model sharded over the GPUs of one box (binding of tsb_comm_*).

One process per GPU.  Rank 0 makes NCCL's unique id, the host program hands its 128 bytes to every rank - here
through a torch.distributed broadcast, which is plumbing only - and every rank creates its communicator; the
collectives themselves are issued inside the library on the session's stream.
"""
import ctypes as C

import numpy as np

from .capi import lib


class Comm:
    def __init__(self, ctx, rank=0, world=1, unique_id=None):
        self.ctx, self.rank, self.world = ctx, rank, world
        h = C.c_void_p()
        idbuf = (C.c_ubyte * 128).from_buffer_copy(bytes(unique_id)) if unique_id is not None else None
        ctx.check(lib().tsb_comm_create(ctx.h, idbuf, C.c_int32(rank), C.c_int32(world), C.byref(h)))
        self.h = h

    @staticmethod
    def unique_id(ctx):
        buf = (C.c_ubyte * 128)()
        ctx.check(lib().tsb_comm_unique_id(ctx.h, buf))
        return bytes(buf)

    @classmethod
    def from_torch_distributed(cls, ctx):
        """Inside an initialised torch.distributed job: rank 0's id travels by broadcast (any backend)."""
        import torch
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        if world == 1:
            return cls(ctx, 0, 1)
        t = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            t = torch.tensor(list(cls.unique_id(ctx)), dtype=torch.uint8)
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        t = t.to(dev)
        dist.broadcast(t, 0)
        return cls(ctx, rank, world, bytes(t.cpu().numpy().tobytes()))

    def all_reduce_f32(self, buf, count, stream=None):
        self.ctx.check(lib().tsb_comm_all_reduce_f32(self.h, stream, C.c_void_p(buf.ptr), C.c_size_t(count)))

    def close(self):
        if getattr(self, "h", None):
            lib().tsb_comm_destroy(self.h)
            self.h = None
