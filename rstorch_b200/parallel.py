"""Data-parallel gradient exchange: one process per GPU, NCCL over NVLink.

The reference is single-threaded (no counterpart).  Each rank runs the step on
its `B/G` rows; `Linear::backward` divides by the local row count
(src/module/linear.rs:62-66), so the average over ranks of every dW/db equals
the full-batch gradient.  The exchange of a layer starts as soon as its
gradients are queued and overlaps the rest of the backward pass.

A `Communicator` switches its context to exchanging shares: `Linear::backward`
divides by the global row count `B` instead of `B/G`, and the exchange adds the
shares up.  The gradients after the exchange are the same averages; between a
layer's backward and its exchange they hold 1/G of the local-batch gradient.
A plain sum is what NCCL can reduce inside the NVSwitch.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from .core import Context, handle_array
from .module import Linear, Sequential


class Communicator:
    def __init__(self, ctx: Context, rank: int, world: int, id_bytes: bytes):
        self.ctx, self.rank, self.world = ctx, int(rank), int(world)
        if len(id_bytes) != _lib.COMM_ID_BYTES:
            raise ValueError("bad communicator id")
        buf = C.create_string_buffer(id_bytes, _lib.COMM_ID_BYTES)
        h = C.c_void_p()
        ctx._check(ctx._lib.rst_comm_create(ctx.handle, buf, self.rank, self.world, C.byref(h)))
        self.handle = h
        # Ranks exchange shares of the global-batch gradient (each divides by B, not B/G) and
        # the exchange is a plain sum, which NCCL can reduce inside the NVSwitch; the result is
        # the same average.  RSTORCH_B200_SHARE_GRADIENTS=0 keeps the averaging exchange.
        import os
        self.shares = os.environ.get("RSTORCH_B200_SHARE_GRADIENTS", "1") != "0"
        if self.shares:
            ctx._check(ctx._lib.rst_comm_share_gradients(h, 1))

    @staticmethod
    def new_id() -> bytes:
        """Rank 0 calls this and ships the bytes to the other ranks."""
        lib = _lib.load()
        buf = C.create_string_buffer(_lib.COMM_ID_BYTES)
        _lib.check(lib.rst_comm_get_id(buf))
        return buf.raw

    @classmethod
    def from_torch_distributed(cls, ctx: Context) -> "Communicator":
        """Bootstraps over an initialised torch.distributed process group (any backend)."""
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        box = [cls.new_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        return cls(ctx, rank, world, box[0])

    def allreduce_avg(self, tensors) -> None:
        if tensors:
            self.ctx._check(self.ctx._lib.rst_allreduce_avg(self.handle, len(tensors), handle_array(tensors)))

    def join(self) -> None:
        """Makes the compute stream wait for every exchange queued so far."""
        self.ctx._check(self.ctx._lib.rst_comm_join(self.handle))

    def close(self) -> None:
        if self.handle is not None and self.handle.value and self.ctx.handle.value:
            self.ctx._lib.rst_comm_destroy(self.handle)
        self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_rows(global_batch: int, rank: int, world: int) -> tuple[int, int]:
    """(first_row, rows) of rank `rank`; the batch must split evenly, as the
    average of per-rank means equals the global mean only for equal shards."""
    if global_batch % world != 0:
        raise ValueError(f"global batch {global_batch} does not split evenly over {world} ranks")
    rows = global_batch // world
    return rank * rows, rows


def backward_with_exchange(model: Sequential, gradient, comm: Communicator | None,
                           need_input_grad: bool = False):
    """`model.backward` with each Linear's dW/db all-reduced (averaged) as soon
    as they are queued; returns once every exchange is ordered before the next
    work on the compute stream (i.e. the optimiser step)."""
    if comm is None or comm.world == 1:
        return model.backward(gradient, need_input_grad=need_input_grad)

    def exchange(layer: Linear) -> None:
        comm.allreduce_avg([layer.grad_weight, layer.grad_bias])

    out = model.backward(gradient, need_input_grad=need_input_grad, on_layer_grads=exchange)
    comm.join()
    return out
