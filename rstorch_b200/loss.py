"""`Loss` trait and `CrossEntropyLoss` (src/loss/mod.rs:6-11, src/loss/cross_entropy.rs)."""
from __future__ import annotations

import ctypes as C

from .core import Tensor


class Loss:
    def forward(self, pred: Tensor, truth: Tensor) -> float:
        raise NotImplementedError

    def backward(self) -> Tensor:
        raise NotImplementedError


class CrossEntropyLoss(Loss):
    """softmax + `-(Σ t·ln p)/B`; backward returns `p - t` (cross_entropy.rs:32-48).

    One kernel produces the loss, the gradient and the accuracy of the batch, so
    `forward` already holds what `backward` returns and what `accuracy(pred, y)`
    would compute (`last_accuracy`).  `forward` blocks on the scalar like the
    reference's `-> f64`; `forward_async` queues the same work and returns a slot
    to read later with `result(slot)`."""

    def __init__(self):
        self._grad: Tensor | None = None
        self.last_accuracy: float | None = None

    def forward_async(self, pred: Tensor, truth: Tensor, slot: int | None = None) -> int:
        ctx = pred.ctx
        slot = ctx.next_result_slot() if slot is None else slot
        grad = ctx.empty(pred.rows, pred.cols)
        ctx._check(ctx._lib.rst_xent_forward_backward(ctx.handle, pred.handle, truth.handle, grad.handle, slot))
        self._grad = grad
        self._ctx = ctx
        return slot

    def result(self, slot: int) -> tuple[float, float]:
        """(loss, accuracy) of the forward that used `slot`; blocks until it is ready."""
        loss, acc = C.c_double(), C.c_double()
        self._ctx._check(self._ctx._lib.rst_xent_result(self._ctx.handle, slot, C.byref(loss), C.byref(acc)))
        return loss.value, acc.value

    def forward(self, pred: Tensor, truth: Tensor) -> float:
        slot = self.forward_async(pred, truth)
        loss, self.last_accuracy = self.result(slot)
        return loss

    def backward(self) -> Tensor:
        if self._grad is None:
            raise RuntimeError("CrossEntropyLoss::backward called without a preceding forward "
                               "(the reference panics on `truth.take().unwrap()`, cross_entropy.rs:46)")
        g, self._grad = self._grad, None
        return g
