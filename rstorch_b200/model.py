"""`BasicModel` (src/model.rs:4-32): a module, a loss and an optimiser bundled
into the reference's own statement of the training step and of inference."""
from __future__ import annotations

from .core import Tensor
from .loss import Loss
from .module import Module
from .optim import Optimizer


class BasicModel:
    """`BasicModel::new(module, loss, optim)` (model.rs:11-17)."""

    def __init__(self, module: Module, loss: Loss, optim: Optimizer):
        self.module, self.loss, self.optim = module, loss, optim

    @classmethod
    def new(cls, module: Module, loss: Loss, optim: Optimizer) -> "BasicModel":
        return cls(module, loss, optim)

    def step(self, input: Tensor, truth: Tensor) -> None:
        """forward, loss.forward, loss.backward, backward, optim.step, in that order
        (model.rs:19-27).  The loss value is dropped, as in the reference; read it from
        `self.loss` if the loss keeps it."""
        pred = self.module.forward(input)
        self.loss.forward(pred, truth)
        gradient = self.loss.backward()
        self.module.backward(gradient)
        self.optim.step(self.module)

    def predict(self, input: Tensor) -> Tensor:
        """`module.forward(input)` (model.rs:29-31).  Like the reference it goes through
        the training forward, so the layers cache their inputs; a following `step` simply
        overwrites those caches."""
        return self.module.forward(input)
