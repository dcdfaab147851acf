"""`Optimizer` trait and `SGD` (src/optim/mod.rs:6-8, src/optim/sgd.rs)."""
from __future__ import annotations

from .core import handle_array
from .module import Module


class Optimizer:
    def step(self, module: Module) -> None:
        raise NotImplementedError


class SGD(Optimizer):
    """`parm = parm - (lr * grad)` for every parameter of the module (sgd.rs:18-25),
    as one kernel launch over all of them."""

    def __init__(self, lr: float):
        self.lr = float(lr)

    @classmethod
    def new(cls, lr: float) -> "SGD":
        return cls(lr)

    def step(self, module: Module) -> None:
        params = module.parameters()
        if not params:
            return
        ctx = params[0].parm.ctx
        p = handle_array([q.parm for q in params])
        g = handle_array([q.grad for q in params])
        ctx._check(ctx._lib.rst_sgd_step(ctx.handle, len(params), p, g, self.lr))
