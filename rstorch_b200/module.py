"""Host-side mirror of the reference's `module` layer over the C ABI.

Names, argument meaning and error behaviour follow the Rust crate:
`Module` (src/module/mod.rs:42-56), `Parameter`/`Parameters` (:16-40), `Linear`
(src/module/linear.rs), `ReLU` (src/module/activation/relu.rs), `Identity`
(src/module/activation/identity.rs), `Sequential` and `sequential!`
(src/module/sequential.rs), `InitParameters`/`KaimingNormal`
(src/module/init/mod.rs:11-18, he.rs:9-15).  Where the reference panics
(`unwrap()` on a missing cache) these classes raise `RstError`/`RuntimeError`.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Iterable, Sequence

import numpy as np

from . import synth
from .core import Context, Tensor


@dataclass
class Parameter:
    """One `(parm, grad)` pair, as `Parameters::iter` yields them (module/mod.rs:16-19)."""
    parm: Tensor
    grad: Tensor


class InitParameters:
    """Weight-injection hook (module/init/mod.rs:11-18): `weight` returns an
    `(output_size, input_size)` array, `bias` a `(1, output_size)` array."""

    def weight(self, input_size: int, output_size: int) -> np.ndarray:
        raise NotImplementedError

    def bias(self, input_size: int, output_size: int) -> np.ndarray:
        return np.zeros((1, output_size), dtype=np.float64)


class KaimingNormal(InitParameters):
    """N(0, 1/sqrt(input_size)) weights, zero bias (module/init/he.rs:9-15).  The
    reference draws from a thread-seeded generator and is not reproducible; here
    the stream is the package's counter-based generator keyed by `seed`, advanced
    once per layer so that successive layers get independent streams."""

    def __init__(self, seed: int = 0):
        self.seed = int(seed)
        self._layer = 0

    def weight(self, input_size: int, output_size: int) -> np.ndarray:
        stream = synth.stream_key(self.seed, "weight", self._layer)
        self._layer += 1
        return synth.normal(stream, output_size * input_size, std=1.0 / np.sqrt(input_size)).reshape(
            output_size, input_size)


# The initialiser a `Linear` gets when none is passed.  The reference draws every layer
# from the thread generator (he.rs:13), so successive layers are independent; one shared
# instance, whose stream index advances with every weight matrix it hands out, gives the
# same property (layer k built in a process draws stream ("weight", k) of seed 0).
_default_init = KaimingNormal(0)


def reset_default_init(seed: int = 0) -> None:
    """Restarts the default initialiser's stream counter (tests and reproducible scripts)."""
    global _default_init
    _default_init = KaimingNormal(seed)


class XavierNormal(InitParameters):
    """N(0, sqrt(2 / (input_size + output_size))) weights (module/init/xavier.rs:9-15)."""

    def __init__(self, seed: int = 0):
        self.seed, self._layer = int(seed), 0

    def weight(self, input_size: int, output_size: int) -> np.ndarray:
        stream = synth.stream_key(self.seed, "xavier", self._layer)
        self._layer += 1
        sigma = np.sqrt(2.0 / (float(input_size) + float(output_size)))
        return synth.normal(stream, output_size * input_size, std=sigma).reshape(output_size, input_size)


class Normal(InitParameters):
    """N(mean, std) weights (module/init/sigma.rs:7-37); `new` returns None for a
    non-finite std, like the reference's `Option`."""

    def __init__(self, mean: float, std: float, seed: int = 0):
        self.mean, self.std, self.seed, self._layer = float(mean), float(std), int(seed), 0

    @classmethod
    def new(cls, mean: float, std: float, seed: int = 0) -> "Normal | None":
        return cls(mean, std, seed) if np.isfinite(std) else None

    @classmethod
    def new_std(cls, std: float, seed: int = 0) -> "Normal | None":
        return cls.new(0.0, std, seed)

    def weight(self, input_size: int, output_size: int) -> np.ndarray:
        stream = synth.stream_key(self.seed, "normal", self._layer)
        self._layer += 1
        return synth.normal(stream, output_size * input_size, std=self.std, mean=self.mean).reshape(
            output_size, input_size)


class Module:
    """`trait Module` (module/mod.rs:42-56)."""

    def forward(self, input: Tensor) -> Tensor:      # (batch, in) -> (batch, out)
        raise NotImplementedError

    def backward(self, gradient: Tensor) -> Tensor:  # (batch, out) -> (batch, in)
        raise NotImplementedError

    def parameters(self) -> list[Parameter]:
        return []

    def train(self) -> None:
        pass

    def eval(self) -> None:
        pass


class Identity(Module):
    """Pass-through in both directions (activation/identity.rs:15-29)."""

    def forward(self, input: Tensor) -> Tensor:
        return input

    def backward(self, gradient: Tensor) -> Tensor:
        return gradient


class ReLU(Module):
    """max(x, 0); backward multiplies by (x > 0) (activation/relu.rs:17-32).

    The cache is any tensor whose sign pattern equals the pre-activation's: the
    pre-activation itself when called stand-alone, the post-ReLU output when a
    `Sequential` fused the forward into the preceding Linear's epilogue
    (max(x,0) > 0 exactly when x > 0)."""

    def __init__(self):
        self.prev_input: Tensor | None = None

    def forward(self, input: Tensor) -> Tensor:
        ctx = input.ctx
        out = ctx.empty(input.rows, input.cols)
        ctx._check(ctx._lib.rst_relu_forward(ctx.handle, input.handle, out.handle))
        self.prev_input = input              # the reference keeps a clone (relu.rs:20)
        return out

    def backward(self, gradient: Tensor) -> Tensor:
        prev = self._take()
        ctx = gradient.ctx
        out = ctx.empty(gradient.rows, gradient.cols)
        ctx._check(ctx._lib.rst_relu_backward(ctx.handle, gradient.handle, prev.handle, out.handle))
        return out

    def _take(self) -> Tensor:
        if self.prev_input is None:
            raise RuntimeError("ReLU::backward called without a preceding forward "
                               "(the reference panics on `prev_input.take().unwrap()`, relu.rs:26)")
        prev, self.prev_input = self.prev_input, None
        return prev


class Softmax(Module):
    """Softmax as a layer (activation/softmax.rs:5-34, 55-78).  The backward is the
    reference's, kept as written: a Jacobian `-(Oᵀ·O)` over the whole batch with the
    diagonal replaced by s(1-s), applied as `gradient · jacobian` (softmax.rs:62-75)."""

    def __init__(self, axis: int = 1):
        if axis not in (0, 1):
            raise IndexError(f"axis {axis} out of range for a 2-D array")
        self.axis = axis
        self.output: Tensor | None = None

    @classmethod
    def with_axis(cls, axis: int) -> "Softmax":
        return cls(axis)

    def forward(self, input: Tensor) -> Tensor:
        ctx = input.ctx
        out = ctx.empty(input.rows, input.cols)
        fn = ctx._lib.rst_softmax if self.axis == 1 else ctx._lib.rst_softmax_axis0
        ctx._check(fn(ctx.handle, input.handle, out.handle))
        self.output = out
        return out

    def backward(self, gradient: Tensor) -> Tensor:
        if self.output is None:
            raise RuntimeError("Softmax::backward called without a preceding forward "
                               "(the reference panics on `output.take().unwrap()`, softmax.rs:63)")
        output, self.output = self.output, None
        ctx = gradient.ctx
        dx = ctx.empty(gradient.rows, output.cols)
        ctx._check(ctx._lib.rst_softmax_backward(ctx.handle, output.handle, gradient.handle, dx.handle))
        return dx


class Linear(Module):
    """y = x·Wᵀ + b (module/linear.rs).  `weight` is (out, in), `bias` (1, out)."""

    def __init__(self, input_size: int, output_size: int, init: InitParameters | None = None,
                 ctx: Context | None = None, bias: bool = True):
        init = init if init is not None else _default_init
        self.input_size, self.output_size = int(input_size), int(output_size)
        self._host_weight = np.ascontiguousarray(init.weight(input_size, output_size), dtype=np.float64)
        self.has_bias = bool(bias)
        self._host_bias = (np.ascontiguousarray(init.bias(input_size, output_size), dtype=np.float64)
                           if self.has_bias else None)
        self.weight: Tensor | None = None
        self.bias: Tensor | None = None
        self.prev_input: Tensor | None = None
        self.grad_weight: Tensor | None = None
        self.grad_bias: Tensor | None = None
        if ctx is not None:
            self.to(ctx)

    @classmethod
    def new_with_kernel(cls, input_size: int, output_size: int, init: InitParameters,
                        ctx: Context | None = None) -> "Linear":
        return cls(input_size, output_size, init, ctx)

    @classmethod
    def without_bias(cls, input_size: int, output_size: int, init: InitParameters | None = None,
                     ctx: Context | None = None) -> "Linear":
        """A layer whose `bias` is `None`.  The reference's struct holds `bias:
        Option<Array2<f64>>` and branches on it in forward, backward and parameters
        (linear.rs:51-53, 65-67, 74-77), although its public constructors always fill
        it (:27); this constructor reaches those branches: y = x·Wᵀ, no db, one
        parameter pair."""
        return cls(input_size, output_size, init, ctx, bias=False)

    def to(self, ctx: Context) -> "Linear":
        """Uploads the parameters (done lazily by the first forward otherwise)."""
        if self.weight is None or self.weight.ctx is not ctx:
            self.weight = ctx.tensor(self._host_weight)
            self.bias = ctx.tensor(self._host_bias) if self.has_bias else None
        return self

    # -- forward -------------------------------------------------------------
    def forward(self, input: Tensor) -> Tensor:
        return self._forward(input, fuse_relu=False)

    def _forward(self, input: Tensor, fuse_relu: bool) -> Tensor:
        ctx = input.ctx
        self.to(ctx)
        out = ctx.empty(input.rows, self.output_size)
        ctx._check(ctx._lib.rst_linear_forward(ctx.handle, input.handle, self.weight.handle,
                                               self.bias.handle if self.has_bias else None,
                                               1 if fuse_relu else 0, out.handle))
        self.prev_input = input               # moved in, not copied (linear.rs:55)
        return out

    # -- backward ------------------------------------------------------------
    def backward(self, gradient: Tensor) -> Tensor:
        return self._backward(gradient, relu_mask=False, need_input_grad=True)

    # dX of a layer whose 128x128 output tiles fill the GPU runs 4 % faster from a transposed
    # copy of the incoming gradient (both operands then have the reduction index outermost).
    _TRANSPOSED_GRADIENT_MIN_ELEMS = 148 * 128 * 128

    def _backward(self, gradient: Tensor, relu_mask: bool, need_input_grad: bool,
                  want_transposed: bool = False) -> Tensor | None:
        """`want_transposed`: the caller will hand the returned gradient to another large
        Linear, so attach its transposed companion (`dx.t`), written by the same kernel."""
        if self.prev_input is None:
            raise RuntimeError("Linear::backward called without a preceding forward "
                               "(the reference panics on `prev_input.take().unwrap()`, linear.rs:61)")
        x, self.prev_input = self.prev_input, None
        ctx = gradient.ctx
        # gradients are overwritten, never accumulated (linear.rs:63,66)
        if self.grad_weight is None or self.grad_weight.ctx is not ctx:
            self.grad_weight = ctx.empty(self.output_size, self.input_size)
            self.grad_bias = ctx.empty(1, self.output_size) if self.has_bias else None   # linear.rs:65
        db = self.grad_bias.handle if self.has_bias else None
        dx = ctx.empty(x.rows, x.cols) if need_input_grad else None
        mask = x.handle if (relu_mask and dx is not None) else None
        large = (dx is not None and x.rows * x.cols >= self._TRANSPOSED_GRADIENT_MIN_ELEMS
                 and x.rows % 2 == 0 and x.cols % 4 == 0)
        if not large:
            ctx._check(ctx._lib.rst_linear_backward(
                ctx.handle, gradient.handle, x.handle, self.weight.handle, mask,
                self.grad_weight.handle, db, dx.handle if dx is not None else None))
            return dx
        if gradient.t is None:              # the loss gradient: make the first companion
            gradient.t = ctx.empty(gradient.cols, gradient.rows)
            ctx._check(ctx._lib.rst_transpose(ctx.handle, gradient.handle, gradient.t.handle))
        if want_transposed:
            dx.t = ctx.empty(x.cols, x.rows)
        ctx._check(ctx._lib.rst_linear_backward_t(
            ctx.handle, gradient.handle, gradient.t.handle, x.handle, self.weight.handle, mask,
            self.grad_weight.handle, db, dx.handle,
            dx.t.handle if dx.t is not None else None))
        return dx

    def parameters(self) -> list[Parameter]:
        if self.grad_weight is None or (self.has_bias and self.grad_bias is None):
            raise RuntimeError("Linear::parameters called before any backward "
                               "(the reference panics on `grad_weight.as_mut().unwrap()`, linear.rs:72)")
        if not self.has_bias:                                   # linear.rs:74-77
            return [Parameter(self.weight, self.grad_weight)]
        return [Parameter(self.weight, self.grad_weight), Parameter(self.bias, self.grad_bias)]


class Sequential(Module):
    """Ordered container (module/sequential.rs:11-110): forward folds left, backward
    folds right, `parameters` concatenates in layer order.

    Fusion is a peephole over adjacent layers and changes no result: a `Linear`
    directly followed by a `ReLU` applies the ReLU in the GEMM epilogue, and the
    `Linear` after that `ReLU` applies the ReLU mask in its dX epilogue.  Layers
    called on their own keep the unfused kernels."""

    def __init__(self, layers: Sequence[Module] = ()):
        self.layers: list[Module] = list(layers)

    # editing API (sequential.rs:24-59)
    def push(self, layer: Module) -> None:
        self.layers.append(layer)

    def insert(self, index: int, layer: Module) -> None:
        if index > len(self.layers):
            raise IndexError(f"insertion index (is {index}) should be <= len (is {len(self.layers)})")
        self.layers.insert(index, layer)

    def remove(self, index: int) -> Module | None:
        return None if index >= len(self.layers) else self.layers.pop(index)

    def __len__(self) -> int:
        return len(self.layers)

    def is_empty(self) -> bool:
        return not self.layers

    @staticmethod
    def _plain(layer: Module, kind: type) -> bool:
        return type(layer) is kind       # subclasses may override forward/backward: do not fuse

    def forward(self, input: Tensor) -> Tensor:
        x = input
        i, n = 0, len(self.layers)
        while i < n:
            layer = self.layers[i]
            if self._plain(layer, Linear) and i + 1 < n and self._plain(self.layers[i + 1], ReLU):
                x = layer._forward(x, fuse_relu=True)
                self.layers[i + 1].prev_input = x     # sign pattern of the pre-activation
                i += 2
            else:
                x = layer.forward(x)
                i += 1
        return x

    def backward(self, gradient: Tensor, need_input_grad: bool = True,
                 on_layer_grads: Callable[[Linear], None] | None = None) -> Tensor | None:
        """`need_input_grad=False` skips dX of the first layer when it is a Linear
        (the reference computes it and its training loop discards it, README.md:72);
        the call then returns None.  `on_layer_grads(layer)` is called as soon as a
        Linear's dW/db are queued (used to start their all-reduce early)."""
        if on_layer_grads is None:
            chain = self._small_linear_chain()
            if chain is not None:
                return self._backward_chain(chain, gradient, need_input_grad)
        g: Tensor | None = gradient
        first_compute = next((k for k, l in enumerate(self.layers) if not self._plain(l, Identity)), None)
        i = len(self.layers) - 1
        while i >= 0:
            layer = self.layers[i]
            if self._plain(layer, Linear):
                fuse = i > 0 and self._plain(self.layers[i - 1], ReLU)
                need = need_input_grad or i != first_compute
                # the gradient goes straight (or through a fused ReLU) into another Linear
                # that will compute its own dX: let this kernel write the transposed copy too
                below = i - 2 if fuse else i - 1
                feeds_linear = (below >= 0 and self._plain(self.layers[below], Linear)
                                and (need_input_grad or below != first_compute))
                g = layer._backward(g, relu_mask=fuse, need_input_grad=need, want_transposed=feeds_linear)
                if on_layer_grads is not None:
                    on_layer_grads(layer)
                if fuse:
                    self.layers[i - 1]._take()        # its mask was applied in the epilogue above
                    i -= 1
                if g is None:
                    return None
            else:
                g = layer.backward(g)
            i -= 1
        return g

    # A whole network of small layers goes through one library call, which runs the
    # dependent dX products first and then all dW/db products in one launch.
    _CHAIN_MAX_WEIGHT_ELEMS = 1 << 20

    def _small_linear_chain(self) -> list[tuple[Linear, ReLU | None]] | None:
        """[(linear, the ReLU in front of it or None), ...] in forward order when the
        container is `Identity*, Linear, (ReLU, Linear)*` of plain layers that are all
        small; None otherwise."""
        layers = list(self.layers)
        while layers and self._plain(layers[0], Identity):
            layers.pop(0)
        if len(layers) < 3 or len(layers) % 2 == 0:
            return None
        chain: list[tuple[Linear, ReLU | None]] = []
        for k, layer in enumerate(layers):
            if k % 2 == 0:
                if (not self._plain(layer, Linear) or not layer.has_bias
                        or layer.input_size * layer.output_size > self._CHAIN_MAX_WEIGHT_ELEMS):
                    return None
                chain.append((layer, layers[k - 1] if k else None))
            elif not self._plain(layer, ReLU):
                return None
        return chain

    def _backward_chain(self, chain, gradient: Tensor, need_input_grad: bool) -> Tensor | None:
        ctx, n = gradient.ctx, len(chain)
        xs = []
        for lin, relu in chain:
            if lin.prev_input is None:
                raise RuntimeError("Linear::backward called without a preceding forward "
                                   "(the reference panics on `prev_input.take().unwrap()`, linear.rs:61)")
            xs.append(lin.prev_input)
        for lin, relu in chain:
            lin.prev_input = None
            if relu is not None:
                relu._take()
            if lin.grad_weight is None or lin.grad_weight.ctx is not ctx:
                lin.grad_weight = ctx.empty(lin.output_size, lin.input_size)
                lin.grad_bias = ctx.empty(1, lin.output_size)
        dxs = [ctx.empty(x.rows, x.cols) if (l > 0 or need_input_grad) else None for l, x in enumerate(xs)]

        def handles(tensors):
            return (C.c_void_p * n)(*[t.handle.value if t is not None else None for t in tensors])

        masks = (C.c_ubyte * n)(*[1 if relu is not None else 0 for _, relu in chain])
        ctx._check(ctx._lib.rst_linear_backward_chain(
            ctx.handle, n, gradient.handle, handles(xs), handles([lin.weight for lin, _ in chain]), masks,
            handles([lin.grad_weight for lin, _ in chain]), handles([lin.grad_bias for lin, _ in chain]),
            handles(dxs)))
        return dxs[0]

    def train(self) -> None:
        for layer in self.layers:
            layer.train()

    def eval(self) -> None:
        for layer in self.layers:
            layer.eval()

    def parameters(self) -> list[Parameter]:
        return [p for layer in self.layers for p in layer.parameters()]

    def to(self, ctx: Context) -> "Sequential":
        for layer in self.layers:
            if hasattr(layer, "to"):
                layer.to(ctx)
        return self


def sequential(*layers: Module | Iterable[Module]) -> Sequential:
    """`sequential!(Identity(), Linear(784, 100), ReLU(), ...)` (sequential.rs:62-74)."""
    if len(layers) == 1 and not isinstance(layers[0], Module):
        layers = tuple(layers[0])
    return Sequential(layers)
