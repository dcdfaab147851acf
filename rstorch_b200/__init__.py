"""rstorch_b200: the f64 training step of the `rstorch` crate on B200 GPUs.

Host-side mirror of the crate's API for that path (same names and call order as
its README loop) over a C-ABI library of sm_100a kernels:

    model = sequential(Identity(), Linear(784, 100), ReLU(), Linear(100, 100), ReLU(), Linear(100, 10))
    loss, optim = CrossEntropyLoss(), SGD.new(0.01)
    for x, y in data_loader.iter_array():
        pred = model.forward(x)
        l = loss.forward(pred, y)
        acc = accuracy(pred, y)          # or loss.last_accuracy, computed by the same kernel
        model.backward(loss.backward())
        optim.step(model)
"""
from ._lib import RstError, exported_symbols
from .core import Context, Graph, Tensor, Timer
from .data import ArrayDataset, DataLoader, DeviceDataset, SequentialSampler
from .loss import CrossEntropyLoss, Loss
from .model import BasicModel
from .module import (Identity, InitParameters, KaimingNormal, Linear, Module, Normal, Parameter, ReLU,
                     Sequential, Softmax, XavierNormal, sequential)
from .optim import SGD, Optimizer
from .parallel import Communicator, backward_with_exchange, shard_rows
from .utils import accuracy, argmax, one_hot

__all__ = [
    "RstError", "exported_symbols", "Context", "Graph", "Tensor", "Timer", "ArrayDataset", "DataLoader",
    "DeviceDataset",
    "SequentialSampler", "CrossEntropyLoss", "Loss", "Identity", "InitParameters", "KaimingNormal",
    "Linear", "Module", "Normal", "Parameter", "ReLU", "Sequential", "Softmax", "XavierNormal", "sequential",
    "SGD", "Optimizer", "BasicModel",
    "Communicator", "backward_with_exchange", "shard_rows", "accuracy", "argmax", "one_hot",
]
