"""``from ferrotorch_b200.prelude import *`` -- the working set of the reference's prelude
(ferrotorch/src/lib.rs:61-70): the flat tensor API, the common layers, losses, activations,
recurrent layers and optimizers."""
from torch import Tensor, arange, cat, eye, full, linspace, ones, ones_like, rand, randn, stack, tensor, zeros, zeros_like  # noqa: F401
from torch.nn import Module, Parameter  # noqa: F401

from .autograd import backward, enable_grad, grad, no_grad  # noqa: F401
from .core import Device, MemoryFormat  # noqa: F401
from .nn import (GELU, GRU, LSTM, BatchNorm2d, Conv2d, CrossEntropyLoss, Dropout, LayerNorm, Linear, MSELoss, ReLU,  # noqa: F401
                 Sequential, Sigmoid, SiLU, Softmax, Tanh)
from .optim import Adam, AdamW, Optimizer, Sgd  # noqa: F401
from .tensor_ops import DType, FerrotorchError, from_slice, from_vec, mean_dim, scalar, sum_dim  # noqa: F401

__all__ = [n for n in dir() if not n.startswith("_")]
