"""Layers.  Everything in :mod:`torch.nn` is re-exported under the same names (the reference's
``ferrotorch-nn`` mirrors that surface: activations, convolutions, norms, pools, RNNs,
transformer blocks, losses, containers, init), and the layers that have a native sm_100a
kernel are replaced by the versions in :mod:`ferrotorch_b200.nn.layers`."""
from torch.nn import *  # noqa: F401,F403
from torch.nn import functional, init, utils  # noqa: F401

from .layers import (FusedLinearActivation, GQAAttention, KVCache, Linear, RMSNorm,  # noqa: F401
                     RotaryPositionEmbedding, SwiGLU, clip_grad_norm_, clip_grad_value_, repeat_kv,
                     scaled_dot_product_attention)

from ..ops.batchnorm import BatchNormAct2d, batch_norm_act  # noqa: F401,E402
from .fake_quant import FakeQuantize, MinMaxObserver, MovingAverageObserver, QatLinear, prepare_qat  # noqa: F401,E402
from .extra import (HookedModule, HookHandle, LoRALinear, SqueezeExcitation, flash_attention,  # noqa: F401,E402
                    standard_attention)
from ..core import BlockMask, flex_attention  # noqa: F401,E402
from .paged import OutOfPages, PagedAttentionManager, PagedKVCache  # noqa: F401,E402
from ..ops.conv import IgemmConv2d, convert_convs  # noqa: F401,E402  (implicit-GEMM convolution; opt-in, see ops.conv)
from ..ops.pool import MaxPool2d as NhwcMaxPool2d  # noqa: F401,E402
from .compat import *  # noqa: F401,F403,E402
from .compat import (BackwardHook, ForwardHook, ForwardPreHook, HardSigmoid, HardSwish, KVPage, StateDict)  # noqa: F401,E402
