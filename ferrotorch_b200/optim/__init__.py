"""Optimizers, schedulers, gradient scaling.

The reference's ``ferrotorch-optim`` has 18 optimizers, 15 schedulers, ``GradScaler``, a gradient
accumulator, EMA and SWA (ferrotorch-optim/src/*.rs, scheduler/*.rs, grad_scaler.rs:153-376); its
defaults are torch's (adamw.rs:68-79, sgd.rs:44-86).  Everything torch ships is re-exported under
the same names; what torch lacks is implemented in :mod:`.extra` (Muon, Adafactor, K-FAC-style
natural gradient, EMA / SWA helpers, the gradient accumulator, warm-up and cosine-warm-up
schedules); ``FusedAdamW`` / ``FusedSGD`` are torch-API optimizers backed by the flat-arena
kernels (``ft_adamw_flat`` / ``ft_sgd_flat``): one launch per parameter group instead of ~17 per
parameter (adamw.rs:239-384).
"""
from torch.optim import (ASGD, LBFGS, SGD, Adadelta, Adagrad, Adam, Adamax, AdamW, NAdam, Optimizer, RAdam,  # noqa: F401
                         RMSprop, Rprop, SparseAdam)
from torch.optim import lr_scheduler  # noqa: F401
from torch.optim.lr_scheduler import (ChainedScheduler, ConstantLR, CosineAnnealingLR,  # noqa: F401
                                      CosineAnnealingWarmRestarts, CyclicLR, ExponentialLR, LambdaLR, LinearLR,
                                      MultiplicativeLR, MultiStepLR, OneCycleLR, PolynomialLR, ReduceLROnPlateau,
                                      SequentialLR, StepLR)
from torch.optim.swa_utils import SWALR  # noqa: F401

try:  # torch >= 2.3
    from torch.amp import GradScaler  # noqa: F401
except ImportError:  # pragma: no cover
    from torch.cuda.amp import GradScaler  # noqa: F401

from .extra import (EMA, Adafactor, AveragedModel, Kfac, GradientAccumulator, Muon, NaturalGradient, WarmupLR,  # noqa: F401
                    cosine_warmup_scheduler)
from .fused import FusedAdamW, FusedSGD  # noqa: F401


ExponentialMovingAverage = EMA          # noqa: F405  (ferrotorch-optim/src/ema.rs)
from .extra import diff_sgd_momentum_step, diff_sgd_step, elemwise_max, f64_scalar_on, scalar_on  # noqa: F401,E402
from .configs import *  # noqa: F401,F403,E402
from .configs import (ParamGroup, ParamKey, OptimizerState, Sgd, Asgd, Lbfgs, Rmsprop, LrScheduler, SequentialLr,  # noqa: F401,E402
                      MetricScheduler, Swalr, LinearWarmup)
