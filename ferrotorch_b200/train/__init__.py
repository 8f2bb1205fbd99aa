"""Training: the flat-arena engine, the Learner loop, callbacks, metrics, TensorBoard output."""
from .engine import FlatArena, FlatTrainer  # noqa: F401
from .learner import (AccuracyMetric, AmpContext, Callback, EarlyStopping, EMACallback, EpochResult, EvalResult, Learner,  # noqa: F401
                      LossFn, LossMetric, Metric, ProgressLogger, RunningAverage, TensorBoardCallback, TopKAccuracy,
                      TrainingHistory, checkpoint_sequential)
from .metrics_log import MetricsCallback, MetricsLogger, Report, StepTimer, read_metrics  # noqa: F401
from .tensorboard import TensorBoardWriter  # noqa: F401
from ..autograd import checkpoint  # noqa: F401,E402
from ..nn.layers import clip_grad_norm_, clip_grad_value_  # noqa: F401,E402

EmaCallback = EMACallback
