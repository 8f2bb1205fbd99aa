"""Training: the flat-arena engine, the Learner loop, callbacks, metrics, TensorBoard output."""
from .engine import FlatArena, FlatTrainer  # noqa: F401
from .learner import (AccuracyMetric, AmpContext, Callback, EarlyStopping, EMACallback, EpochResult, Learner,  # noqa: F401
                      LossMetric, Metric, ProgressLogger, RunningAverage, TensorBoardCallback, TopKAccuracy,
                      TrainingHistory, checkpoint_sequential)
from .tensorboard import TensorBoardWriter  # noqa: F401
