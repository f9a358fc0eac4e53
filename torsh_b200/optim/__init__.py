"""Optimizers, LR schedulers and mixed-precision helpers."""
from . import lr_scheduler
from .extra import (ASGD, FTRL, LARS, LBFGS, AccumulatingOptimizer, AdaBelief, AdaBound, Adadelta, Adagrad, Adamax,
                    GradientAccumulator, Lion, Lookahead, NAdam, Prodigy, RAdam, Ranger, RMSprop, Rprop,
                    ScheduleFreeSGD, SophiaG, SparseAdam, Yogi)
from .flat import FlatAdamW, FlatParameters
from .fused import LAMB, SGD, Adam, AdamW
