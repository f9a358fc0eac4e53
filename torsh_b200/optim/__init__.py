"""Optimizers, LR schedulers and mixed-precision helpers."""
from . import lr_scheduler
from .extra import (ASGD, FTRL, LARS, LBFGS, AccumulatingOptimizer, AdaBelief, AdaBound, Adadelta, Adagrad, Adamax,
                    GradientAccumulator, Lion, Lookahead, NAdam, Prodigy, RAdam, Ranger, RMSprop, Rprop,
                    ScheduleFreeSGD, SophiaG, SparseAdam, Yogi)
from .flat import FlatAdamW, FlatParameters
from .fused import LAMB, SGD, Adam, AdamW
from . import advanced, checkpointing, distributed, gradient_free, mixed_precision, second_order
from .gradient_free import BayesianOptimizer, EvolutionStrategy, NelderMead, RandomSearch
from .distributed import AsyncSGD, DistributedOptimizer, ElasticAveragingSGD
from .mixed_precision import (AutocastModel, BF16Config, BF16Trainer, DynamicLossScaler, GradScaler, MixedPrecisionConfig,
                              MixedPrecisionOptimizer, MixedPrecisionTrainer)
from .second_order import KFAC, AdaHessian, NaturalGradient, NewtonCG, Shampoo, TrustRegion, YellowFin
from .more import (AdaDelta, AdaGrad, AdaMax, AdvancedAdam, Branin, CarbonConsciousOptimizer, CheckpointingOptimizer, CMAES, ConvergenceTracker, GaussianProcess,  # noqa: E402,F401
                   LowPrecisionOptimizer, OpenAIES, OptimizerBenchmarks, OptimizerBuilder, OptimizerStressTester, ParamGroupBuilder, ParticleSwarmOptimizer, PowerCappedOptimizer, Rastrigin,
                   Rosenbrock, ScheduleFreeAdamW, Sophia, Sphere, TaskMatcher, TemporalCreditOptimizer)
