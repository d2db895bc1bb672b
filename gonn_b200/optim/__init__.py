"""Optimizers, gradient clipping, vector utilities and LR schedulers."""
from .base import Group, Optimizer, State, as_groups  # noqa
from .fused import SGD, Adam, AdamW, Lion, LAMB  # noqa
from .more import (RMSprop, Adagrad, Adadelta, NAdam, Adamax, RAdam, Rprop, Adafactor, ASGD, SparseAdam,  # noqa
                   LBFGS)
from .clip import (ClipGradNorm, TotalGradNorm, ClipGradsWithNorm, ClipGradValue, ParametersToVector,  # noqa
                   VectorToParameters, GradsToVector)
from .scheduler import (Scheduler, StepLR, MultiStepLR, ExponentialLR, CosineAnnealingLR, LinearLR,  # noqa
                        ReduceLROnPlateau, PolynomialLR, ChainedScheduler, SequentialLR, CyclicLR, OneCycleLR)


def _groups_ctor(cls):
    def make(groups, **kw):
        """Constructor over explicit ``Group`` lists; optimizer defaults are NOT injected."""
        return cls(groups, **kw)
    make.__name__ = "New" + cls.__name__ + "Groups"
    return make


for _c in (SGD, Adam, AdamW, Lion, LAMB, RMSprop, Adagrad, Adadelta, NAdam, Adamax, RAdam, Rprop, Adafactor, ASGD,
           SparseAdam):
    globals()["New" + _c.__name__ + "Groups"] = _groups_ctor(_c)
