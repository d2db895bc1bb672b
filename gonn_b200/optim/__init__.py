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
    def make(groups, *opts, **kw):
        """Constructor over explicit ``Group`` lists; optimizer defaults are NOT injected.
        Functional options (``optim.WithBeta2(0.95)``) are accepted after the groups."""
        from ..options import Option, resolve
        bad = [o for o in opts if not isinstance(o, Option)]
        if bad:
            raise TypeError(f"{make.__name__}: unexpected positional arguments {bad}")
        for k, v in resolve(cls, opts).items():
            kw.setdefault(k, v)
        return cls(groups, **kw)
    make.__name__ = "New" + cls.__name__ + "Groups"
    return make


for _c in (SGD, Adam, AdamW, Lion, LAMB, RMSprop, Adagrad, Adadelta, NAdam, Adamax, RAdam, Rprop, Adafactor, ASGD,
           SparseAdam):
    globals()["New" + _c.__name__ + "Groups"] = _groups_ctor(_c)


class MetricScheduler:
    """A scheduler stepped with a metric, ``Step(metric)`` (optim/scheduler.go:13-15):
    ``ReduceLROnPlateau`` is the one implementation."""

    def Step(self, metric: float) -> None:
        raise NotImplementedError


def _constructor_aliases(ns) -> None:
    """``NewX`` for every public class ``X`` (the reference's constructor functions)."""
    for name, obj in list(ns.items()):
        if isinstance(obj, type) and name[0].isupper() and "New" + name not in ns:
            ns["New" + name] = _accepting_options(obj)


from ..options import accepting_options as _accepting_options, package_getattr as _package_getattr  # noqa: E402

_constructor_aliases(globals())
__getattr__ = _package_getattr(__name__)     # optim.WithMomentum(0.9), optim.WithNesterov(True), ...
