"""Functional options in the reference's style.

The reference configures layers, losses and optimizers with option functions
(``nn.NewConv2d(3, 16, 3, nn.WithPadding(1), nn.WithStride(2))``, ``optim.NewSGD(params, 0.1,
optim.WithMomentum(0.9), optim.WithNesterov(true))``; nn/conv.go:17-75, nn/pool.go:36-84,
optim/sgd.go:14-30 and the other ``XOption`` types).  Here the same settings are keyword
arguments; this module lets code written with option functions run unchanged:

* ``pkg.WithAnything(values...)`` (any name starting with ``With`` that the package does not
  define itself) builds an :class:`Option`;
* the ``NewX`` constructors and the loss functions accept options after their positional
  arguments and turn each into the keyword argument of the same meaning.

An option name is resolved against the callee's signature: a table covers the names that do not
follow the pattern (``WithLayers`` -> ``num_layers``, ``WithNoBias`` -> ``bias=False``,
``WithBeta1`` -> first element of ``betas``), otherwise the CamelCase name is converted to
snake_case and leading family words are dropped until a parameter matches
(``WithAdamWWeightDecay`` -> ``weight_decay``, ``WithPoolStride`` -> ``stride``).  An option
that matches nothing raises ``TypeError`` naming the callee.
"""
from __future__ import annotations

import functools
import inspect
import re
from typing import Callable, Dict, List, Sequence, Tuple


class Option:
    """One functional option: the part of its name after ``With`` and its values."""
    __slots__ = ("name", "args")

    def __init__(self, name: str, args: Tuple):
        self.name, self.args = name, tuple(args)

    def __repr__(self):
        return f"With{self.name}({', '.join(map(repr, self.args))})"


def make_with(name: str) -> Callable[..., Option]:
    """The option function of this name (``name`` starts with ``With``)."""
    def with_(*args) -> Option:
        return Option(name[4:], args)
    with_.__name__ = with_.__qualname__ = name
    return with_


def package_getattr(module_name: str):
    """A module-level ``__getattr__`` that supplies ``WithX`` option functions on demand."""
    def __getattr__(name: str):
        if name.startswith("With") and len(name) > 4 and name[4].isupper():
            return make_with(name)
        raise AttributeError(f"module {module_name!r} has no attribute {name!r}")
    return __getattr__


# names that do not follow the CamelCase -> snake_case pattern: option -> (keyword, fixed value or None)
_FIXED = {
    "NoBias": ("bias", False), "Bidirectional": ("bidirectional", True), "ReLU": ("relu", True),
    "Causal": ("causal", True), "PreNorm": ("pre_norm", True), "PoolCeilMode": ("ceil_mode", True),
    "PerChannelWeights": ("per_channel_weights", True),
}
_RENAMED = {
    "Layers": "num_layers", "Pad": "padding", "Kernel": "kernel_size", "PoolKernel": "kernel_size",
    "FracKernel": "kernel_size", "ASGDLambda": "lambd", "LRNAlpha": "alpha", "LRNBeta": "beta", "LRNK": "k",
    "AdagradLRDecay": "lr_decay", "BagMode": "mode", "BagPaddingIdx": "padding_idx", "BagMaxNorm": "max_norm",
    "FFActivation": "activation", "TransformerDropout": "dropout", "RNNDropout": "dropout", "SpectralEps": "eps",
    "KDim": "kdim", "VDim": "vdim", "RpropStepBounds": "step_sizes", "ClassWeights": "weight",
    "FractionalSamples": "samples", "NormType": "norm_type", "ASGDT0": "t0", "DType": "dtype",
}
# options that set one element of a tuple-valued keyword: option suffix -> (keyword, position)
_ELEMENT = {"Beta1": ("betas", 0), "Beta2": ("betas", 1), "EtaMinus": ("etas", 0), "EtaPlus": ("etas", 1),
            "Eps1": ("eps", 0), "Eps2": ("eps", 1)}


def _snake(words: Sequence[str]) -> str:
    return "_".join(w.lower() for w in words)


def _words(name: str) -> List[str]:
    return re.findall(r"[A-Z]+(?![a-z])|[A-Z][a-z0-9]*|[a-z0-9]+", name)


def _value(args: Tuple):
    if len(args) == 0:
        return True
    return args[0] if len(args) == 1 else tuple(args)


def resolve(callee: Callable, options: Sequence[Option]) -> Dict[str, object]:
    """Keyword arguments of ``callee`` that ``options`` stand for."""
    target = callee.__init__ if inspect.isclass(callee) else callee
    params = inspect.signature(target).parameters
    has_kwargs = any(p.kind == p.VAR_KEYWORD for p in params.values())
    out: Dict[str, object] = {}
    for opt in options:
        if opt.name in _FIXED and _FIXED[opt.name][0] in params:
            k, v = _FIXED[opt.name]
            out[k] = v
            continue
        if opt.name in _RENAMED and _RENAMED[opt.name] in params:
            out[_RENAMED[opt.name]] = _value(opt.args)
            continue
        words = _words(opt.name)
        done = False
        for suffix, (key, pos) in _ELEMENT.items():
            if opt.name.endswith(suffix) and key in params and isinstance(params[key].default, (tuple, list)):
                cur = list(out.get(key, params[key].default))
                cur[pos] = opt.args[0]
                out[key] = tuple(cur)
                done = True
                break
        if done:
            continue
        for start in range(len(words)):
            cand = _snake(words[start:])
            if cand in params:
                out[cand] = _value(opt.args)
                done = True
                break
        if not done and has_kwargs:
            out[_snake(words)] = _value(opt.args)
            done = True
        if not done:
            raise TypeError(f"{getattr(callee, '__name__', callee)}: no argument matches option {opt!r}")
    return out


def accepting_options(callee: Callable) -> Callable:
    """Wraps a class or function so that :class:`Option` objects among its positional arguments
    become keyword arguments.  The wrapped object is available as ``__wrapped__``."""
    @functools.wraps(callee, updated=())
    def call(*args, **kwargs):
        opts = [a for a in args if isinstance(a, Option)]
        if opts:
            args = [a for a in args if not isinstance(a, Option)]
            target = callee.__init__ if inspect.isclass(callee) else callee
            names = [n for n, p in inspect.signature(target).parameters.items()
                     if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
            if inspect.isclass(callee):
                names = names[1:]                       # self
            for k, v in resolve(callee, opts).items():
                if k in names and names.index(k) < len(args):
                    args[names.index(k)] = v            # an option overrides the positional value
                else:
                    kwargs.setdefault(k, v)
        return callee(*args, **kwargs)
    call.__wrapped__ = callee
    return call
