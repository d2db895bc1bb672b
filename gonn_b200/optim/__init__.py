"""Optimizers, gradient clipping, vector utilities and LR schedulers."""
from .base import Group, Optimizer, State, as_groups  # noqa
from .fused import SGD, Adam, AdamW, Lion, LAMB  # noqa
