"""Model definitions used by the examples and benchmarks."""
from .mlp import MLP  # noqa: F401
from .lm import TransformerLM, GPT, GPTBlock  # noqa: F401
