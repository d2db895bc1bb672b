"""gonn_b200: a Blackwell (sm_100a) deep-learning framework with GoNN's capabilities.

PyTorch provides storage, streams and the autograd tape; the hot operators are
hand-written CUDA kernels in ``csrc/`` reached through ``gonn_b200.lib``.
"""
__version__ = "0.1.0"
