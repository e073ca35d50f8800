"""B200-native ring-attractor recurrent forward / backward-through-time operator.

`ring_rnn_cuda`  -- the reference's autograd surface (cpp/ring_rnn_cuda.py) on libringrnn.so
`rnn_cuda`       -- the reference's raw fwd/bwd extension objects (cpp/rnn_cuda.py)
`fused`          -- loss-fused surface that never materialises the [T,B,N] history in fp32
`dp`             -- data-parallel training step (batch sharded, one gradient all-reduce)
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
