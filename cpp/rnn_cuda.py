"""Drop-in for the reference module of the same path (cpp/rnn_cuda.py): exports fwd_cuda and bwd_cuda."""
from rnn_train_ring_attractor_b200.rnn_cuda import fwd_cuda, bwd_cuda  # noqa: F401
