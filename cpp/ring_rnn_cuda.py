"""Drop-in for the reference module of the same path (cpp/ring_rnn_cuda.py).  No __all__: the
reference's training script relies on `torch` leaking through the star import."""
import torch  # noqa: F401
from torch.autograd import Function  # noqa: F401

from rnn_train_ring_attractor_b200.rnn_cuda import fwd_cuda, bwd_cuda  # noqa: F401
from rnn_train_ring_attractor_b200.ring_rnn_cuda import (  # noqa: F401
    RingRnnCudaFunc,
    get_precision,
    ring_rnn_cuda_func,
    set_precision,
)
