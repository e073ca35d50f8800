"""Import shim: lets `from cpp.ring_rnn_cuda import *` in the reference's training script resolve to this
repository's operator when this repository precedes the reference checkout on sys.path."""
