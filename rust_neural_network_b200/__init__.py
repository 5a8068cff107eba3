"""B200-native neural-network framework with the capabilities of rust-nn 2.1.0.

PyTorch is the tensor/autograd layer; every hot op is a hand-written sm_100a CUDA kernel
(tcgen05 + TMEM + TMA) loaded from ``lib/libb200nn_cuda.so``; the host runtime (checkpoint
format, tokenizer, parsers, tiered store) is C++ in ``lib/libb200nn_host.so``.
"""
VERSION = "2.1.0-b200"
__version__ = VERSION

from . import _native  # noqa: F401
