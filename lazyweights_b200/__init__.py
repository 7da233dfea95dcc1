"""lazyweights_b200: Huffman-coded llama.cpp block weights decoded on B200 GPUs, fused with dequantisation and
the matrix-vector product.  The compute path lives in liblwb200.so (CUDA, sm_100a); see include/lwb200.h."""
from . import bundle  # noqa: F401
from ._native import LwError, lib  # noqa: F401
from .runtime import Bundle, CodedMatrix, ProductBatch  # noqa: F401
