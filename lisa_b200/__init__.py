"""B200 (sm_100a) quantized-weight matmul path of the LISA engine.

``lisa_b200.ops`` mirrors the reference's operator API over the C ABI of
``lisa_b200/lib/liblisa_cuda.so`` (hand-written CUDA, no torch inside); build it with
``python -m lisa_b200.build``.
"""
from ._cabi import LisaError, LIB_PATH  # noqa: F401
from . import ops, quant  # noqa: F401
