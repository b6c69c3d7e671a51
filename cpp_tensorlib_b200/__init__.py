"""B200 (sm_100a) implementation of cpp-tensorlib's quantized-decode hot path.

The product is the C-ABI library ``libtlb200.so`` (``include/tlb200.h``);
``cpp_tensorlib_b200.cuda`` mirrors the reference's ``tl::cuda::`` operator
interface on top of it for Python callers, with torch used only to own device
memory and streams.
"""
from ._lib import TlbError, lib, check  # noqa: F401
