"""bonsai_vk_b200 - B200-native device layer for the bonsai-vk decode path.

The product is libbonsai_cuda.so (hand-written sm_100a kernels behind the C ABI declared in
include/bonsai_cuda.h). This package holds the ctypes binding used by the tests and the benchmark,
and the host-side data-format helpers. There is no CPU fallback: loading fails loudly when the
library is missing, and creating a context fails loudly without a B200.
"""
from .lib import Context, Buffer, Model, BonsaiError, load_library, LIB_PATH  # noqa: F401
