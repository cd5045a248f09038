"""libosmos_b200: sm_100a kernels for libosmos's quantized-weight matrix path, behind the reference's C ABI.

The product is the shared library `libosmos_b200.so` (headers in include/osmos_b200/). This package holds its
sources (csrc/, host/), the build script, and a thin ctypes loader used by the tests and the benchmark. There is no
CPU fallback: loading fails loudly when the library is missing.
"""
from .api import Lib, load  # noqa: F401
