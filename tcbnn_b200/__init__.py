"""B200-native binarised-network inference hot path (bit packing, 1-bit GEMM, 1-bit conv with
fused threshold / pool / residual / repack) behind a C ABI; this package is the thin Python
host side used by the tests and the benchmark."""
from . import lib  # noqa: F401

__all__ = ["lib"]
