"""glq_b200 — B200 (sm_100a) kernels for GLQ's compressed-weight matmul, behind the reference's
operator names.  Host side is Python/PyTorch (device memory, streams); all compute is in
libglq_b200.so, reached through a plain C ABI."""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
__version__ = "0.1"
