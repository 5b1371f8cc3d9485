"""B200-native MoE grouped-GEMM hot path behind cudnn-frontend's Python signatures."""

__version__ = "0.1.0"

from . import _lib  # noqa: F401
