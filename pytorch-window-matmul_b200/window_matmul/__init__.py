"""Drop-in for the reference package `window_matmul` (window_matmul/__init__.py:1-4) on B200."""
import torch  # noqa: F401

from .softmax import window_softmax
from .window_matmul import unwindow_matmul, window_matmul

__all__ = ["window_matmul", "unwindow_matmul", "window_softmax"]
