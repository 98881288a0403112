"""gorgonia_b200: sm_100a execution engine for gorgonia's tape VM.

The product is libgorgonia_b200.so (C ABI in include/gorgonia_b200.h). This package holds its
sources (csrc/) and a thin host-side mirror of gorgonia's engine interface used by the
tests and the benchmark. Importing it fails if the library has not been built.
"""
from ._lib import B200Error, lib, LIB_PATH  # noqa: F401
from .engine import Engine, Tensor  # noqa: F401
