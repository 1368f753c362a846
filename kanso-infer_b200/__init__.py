"""B200 (sm_100a) `cuda` backend for kanso-infer's quantized hot path.

The product is the C-ABI shared library built from csrc/ (see include/kanso_cuda.h);
`backend` binds it with ctypes for tests and measurement, `build` compiles it.
"""
from . import backend, build, sharded  # noqa: F401

__all__ = ["backend", "build", "sharded"]
