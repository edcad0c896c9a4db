"""triteia_b200 — B200 (sm_100a) implementation of Triteia's indexed low-precision delta matmul
path behind the reference's Python op API.  Importing the package loads libtriteia_b200.so and
raises if it has not been built: there is no CPU or PyTorch fallback for the CUDA operators."""
from . import _lib  # noqa: F401  (fails loudly when the native library is missing)
from . import ops, capi, nn  # noqa: F401

__version__ = "0.1.0"
