"""triteia_b200 — B200 (sm_100a) implementation of Triteia's indexed low-precision delta matmul
path behind the reference's Python op API.

Sub-packages (`ops`, `capi`, `nn`, `triteia_cuda`, `sharded`) load on first use.  Any of them loads
libtriteia_b200.so and raises if it has not been built (`python -m triteia_b200.build`): there is no
CPU or PyTorch fallback for the CUDA operators.
"""
import importlib

__version__ = "0.1.0"
_LAZY = ("ops", "capi", "nn", "triteia_cuda", "sharded", "stack", "converters", "configs", "utils", "_lib", "build")


def __getattr__(name):
    if name in _LAZY:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
