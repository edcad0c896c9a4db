from .linear import sparse_low_precision_linear
