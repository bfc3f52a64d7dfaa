"""Drop-in Linear wrappers over the packed decode kernels."""
from .hybrid_int2 import HybridInfo, HybridInt2Linear
from .hybrid_int4 import HybridInt4Linear

__all__ = ["HybridInfo", "HybridInt2Linear", "HybridInt4Linear"]
