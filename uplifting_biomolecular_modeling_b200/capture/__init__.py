"""Launch-bound loops: CUDA-graph capture keyed by argument signature, capture policies, step-invariant hoisting."""
from .graphs import GraphCache  # noqa: F401
from .hoist import ConstMemo  # noqa: F401
