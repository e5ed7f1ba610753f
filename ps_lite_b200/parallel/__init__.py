"""Device data plane objects: symmetric heap, dense and sparse tables, schedulers."""
from .heap import SymmetricHeap, tensor_from_ptr  # noqa: F401
from .dense import DenseTable, ServerOptimizer  # noqa: F401
from .sparse import SparseTable  # noqa: F401
