from .symm import SymmetricHeap  # noqa: F401
