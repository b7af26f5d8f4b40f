"""``from operators.Softmax import Softmax`` (the reference's module path); the class lives with its
row-wise siblings in ``Rowwise.py``."""

from .Rowwise import Softmax  # noqa: F401
