"""``from operators.RMSNorm import RMSNorm`` (the reference's module path); the class lives with its
row-wise siblings in ``Rowwise.py``."""

from .Rowwise import RMSNorm  # noqa: F401
