"""Root of the operator records (the role of the reference's src/operators/Op.py): an operator has
a ``name`` and is called with its input tensors to run its kernel."""

import abc


class Operator(abc.ABC):
    def __init__(self, name: str):
        self.name = name

    @abc.abstractmethod
    def __call__(self, *args, **kwargs):
        """Runs the operator's kernel on the given tensors."""
