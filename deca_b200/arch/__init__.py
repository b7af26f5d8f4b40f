from .Arch import Arch
from .B200 import B200

__all__ = ["Arch", "B200"]
