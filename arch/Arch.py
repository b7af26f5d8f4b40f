from deca_b200.arch.Arch import *  # noqa: F401,F403
from deca_b200.arch.Arch import Arch  # noqa: F401
