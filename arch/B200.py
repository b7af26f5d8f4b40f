from deca_b200.arch.B200 import *  # noqa: F401,F403
from deca_b200.arch.B200 import B200  # noqa: F401
