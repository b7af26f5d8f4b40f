from deca_b200.operators import *  # noqa: F401,F403
from deca_b200.operators import __all__  # noqa: F401
