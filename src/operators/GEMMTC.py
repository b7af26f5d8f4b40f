from deca_b200.operators.GEMMTC import *  # noqa: F401,F403
