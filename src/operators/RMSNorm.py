from deca_b200.operators.RMSNorm import *  # noqa: F401,F403
