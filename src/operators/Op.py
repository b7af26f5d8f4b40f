from deca_b200.operators.Op import *  # noqa: F401,F403
