from deca_b200.operators.Rowwise import *  # noqa: F401,F403
