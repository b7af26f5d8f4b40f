from deca_b200.Solver import *  # noqa: F401,F403
