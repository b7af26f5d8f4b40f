from deca_b200.kernels.rowwise_b200 import *  # noqa: F401,F403
