from deca_b200.kernels.rowwise_bench import *  # noqa: F401,F403
