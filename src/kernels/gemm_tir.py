from deca_b200.kernels.gemm_b200 import *  # noqa: F401,F403
