from deca_b200.kernels.gemm_bench import *  # noqa: F401,F403
