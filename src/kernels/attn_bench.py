from deca_b200.kernels.attn_bench import *  # noqa: F401,F403
