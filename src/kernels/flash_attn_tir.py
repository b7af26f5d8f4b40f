from deca_b200.kernels.flash_attn_b200 import *  # noqa: F401,F403
