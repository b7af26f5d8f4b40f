from deca_b200.operators.FlashAttention import *  # noqa: F401,F403
