from deca_b200.operators.Softmax import *  # noqa: F401,F403
