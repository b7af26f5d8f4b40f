from deca_b200.utils.helper import *  # noqa: F401,F403
from deca_b200.utils.helper import GPUDetector, byte_size  # noqa: F401
