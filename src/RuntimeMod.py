from deca_b200.RuntimeMod import *  # noqa: F401,F403
from deca_b200.RuntimeMod import RuntimeMod  # noqa: F401
