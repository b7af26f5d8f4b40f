from deca_b200.cost_model.CostModel import *  # noqa: F401,F403
