"""KL-projection (entropic OT) routers: the logits are turned into a transport plan whose rows
sum to 1 and whose columns sum to S/E, with Sinkhorn iterations or an L-BFGS solve of the
dual, then dispatched with Top-K / Top-C (``vmoe/projects/sparsity_constrained_ot/
kl_projection_routing.py:35-250``). The implementation lives in ``ot_routing``."""
from vmoe_b200.projects.sparsity_constrained_ot.ot_routing import (  # noqa: F401
    KLProjectionNoisyTopExpertsPerItemRouter, KLProjectionNoisyTopItemsPerExpertRouter,
    kl_projection_lbfgs_plan, sinkhorn_plan)
