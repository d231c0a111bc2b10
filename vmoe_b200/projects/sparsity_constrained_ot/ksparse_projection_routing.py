"""k-sparse projection routers: semi-dual OT whose plan has at most k non-zeros per token
(tokens choose) or at most C per expert (experts choose)
(``vmoe/projects/sparsity_constrained_ot/ksparse_projection_routing.py:35-239``). The
implementation lives in ``ot_routing``."""
from vmoe_b200.projects.sparsity_constrained_ot.ot_routing import (  # noqa: F401
    KSparseProjectionTransportTopExpertsPerItemRouter,
    KSparseProjectionTransportTopItemsPerExpertRouter, projection_sparse_simplex,
    regularized_semi_dual_plan)
