"""Quadratically regularised OT router (sparse plan without an explicit sparsity constraint)
(``vmoe/projects/sparsity_constrained_ot/sparse_projection_routing.py:35-124``). The
implementation lives in ``ot_routing``."""
from vmoe_b200.projects.sparsity_constrained_ot.ot_routing import (  # noqa: F401
    SparseProjectionTransportTopItemsPerExpertRouter, projection_simplex,
    regularized_semi_dual_plan)
