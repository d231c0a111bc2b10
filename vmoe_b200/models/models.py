"""All classification models by name (``vmoe/nn/models.py``)."""
from vmoe_b200.models.external import MlpMixer  # noqa: F401
from vmoe_b200.models.external import VisionTransformer  # noqa: F401
from vmoe_b200.models.vit_moe import VisionTransformerMoe  # noqa: F401
from vmoe_b200.models.vit_moe_ensemble import VisionTransformerMoeEnsemble  # noqa: F401
