"""Names shared across the code base (``vmoe/constants.py``)."""


class FlaxCollection:
  """Names of the variable collections of the reference checkpoints' layout."""
  PARAMS: str = "params"
  INTERMEDIATES: str = "intermediates"
  PROBES: str = "probes"
  AUX_LOSS: str = "aux_loss"
