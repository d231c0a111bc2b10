"""Training script of the Soft MoE contrastive (two-tower) experiments:
``python -m vmoe_b200.projects.soft_moe.main_contrastive --config=<file> --workdir=<dir>``
(``vmoe/projects/soft_moe/main_contrastive.py``)."""
from vmoe_b200 import app
from vmoe_b200.projects.contrastive import trainer
from vmoe_b200.projects.soft_moe import router  # noqa: F401  (registers SoftRouter)

if __name__ == "__main__":
  app.run(trainer.train_and_evaluate)
