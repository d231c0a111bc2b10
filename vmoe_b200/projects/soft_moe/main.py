"""Training script of the Soft MoE classification experiments:
``python -m vmoe_b200.projects.soft_moe.main --config=<file> --workdir=<dir>``
(``vmoe/projects/soft_moe/main.py``)."""
from vmoe_b200 import app
from vmoe_b200.projects.soft_moe import router  # noqa: F401  (registers SoftRouter)
from vmoe_b200.train import trainer

if __name__ == "__main__":
  app.run(trainer.train_and_evaluate)
