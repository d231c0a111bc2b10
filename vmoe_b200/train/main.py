"""Entry point: ``python -m vmoe_b200.train.main --config=... --workdir=...``."""
from vmoe_b200 import app
from vmoe_b200.train import trainer

if __name__ == "__main__":
  app.run(trainer.train_and_evaluate)
