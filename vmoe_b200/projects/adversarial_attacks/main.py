"""CLI of the PGD attack: ``python -m vmoe_b200.projects.adversarial_attacks.main
--config=<file> --workdir=<dir>`` (``vmoe/projects/adversarial_attacks/main.py``)."""
from vmoe_b200 import app
from vmoe_b200.projects.adversarial_attacks import lib

if __name__ == "__main__":
  app.run(lib.run_pgd_attack)
