"""Command-line runner: ``python -m vmoe_b200.train.main --config=<file.py>[:arg]
--workdir=<dir> [--config.key=value ...]``.

Loads ``get_config(arg)`` from the config file, applies dotted overrides, locks the config,
initialises ``torch.distributed`` (one process per GPU under torchrun), builds the
('expert', 'replica') mesh from ``config.num_expert_partitions`` and calls
``main(config, workdir, mesh, writer)`` (reference: ``vmoe/app.py:45-93``).
"""
from __future__ import annotations

import argparse
import ast
import importlib.util
import logging
import os
from typing import Any, Callable, List, Optional

from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.utils import metric_writers
from vmoe_b200.utils.config_dict import ConfigDict, as_config_dict


def load_config(spec: str) -> ConfigDict:
  """``path/to/config.py[:arg]`` -> the (unlocked) ConfigDict returned by ``get_config``."""
  path, _, arg = spec.partition(":")
  if not os.path.exists(path):
    # Allow module paths such as vmoe_b200.configs.vmoe_paper.pretrain_imagenet21k
    mod = importlib.import_module(path)
  else:
    modspec = importlib.util.spec_from_file_location("_vmoe_b200_config", path)
    mod = importlib.util.module_from_spec(modspec)
    modspec.loader.exec_module(mod)
  cfg = mod.get_config(arg) if arg else mod.get_config()
  return as_config_dict(cfg)


def _parse_value(text: str) -> Any:
  try:
    return ast.literal_eval(text)
  except (ValueError, SyntaxError):
    return text


def apply_overrides(config: ConfigDict, overrides: List[str]) -> None:
  for item in overrides:
    key, _, value = item.partition("=")
    with config.ignore_type():
      config[key] = _parse_value(value)


def parse_args(argv: Optional[List[str]] = None):
  ap = argparse.ArgumentParser(allow_abbrev=False)
  ap.add_argument("--workdir", required=True, help="Directory to store logs and model data.")
  ap.add_argument("--config", required=True, help="Config file, optionally 'file.py:arg'.")
  args, rest = ap.parse_known_args(argv)
  overrides = []
  for r in rest:
    if r.startswith("--config."):
      overrides.append(r[len("--config."):])
    else:
      ap.error(f"unknown argument {r}")
  return args, overrides


def run(main: Callable[..., Any], argv: Optional[List[str]] = None):
  args, overrides = parse_args(argv)
  logging.basicConfig(level=logging.INFO,
                      format="%(asctime)s %(levelname)s %(filename)s:%(lineno)d] %(message)s")
  config = load_config(args.config)
  apply_overrides(config, overrides)
  config.lock()
  mesh_lib.init_distributed()
  mesh = mesh_lib.get_auto_logical_mesh(int(config.get("num_expert_partitions", 1) or 1))
  mesh_lib.set_mesh(mesh)
  logging.info("Process %d of %d; config:\n%s", mesh.rank, mesh.world_size, config)
  mesh_lib.log_logical_mesh(mesh)
  logdir = os.path.join(args.workdir, "logs")
  writer = metric_writers.create_default_writer(logdir, just_logging=mesh.rank > 0)
  if mesh.rank == 0:
    os.makedirs(args.workdir, exist_ok=True)
  with mesh_lib.use_mesh(mesh), metric_writers.ensure_flushes(writer):
    return main(config, args.workdir, mesh, writer)
