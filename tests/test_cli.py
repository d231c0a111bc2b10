"""The training CLI end to end on CPU: config file, ``--config.x.y=v`` overrides, workdir."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CONFIG = '''
from vmoe_b200.configs.vmoe_paper import common
from vmoe_b200.utils.config_dict import ConfigDict


def get_config():
  config = common.get_base_config()
  pp = 'value_range(-1,1)|onehot(10, inkey="label", outkey="labels")|keep("image", "labels")'
  config.dataset = ConfigDict(type_safe=False)
  for variant, split in (("train", "train"), ("val", "validation[:16]")):
    d = common.get_data_config(name="synthetic", split=split, batch_size=8, process=pp)
    d.image_size, d.num_classes = 32, 10
    setattr(config.dataset, variant, d)
  config.train_steps = 5
  config.loss = ConfigDict({"name": "softmax_xent"})
  config.optimizer = common.get_optimizer_config("ViT-S/32, E=8, K=2, Last 2")
  config.model = common.get_vmoe_config("ViT-S/32, E=8, K=2, Last 2", 32, 10)
  config.model.encoder.num_layers = 2
  config.model.encoder.moe.layers = (1,)
  config.model.encoder.moe.group_size = 8
  config.evaluate.every_steps = 2
  config.save_checkpoint.every_steps = 2
  config.extra_rng_keys = ("dropout", "gating")
  return config
'''


def test_train_main_with_config_file_and_overrides(tmp_path):
  cfg = tmp_path / "cfg.py"
  cfg.write_text(CONFIG)
  workdir = tmp_path / "run"
  env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
  res = subprocess.run(
      [sys.executable, "-m", "vmoe_b200.train.main", f"--config={cfg}", f"--workdir={workdir}",
       "--config.train_steps=2", "--config.optimizer.learning_rate.peak_value=0.001"],
      cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
  assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
  files = os.listdir(workdir / "ckpt")
  assert any(f.startswith("ckpt_2.index") for f in files), files  # the override took effect
  assert "val/prec@1" in res.stderr or "val/prec@1" in res.stdout


def test_bench_reference_arm_prints_one_json_line():
  import json
  import subprocess
  import sys
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference",
                        "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=300, cwd=root)
  assert out.returncode == 0, out.stderr[-2000:]
  lines = [l for l in out.stdout.splitlines() if l.strip()]
  assert len(lines) == 1
  record = json.loads(lines[0])
  assert record["impl"] == "reference"
  assert "unavailable" in record and "\n" not in record["unavailable"]


def test_bench_help_lists_the_contract_flags():
  import subprocess
  import sys
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--help"],
                       capture_output=True, text=True, timeout=120, cwd=root)
  assert out.returncode == 0
  for flag in ("--gpus", "--steps", "--warmup", "--impl", "--mode", "--ensemble-size"):
    assert flag in out.stdout


def test_reference_arm_plumbing_with_fake_modules(monkeypatch, capsys):
  """``bench.py --impl reference``: without JAX it prints the ``unavailable`` line; with the
  reference's dependencies importable (faked here) it hands the benchmark's arguments to
  ``baseline/run_reference.py`` and prints the benchmark's JSON schema with its result."""
  import importlib
  import json
  import sys as _sys
  import types
  _sys.path.insert(0, ROOT)
  bench = importlib.import_module("bench")
  args = types.SimpleNamespace(gpus=2, steps=7, warmup=3, per_gpu_batch=64, model=bench.MODEL_DESC)
  monkeypatch.delenv("RANK", raising=False)
  for name in ("jax", "flax", "optax"):
    monkeypatch.setitem(_sys.modules, name, None)     # import raises ImportError
  assert bench.reference_arm(args) == 0
  line = json.loads(capsys.readouterr().out.strip())
  assert line["impl"] == "reference" and "not installed" in line["unavailable"]

  for name in ("jax", "flax", "optax", "vmoe"):
    monkeypatch.setitem(_sys.modules, name, types.ModuleType(name))
  seen = {}

  def fake_run(**kw):
    seen.update(kw)
    return {"ms_per_step": 50.0, "value": kw["per_gpu_batch"] * kw["gpus"] / 0.05,
            "final_loss": 1.0, "global_batch": kw["per_gpu_batch"] * kw["gpus"],
            "num_partitions": 2,
            "e2e": {"value": 2000.0, "unit": "images/s", "ms_per_step": 64.0,
                    "h2d_bytes_per_step": 123, "d2h_bytes_per_step": 4, "last_loss": 1.0}}

  from baseline import run_reference
  monkeypatch.setattr(run_reference, "run", fake_run)
  assert bench.reference_arm(args) == 0
  line = json.loads(capsys.readouterr().out.strip())
  assert seen == dict(gpus=2, steps=7, warmup=3, per_gpu_batch=64, description=bench.MODEL_DESC,
                      num_classes=21843, image_size=224)
  assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["steps"] == 7
  assert line["value"] == 2560.0 and line["e2e"]["h2d_bytes_per_step"] == 123
  assert line["config"]["global_batch"] == 128 and line["metric"] == "V-MoE B/16 train images/s"
  # other ranks stay silent: JAX drives every local GPU from one process
  monkeypatch.setenv("RANK", "1")
  assert bench.reference_arm(args) == 0 and capsys.readouterr().out == ""
