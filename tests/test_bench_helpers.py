"""Host-side helpers of bench.py: synthetic labels and the clock sampler's parsing, with a
fake in place of nvidia-smi."""
import importlib.util
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
  spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  return mod


class _FakeProc:

  def __init__(self, text):
    self.text = text

  def terminate(self):
    pass

  def communicate(self, timeout=None):
    return self.text, ""


def test_labels_have_one_to_three_positives():
  bench = _bench()
  labels = bench.make_labels(torch, 64, 1000, torch.Generator().manual_seed(0))
  assert labels.shape == (64, 1000) and labels.dtype == torch.float32
  counts = labels.sum(dim=1)
  assert int(counts.min()) >= 1 and int(counts.max()) <= 3
  assert set(labels.unique().tolist()) == {0.0, 1.0}


def test_clock_sampler_reports_median_clock_and_throttle_reasons():
  bench = _bench()
  sampler = bench.ClockSampler(0)
  sampler.proc = _FakeProc(
      "0, 1700, 1965, 950.1, 0x4, Not Active, Not Active, Not Active, Active\n"
      "0, 1650, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active\n"
      "0, 1965, 1965, 300.0, 0x0, Not Active, Not Active, Not Active, Not Active\n"
      "garbage line\n")
  out = sampler.stop()
  assert out["sm_mhz"] == 1700.0 and out["sm_max_mhz"] == 1965.0
  assert out["reasons"] == ["sw_power_cap"] and out["samples"] == 3


def test_clock_sampler_flags_thermal_slowdown_and_missing_tool():
  bench = _bench()
  sampler = bench.ClockSampler(0)
  sampler.proc = _FakeProc("0, 1200, 1965, 700.0, 0x8, Active, Active, Not Active, Not Active\n")
  out = sampler.stop()
  assert out["reasons"] == ["hw_slowdown", "hw_thermal_slowdown"]
  missing = bench.ClockSampler(0)
  assert missing.stop()["reasons"] == ["nvidia-smi unavailable"]
