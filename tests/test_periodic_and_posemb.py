"""Periodic actions, metric writers and the fixed 2-D position embedding.

Golden values of the position embedding follow the reference's test
(``vmoe/nn/vit_moe_test.py:93-129``); the periodic-action cases follow
``vmoe/train/periodic_actions_test.py``.
"""
import json
import math
import os
from unittest import mock

import pytest
import torch

from vmoe_b200.models import vit_moe
from vmoe_b200.train import periodic_actions
from vmoe_b200.utils import metric_writers


class _RecordingWriter(metric_writers.MetricWriter):

  def __init__(self):
    self.calls = []

  def write_scalars(self, step, scalars):
    self.calls.append((step, dict(scalars)))


_S, _C = math.sin(1.0), math.cos(1.0)
_GRID = [
    [0, 0, 1, 1, 0, 0, 1, 1],
    [_S, _S, _C, _C, 0, 0, 1, 1],
    [0, 0, 1, 1, _S, _S, _C, _C],
    [_S, _S, _C, _C, _S, _S, _C, _C],
]


def test_sincos2d_values():
  pe = vit_moe.sincos2d_position_embedding(2, 2, 8, temperature=1.0)
  assert pe.shape == (1, 4, 8)
  torch.testing.assert_close(pe[0], torch.tensor(_GRID, dtype=torch.float32))


@pytest.mark.parametrize("seq_len, rows", [(4, _GRID), (5, [[0.0] * 8] + _GRID)])
def test_encoder_with_sincos2d(seq_len, rows):
  enc = vit_moe.EncoderMoe(num_layers=0, mlp_dim=4, num_heads=1, hidden_size=8, seq_len=seq_len,
                           position_emb={"name": "sincos2d", "h": 2, "w": 2, "temperature": 1.0})
  x = torch.zeros(2, seq_len, 8)
  y, _ = enc(x)
  pe = torch.tensor(rows, dtype=torch.float32)
  expected = torch.nn.functional.layer_norm(pe, (8,), eps=1e-6)
  torch.testing.assert_close(y, torch.stack([expected, expected]), rtol=1e-3, atol=1e-4)


def test_encoder_with_sincos2d_rejects_other_lengths():
  enc = vit_moe.EncoderMoe(num_layers=0, mlp_dim=4, num_heads=1, hidden_size=8, seq_len=6,
                           position_emb={"name": "sincos2d", "h": 2, "w": 2, "temperature": 1.0})
  with pytest.raises(ValueError):
    enc(torch.zeros(2, 6, 8))


def test_sincos2d_rejects_small_hidden_size():
  with pytest.raises(ValueError):
    vit_moe.sincos2d_position_embedding(2, 2, 6)


def test_periodic_action_triggers():
  fired = []
  action = periodic_actions.PeriodicCallback(
      every_steps=3, on_steps=[4], callback_fn=lambda step, t: fired.append(step))
  for step in range(1, 10):
    action(step, t=float(step))
  assert fired == [3, 4, 6, 9]


def test_periodic_action_every_secs():
  fired = []
  action = periodic_actions.PeriodicCallback(
      every_secs=2.5, callback_fn=lambda step, t: fired.append(step))
  for step in range(1, 10):
    action(step, t=float(step))
  assert fired == [4, 7]


def test_periodic_action_rejects_skipped_steps():
  action = periodic_actions.PeriodicCallback(every_steps=2, callback_fn=lambda step, t: None)
  action(1, t=0.0)
  with pytest.raises(ValueError):
    action(3, t=1.0)


@pytest.mark.parametrize("process_index, expected", [(0, [1, 2]), (1, [])])
def test_single_process_periodic_action(process_index, expected):
  calls = []
  inner = periodic_actions.PeriodicCallback(every_steps=1,
                                            callback_fn=lambda step, t: calls.append(step))
  action = periodic_actions.SingleProcessPeriodicAction(periodic_action=inner, process_index=0)
  with mock.patch.object(periodic_actions, "_process_index", return_value=process_index):
    action(1, t=0.0)
    action(2, t=1.0)
  assert calls == expected


def test_report_progress_scalars():
  writer = _RecordingWriter()
  report = periodic_actions.ReportProgress(num_train_steps=10, writer=writer, every_steps=2,
                                           every_secs=None)
  report._t0 = 0.0
  with report.timed("training", wait_jax_async_dispatch=False):
    pass
  report(1, t=1.0)
  report(2, t=2.0, scalar_metrics={"loss": 2.0, "norm": {"grads": 3.0}})
  report(3, t=3.0)
  report(4, t=6.0, scalar_metrics={"loss": 1.0})
  assert [c[0] for c in writer.calls] == [2, 4]
  first, second = writer.calls[0][1], writer.calls[1][1]
  assert first["steps_per_sec"] == pytest.approx(1.0)
  assert first["loss"] == 2.0 and first["norm/grads"] == 3.0
  assert first["uptime"] == pytest.approx(2.0)
  assert "uptime_training" in first
  assert second["steps_per_sec"] == pytest.approx(0.5)
  assert second["loss"] == 1.0 and "norm/grads" not in second


def test_report_progress_only_on_its_process():
  writer = _RecordingWriter()
  report = periodic_actions.ReportProgress(writer=writer, every_steps=1, every_secs=None,
                                           process_index=0)
  with mock.patch.object(periodic_actions, "_process_index", return_value=1):
    report(1, t=0.0)
    report(2, t=1.0)
  assert writer.calls == []


def test_jsonl_writer_and_default_writer(tmp_path):
  writer = metric_writers.create_default_writer(str(tmp_path), just_logging=False)
  with metric_writers.ensure_flushes(writer):
    writer.write_scalars(3, {"a": 1.5, "b": torch.tensor(2.0)})
  files = [f for f in os.listdir(tmp_path) if f.endswith(".jsonl")]
  assert files
  rows = [json.loads(line) for line in open(tmp_path / files[0])]
  assert rows[-1]["step"] == 3 and rows[-1]["a"] == 1.5 and rows[-1]["b"] == 2.0
  just_logging = metric_writers.create_default_writer(str(tmp_path / "other"), just_logging=True)
  just_logging.write_scalars(1, {"a": 1.0})
  assert not os.path.exists(tmp_path / "other") or not os.listdir(tmp_path / "other")
