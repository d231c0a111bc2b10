"""Metric writers: logging, JSON-lines and (optional) TensorBoard back-ends behind one
``write_scalars(step, {name: value})`` protocol; ``create_default_writer`` returns logging +
files on the main process and logging only elsewhere (the reference uses CLU's writers,
``vmoe/app.py:84-86``)."""
from __future__ import annotations

import contextlib
import json
import logging
import os
from typing import Any, List, Mapping, Optional


class MetricWriter:
  def write_scalars(self, step: int, scalars: Mapping[str, Any]) -> None:
    raise NotImplementedError

  def write_hparams(self, hparams: Mapping[str, Any]) -> None:
    pass

  def write_texts(self, step: int, texts: Mapping[str, str]) -> None:
    pass

  def flush(self) -> None:
    pass

  def close(self) -> None:
    self.flush()


def _as_float(v) -> float:
  if hasattr(v, "item"):
    return float(v.item())
  return float(v)


class LoggingWriter(MetricWriter):
  def write_scalars(self, step, scalars):
    vals = ", ".join(f"{k}={_as_float(v):.6g}" for k, v in scalars.items())
    logging.info("[%d] %s", step, vals)

  def write_hparams(self, hparams):
    logging.info("hparams: %s", dict(hparams))


class JsonlWriter(MetricWriter):
  def __init__(self, logdir: str, filename: str = "metrics.jsonl"):
    os.makedirs(logdir, exist_ok=True)
    self._fp = open(os.path.join(logdir, filename), "a")

  def write_scalars(self, step, scalars):
    rec = {"step": int(step)}
    rec.update({k: _as_float(v) for k, v in scalars.items()})
    self._fp.write(json.dumps(rec) + "\n")

  def write_texts(self, step, texts):
    self._fp.write(json.dumps({"step": int(step), "texts": dict(texts)}) + "\n")

  def flush(self):
    self._fp.flush()

  def close(self):
    self.flush()
    self._fp.close()


class TensorBoardWriter(MetricWriter):
  def __init__(self, logdir: str):
    from torch.utils.tensorboard import SummaryWriter  # needs the tensorboard package
    self._w = SummaryWriter(logdir)

  def write_scalars(self, step, scalars):
    for k, v in scalars.items():
      self._w.add_scalar(k, _as_float(v), step)

  def flush(self):
    self._w.flush()

  def close(self):
    self._w.close()


class MultiWriter(MetricWriter):
  def __init__(self, writers: List[MetricWriter]):
    self.writers = list(writers)

  def write_scalars(self, step, scalars):
    for w in self.writers:
      w.write_scalars(step, scalars)

  def write_hparams(self, hparams):
    for w in self.writers:
      w.write_hparams(hparams)

  def write_texts(self, step, texts):
    for w in self.writers:
      w.write_texts(step, texts)

  def flush(self):
    for w in self.writers:
      w.flush()

  def close(self):
    for w in self.writers:
      w.close()


def create_default_writer(logdir: Optional[str] = None, just_logging: bool = False) -> MetricWriter:
  writers: List[MetricWriter] = [LoggingWriter()]
  if logdir and not just_logging:
    writers.append(JsonlWriter(logdir))
    try:
      writers.append(TensorBoardWriter(logdir))
    except Exception:  # tensorboard not installed
      pass
  return MultiWriter(writers)


@contextlib.contextmanager
def ensure_flushes(*writers: MetricWriter):
  try:
    yield
  finally:
    for w in writers:
      w.flush()
