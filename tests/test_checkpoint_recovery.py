"""Recovery from checkpoints damaged on the host: truncated shard files, a corrupted index,
leftover temporary files. The newest readable step is restored; a step asked for by number
raises a clear error. No GPU is involved."""
import glob
import os

import pytest
import torch

from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.parallel import multihost_utils
from vmoe_b200.train import trainer

MODEL = {
    "name": "VisionTransformerMoe", "num_classes": 5, "patch_size": (8, 8), "hidden_size": 16,
    "classifier": "token", "representation_size": None,
    "encoder": {"num_layers": 2, "num_heads": 2, "mlp_dim": 32, "dropout_rate": 0.0,
                "attention_dropout_rate": 0.0,
                "moe": {"num_experts": 2, "layers": (1,), "group_size": 10,
                        "router": {"num_selected_experts": 1, "noise_std": 1.0,
                                   "dispatcher": {"name": "einsum", "capacity_factor": 2.0,
                                                  "batch_priority": False}}}},
}
OPTIMIZER = {"name": "adam", "learning_rate": 0.01}


def _state(mesh, seed=0):
  return trainer.create_train_state(model_config=MODEL, optimizer_config=OPTIMIZER,
                                    total_steps=10, mesh=mesh, seed=seed, image_size=16)


def _manager(tmp_path, mesh):
  return trainer.CheckpointManager(workdir=str(tmp_path), every_steps=1, keep_last=10, mesh=mesh)


def _save_steps(tmp_path, mesh, steps):
  """Saves checkpoints whose head bias equals the step number."""
  state = _state(mesh)
  manager = _manager(tmp_path, mesh)
  for step in steps:
    with torch.no_grad():
      state.model.head.bias.fill_(float(step))
    state.step = step
    manager.save(step, state, force=True)
  manager.close()
  return manager.prefix


@pytest.fixture
def mesh():
  m = mesh_lib.get_auto_logical_mesh(1)
  mesh_lib.set_mesh(m)
  return m


def _restore_into_fresh_state(tmp_path, mesh, step=None):
  state = _state(mesh, seed=1)
  manager = _manager(tmp_path, mesh)
  try:
    return manager.restore(state, step=step), state
  finally:
    manager.close()


def test_restores_the_newest_step(tmp_path, mesh):
  _save_steps(tmp_path, mesh, [1, 2, 3])
  step, state = _restore_into_fresh_state(tmp_path, mesh)
  assert step == 3 and state.step == 3
  assert state.model.head.bias.detach()[0].item() == 3.0


def test_truncated_shard_falls_back_to_the_previous_step(tmp_path, mesh, caplog):
  prefix = _save_steps(tmp_path, mesh, [1, 2, 3])
  shards = sorted(glob.glob(f"{prefix}_3.data-*"))
  assert shards
  size = os.path.getsize(shards[0])
  with open(shards[0], "r+b") as fp:
    fp.truncate(size // 2)
  step, state = _restore_into_fresh_state(tmp_path, mesh)
  assert step == 2 and state.model.head.bias.detach()[0].item() == 2.0
  assert any("Skipping checkpoint step 3" in r.getMessage() for r in caplog.records)


def test_corrupted_index_falls_back_and_explicit_step_raises(tmp_path, mesh):
  prefix = _save_steps(tmp_path, mesh, [1, 2])
  with open(f"{prefix}_2.index", "wb") as fp:
    fp.write(b"\x00not a msgpack index\xff")
  step, state = _restore_into_fresh_state(tmp_path, mesh)
  assert step == 1 and state.model.head.bias.detach()[0].item() == 1.0
  with pytest.raises(trainer.CheckpointReadError, match="ckpt_2 cannot be read"):
    _restore_into_fresh_state(tmp_path, mesh, step=2)


def test_steps_with_temporary_or_missing_files_are_not_candidates(tmp_path, mesh):
  prefix = _save_steps(tmp_path, mesh, [1, 2, 3])
  # Step 3: a writer died before renaming one shard. Step 2: its index never appeared.
  shard = sorted(glob.glob(f"{prefix}_3.data-*"))[0]
  os.rename(shard, os.path.join(os.path.dirname(shard), ".tmp." + os.path.basename(shard)))
  os.remove(f"{prefix}_2.index")
  manager = _manager(tmp_path, mesh)
  assert manager.all_steps() == [1]
  manager.close()
  step, state = _restore_into_fresh_state(tmp_path, mesh)
  assert step == 1 and state.model.head.bias.detach()[0].item() == 1.0


def test_nothing_readable_returns_none_and_leaves_the_state_alone(tmp_path, mesh):
  prefix = _save_steps(tmp_path, mesh, [1])
  for f in glob.glob(f"{prefix}_1.data-*"):
    with open(f, "wb") as fp:
      fp.write(b"")
  fresh = _state(mesh, seed=1)
  before = fresh.model.head.bias.detach().clone()
  manager = _manager(tmp_path, mesh)
  assert manager.restore(fresh) is None
  manager.close()
  assert torch.equal(fresh.model.head.bias.detach(), before) and fresh.step == 0


def test_all_ranks_ok_without_a_process_group():
  assert multihost_utils.all_ranks_ok(True) is True
  assert multihost_utils.all_ranks_ok(False) is False


def test_saved_values_are_those_at_the_time_of_the_call(tmp_path, mesh):
  # The writer threads run while training goes on: changing a parameter right after save()
  # must not change what ends up in the file.
  state = _state(mesh)
  manager = _manager(tmp_path, mesh)
  with torch.no_grad():
    state.model.head.bias.fill_(7.0)
  state.step = 1
  manager.save(1, state, force=True)
  with torch.no_grad():
    state.model.head.bias.fill_(-1.0)
    for p in state.model.parameters():
      p.mul_(0.0)
  manager.close()
  step, restored = _restore_into_fresh_state(tmp_path, mesh)
  assert step == 1 and restored.model.head.bias.detach()[0].item() == 7.0
  assert float(restored.model.head.weight.detach().abs().sum()) >= 0.0
  assert any(float(p.detach().abs().sum()) > 0 for p in restored.model.parameters())


def test_older_checkpoints_survive_a_failed_write(tmp_path, mesh, monkeypatch):
  """keep_last = 1: the previous step is deleted only after the new one is completely on disk.
  A write that fails leaves the previous step restorable."""
  from vmoe_b200.checkpoints import partitioned
  state = _state(mesh)
  manager = trainer.CheckpointManager(workdir=str(tmp_path), every_steps=1, keep_last=1, mesh=mesh)
  with torch.no_grad():
    state.model.head.bias.fill_(1.0)
  state.step = 1
  manager.save(1, state, force=True)
  manager.wait_until_finished()
  assert manager.all_steps() == [1]

  class _Failing:
    def get(self, timeout=None):
      raise IOError("disk full")

  real_save = partitioned.save_checkpoint
  monkeypatch.setattr(partitioned, "save_checkpoint", lambda *a, **k: _Failing())
  state.step = 2
  manager.save(2, state, force=True)
  assert 1 in manager.all_steps()          # nothing is deleted while the write is in flight
  with pytest.raises(IOError):
    manager.wait_until_finished()
  assert 1 in manager.all_steps()          # ... nor after it failed
  monkeypatch.setattr(partitioned, "save_checkpoint", real_save)
  other = _state(mesh, seed=3)
  assert manager.restore(other) == 1
  assert float(other.model.head.bias[0]) == 1.0
  # A later successful save removes the old step once it has finished.
  state.step = 3
  manager.save(3, state, force=True)
  assert 1 in manager.all_steps()
  manager.wait_until_finished()
  assert manager.all_steps() == [3]
  manager.close()


def test_adafactor_resumes_with_its_second_moments(tmp_path, mesh):
  """k steps, save, restore into a fresh state, one more step == k + 1 uninterrupted steps."""
  opt_cfg = {"name": "big_vision_adafactor", "learning_rate": 0.01, "momentum": 0.9}
  def make(seed):
    return trainer.create_train_state(model_config=MODEL, optimizer_config=opt_cfg,
                                      total_steps=10, mesh=mesh, seed=seed, image_size=16)
  loss_fn, _, _ = trainer.get_loss_fn("softmax_xent")
  g = torch.Generator().manual_seed(0)
  batches = [(torch.rand(4, 16, 16, 3, generator=g),
              torch.nn.functional.one_hot(torch.randint(0, 5, (4,), generator=g), 5).float())
             for _ in range(4)]
  ref = make(0)
  for x, y in batches[:3]:
    trainer.train_step(ref, x, y, loss_fn)
  torch.manual_seed(77)   # the router's noise comes from the global generator
  trainer.train_step(ref, *batches[3], loss_fn)
  run = make(0)
  for x, y in batches[:3]:
    trainer.train_step(run, x, y, loss_fn)
  manager = trainer.CheckpointManager(workdir=str(tmp_path), every_steps=1, keep_last=1, mesh=mesh)
  manager.save(3, run, force=True)
  manager.wait_until_finished()
  resumed = make(5)
  assert manager.restore(resumed) == 3
  manager.close()
  torch.manual_seed(77)
  trainer.train_step(resumed, *batches[3], loss_fn)
  for (n, a), (_, b) in zip(ref.model.named_parameters(), resumed.model.named_parameters()):
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6, msg=n)
