"""Worker for the multi-process CPU (gloo) tests; launched by tests/test_distributed_cpu.py."""
import json
import logging
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vmoe_b200.configs.vmoe_paper import common  # noqa: E402
from vmoe_b200.parallel import mesh as mesh_lib  # noqa: E402
from vmoe_b200.parallel import multihost_utils  # noqa: E402
from vmoe_b200.train import trainer  # noqa: E402


def small_config():
  cfg = common.get_vmoe_config("ViT-S/32, E=8, K=2, Last 2", 64, 10)
  cfg.hidden_size = 64
  cfg.representation_size = None
  cfg.head_kernel_zero_init = False
  cfg.encoder.num_layers = 4
  cfg.encoder.mlp_dim = 128
  cfg.encoder.num_heads = 4
  cfg.encoder.moe.layers = (1, 3)
  cfg.encoder.moe.num_experts = 4
  cfg.encoder.moe.group_size = 10  # two images of 5 tokens
  cfg.encoder.moe.split_rngs = True
  cfg.encoder.moe.router.noise_std = 0.0
  cfg.encoder.moe.router.dispatcher.batch_priority = True
  return cfg


def main():
  logging.disable(logging.WARNING)
  mode, outdir = sys.argv[1], sys.argv[2]
  mesh_lib.init_distributed(backend="gloo")
  world = dist.get_world_size() if dist.is_initialized() else 1
  rank = dist.get_rank() if dist.is_initialized() else 0
  partitions = int(os.environ.get("EXPERT_PARTITIONS", "2"))
  mesh = mesh_lib.get_auto_logical_mesh(partitions)
  mesh_lib.set_mesh(mesh)
  if mode == "barrier_mismatch":
    try:
      multihost_utils.sync_devices("same" if rank == 0 else "different", main_process=rank)
      ok = "no error"
    except ValueError as e:
      ok = "ValueError"
    json.dump({"result": ok}, open(os.path.join(outdir, f"r{rank}.json"), "w"))
    return
  if mode in ("peer_stops", "peer_leaves", "barrier_absent"):
    from vmoe_b200.parallel import failure
    hb = failure.Heartbeat()
    result = {}
    if mode == "barrier_absent":
      if rank == 0:
        try:
          failure.store_barrier("sync", timeout_s=1.5)
          result["result"] = "no error"
        except failure.BarrierTimeout as e:
          result["result"], result["missing"] = "BarrierTimeout", e.missing
      else:
        result["result"] = "absent"  # this rank never joins the barrier
    else:
      hb.beat(1)
      hb.check(1, timeout_s=30.0)  # everybody reached step 1
      if rank == 0:
        hb.beat(2)
        try:
          hb.check(2, timeout_s=1.5)
          result["result"] = "no error"
        except failure.PeerFailure as e:
          result["result"], result["ranks"], result["left"] = "PeerFailure", e.ranks, e.left
      else:
        # The failure is made on the host: this rank stops (or leaves) before step 2 and
        # never publishes it.
        if mode == "peer_leaves":
          hb.leave()
        result["result"] = "stopped"
    json.dump(result, open(os.path.join(outdir, f"r{rank}.json"), "w"))
    # Both processes are still alive (the failure was only acted out): leave together so the
    # store outlives every client.
    dist.barrier()
    dist.destroy_process_group()
    return
  if mode == "ckpt_fallback":
    # Both ranks save steps 1 and 2; reading step 2 then fails on rank 1 only (a fake of the
    # failing call), and both ranks must fall back to step 1 together.
    from vmoe_b200.checkpoints import partitioned
    make = lambda seed: trainer.create_train_state(
        model_config=small_config(), optimizer_config=dict(name="adam", learning_rate=1e-3),
        total_steps=10, mesh=mesh, seed=seed, image_size=64)
    state = make(0)
    mgr = trainer.CheckpointManager(workdir=outdir, every_steps=1, keep_last=5, mesh=mesh)
    for step in (1, 2):
      with torch.no_grad():
        state.model.head.bias.fill_(float(step))
      state.step = step
      mgr.save(step, state, force=True)
    mgr.wait_until_finished()
    multihost_utils.sync_devices("saved")
    real = partitioned.restore_checkpoint

    def flaky(prefix, *args, **kwargs):
      if rank == 1 and prefix.endswith("_2"):
        raise OSError("injected read failure")
      return real(prefix, *args, **kwargs)

    partitioned.restore_checkpoint = flaky
    fresh = make(1)
    restored = mgr.restore(fresh)
    result = {"restored": restored, "bias": float(fresh.model.head.bias.detach()[0]),
              "step": fresh.step}
    try:
      mgr.restore(make(1), step=2)
      result["explicit"] = "no error"
    except trainer.CheckpointReadError as e:
      result["explicit"] = str(e)
    mgr.close()
    json.dump(result, open(os.path.join(outdir, f"r{rank}.json"), "w"))
    dist.barrier()
    dist.destroy_process_group()
    return
  if mode == "contrastive":
    # Two-tower SigLIP step: 8 (image, text) pairs split over the ranks; dense towers so that
    # the only thing the split can change is which texts each image is contrasted with.
    from vmoe_b200.projects.contrastive import trainer as ctrainer
    enc = {"num_layers": 1, "mlp_dim": 32, "num_heads": 2, "dropout_rate": 0.0,
           "attention_dropout_rate": 0.0, "moe": {"layers": ()}}
    image = {"num_classes": 12, "patch_size": (8, 8), "hidden_size": 16, "classifier": "token",
             "representation_size": None, "encoder": dict(enc)}
    text = {"vocab_size": 50, "num_classes": 12, "hidden_size": 16, "encoder": dict(enc)}
    state = ctrainer.create_train_state(
        model_config={"image": image, "text": text, "scale_init": 10.0, "bias_init": -10.0},
        optimizer_config=dict(name="sgd", learning_rate=0.1), total_steps=10, mesh=mesh, seed=0,
        image_size=16)
    gen = torch.Generator().manual_seed(5)
    images = torch.rand(8, 16, 16, 3, generator=gen)
    texts = torch.randint(1, 50, (8, 16), generator=gen)
    per = 8 // world
    sl = slice(rank * per, (rank + 1) * per)
    before = {n: p.detach().clone() for n, p in state.model.named_parameters()}
    _, metrics = ctrainer.train_step(state, images[sl], texts[sl], ctrainer.sigmoid_loss)
    delta = {n: float((p.detach() - before[n]).double().abs().sum())
             for n, p in state.model.named_parameters()}
    out = {"main_loss": float(metrics["main_loss"]),
           "grad_norm": float(metrics["global_norm/grads"]),
           "delta_txt": sum(v for n, v in delta.items() if n.startswith("txt.")),
           "delta_img": sum(v for n, v in delta.items() if n.startswith("img.")),
           "scale": float(state.model.s.detach()), "bias": float(state.model.b.detach())}
    json.dump(out, open(os.path.join(outdir, f"r{rank}.json"), "w"))
    if dist.is_initialized():
      dist.barrier()
      dist.destroy_process_group()
    return
  multihost_utils.sync_devices("start")
  state = trainer.create_train_state(
      model_config=small_config(),
      optimizer_config=dict(name="adam", learning_rate=1e-3, weight_decay=0.1),
      total_steps=10, mesh=mesh, seed=0, image_size=64)
  gen = torch.Generator().manual_seed(123)
  images = torch.rand(8, 64, 64, 3, generator=gen) * 2 - 1
  labels = torch.nn.functional.one_hot(torch.randint(0, 10, (8,), generator=gen), 10).float()
  per = 8 // world
  loss_fn, _, _ = trainer.get_loss_fn("softmax_xent")
  _, metrics = trainer.train_step(state, images[rank * per:(rank + 1) * per],
                                  labels[rank * per:(rank + 1) * per], loss_fn)
  out = {"main_loss": float(metrics["main_loss"]), "grad_norm": float(metrics["global_norm/grads"]),
         "aux_loss": float(metrics.get("auxiliary_loss", 0.0))}
  # Save and reload the sharded checkpoint, then compare against the live state.
  mgr = trainer.CheckpointManager(workdir=outdir, every_steps=1, mesh=mesh)
  mgr.save(1, state, force=True)
  mgr.wait_until_finished()
  multihost_utils.sync_devices("saved")
  state2 = trainer.create_train_state(
      model_config=small_config(),
      optimizer_config=dict(name="adam", learning_rate=1e-3, weight_decay=0.1),
      total_steps=10, mesh=mesh, seed=1, image_size=64)
  restored = mgr.restore(state2)
  same = all(torch.equal(a.data, b.data) for a, b in
             zip(state.model.parameters(), state2.model.parameters()))
  out.update(restored=restored, same=bool(same), step=state2.step)
  mgr.close()
  # Full (global) parameter values for comparison across world sizes.
  from vmoe_b200.checkpoints import partitioned
  full = partitioned.restore_checkpoint(os.path.join(outdir, "ckpt", "ckpt_1"),
                                        mesh=mesh_lib.Mesh())
  w = full["params"]["Encoder"]["encoderblock_1"]["Moe"]["Mlp"]["Dense_0"]["kernel"]
  h = full["params"]["head"]["kernel"]
  out.update(expert_kernel_sum=float(np.abs(w).sum()), expert_kernel_shape=list(w.shape),
             head_sum=float(np.abs(h).sum()),
             q_sum=float(np.abs(full["params"]["Encoder"]["encoderblock_0"]["SelfAttention"]["query"]["kernel"]).sum()))
  json.dump(out, open(os.path.join(outdir, f"r{rank}.json"), "w"))
  if dist.is_initialized():
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  main()
