"""Worker (one process per GPU): training steps with the overlapped peer-memory gradient
all-reduce must match the same steps with the NCCL all-reduce."""
import json
import logging
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tests.dist_worker import small_config  # noqa: E402
from vmoe_b200.parallel import grad_allreduce  # noqa: E402
from vmoe_b200.parallel import mesh as mesh_lib  # noqa: E402
from vmoe_b200.train import trainer  # noqa: E402


def run(mesh, device, use_p2p, rank, steps=3):
  os.environ["VMOE_B200_GRAD_P2P"] = "1" if use_p2p else "0"
  cfg = small_config()
  cfg.encoder.dtype = "bfloat16"
  state = trainer.create_train_state(
      model_config=cfg, optimizer_config=dict(name="adam", learning_rate=1e-3, weight_decay=0.1),
      total_steps=10, mesh=mesh, device=device, seed=0, image_size=64)
  assert (state.optimizer.grad_reducer is not None) == use_p2p
  loss_fn, _, _ = trainer.get_loss_fn("softmax_xent")
  gen = torch.Generator().manual_seed(1000 + rank)
  norms = []
  for _ in range(steps):
    images = (torch.rand(8, 64, 64, 3, generator=gen) * 2 - 1).to(device)
    labels = torch.nn.functional.one_hot(torch.randint(0, 10, (8,), generator=gen), 10).float()
    _, metrics = trainer.train_step(state, images, labels.to(device), loss_fn)
    norms.append(float(metrics["global_norm/grads"]))
  torch.cuda.synchronize()
  status = 0
  if state.optimizer.grad_reducer is not None:
    status = int(state.optimizer.grad_reducer.status.item())
    state.optimizer.grad_reducer.buf.check_guards("gradient all-reduce buffer")
    ranges = state.optimizer.grad_reducer.num_ranges
    state.optimizer.grad_reducer.deactivate()
  else:
    ranges = 0
  params = [p.detach().float().clone() for p in state.model.parameters()]
  return params, norms, status, ranges


def main():
  logging.disable(logging.WARNING)
  watchdog = int(os.environ.get("WORKER_WATCHDOG_S", "0"))
  if watchdog:
    # Dump every thread's Python stack and exit if the worker is still running by then.
    import faulthandler
    faulthandler.dump_traceback_later(watchdog, exit=True)
  outdir = sys.argv[1]
  mesh_lib.init_distributed()
  rank, world = dist.get_rank(), dist.get_world_size()
  mesh = mesh_lib.get_auto_logical_mesh(min(world, 4))
  mesh_lib.set_mesh(mesh)
  device = torch.device("cuda", torch.cuda.current_device())
  ref, ref_norms, _, _ = run(mesh, device, False, rank)
  got, got_norms, status, ranges = run(mesh, device, True, rank)
  err = max(((a - b).abs().max() / (b.abs().max() + 1e-6)).item() for a, b in zip(got, ref))
  json.dump({"err": err, "norms": got_norms, "ref_norms": ref_norms, "status": status,
             "ranges": ranges}, open(os.path.join(outdir, f"ar_r{rank}.json"), "w"))
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
