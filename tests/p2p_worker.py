"""Worker (one process per GPU) comparing the peer-to-peer MoE path with the NCCL path."""
import json
import logging
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vmoe_b200.ops import moe_ops  # noqa: E402
from vmoe_b200.parallel import mesh as mesh_lib  # noqa: E402
from vmoe_b200.parallel.exchange import ExpertExchange  # noqa: E402


class Mlp:
  training = False
  dropout_rate = 0.0


def run(exchange, use_p2p, tensors, k, c, steps=2):
  os.environ["VMOE_B200_P2P"] = "1" if use_p2p else "0"
  x0, res0, logits0, w1, b1, w2, b2, dy = tensors
  outs = []
  mlp = Mlp()
  mlp.w1, mlp.b1, mlp.w2, mlp.b2 = [t.detach().clone().requires_grad_() for t in (w1, b1, w2, b2)]
  for _ in range(steps):  # two rounds exercise the epoch counters and buffer reuse
    x = x0.detach().clone().requires_grad_()
    res = res0.detach().clone().requires_grad_()
    logits = logits0.detach().clone().requires_grad_()
    for p in (mlp.w1, mlp.b1, mlp.w2, mlp.b2):
      p.grad = None
    gates = torch.softmax(logits, -1)
    disp = moe_ops.FusedTopKDispatcher(gates, k, c, True, exchange=exchange)
    y = disp.apply_experts(mlp, x, residual=res)
    y.backward(dy)
    outs = [y.detach(), x.grad, res.grad, logits.grad, mlp.w1.grad, mlp.b1.grad, mlp.w2.grad,
            mlp.b2.grad]
  torch.cuda.synchronize()
  return outs


def main():
  logging.disable(logging.WARNING)
  outdir = sys.argv[1]
  mesh_lib.init_distributed()
  rank, world = dist.get_rank(), dist.get_world_size()
  mesh = mesh_lib.get_auto_logical_mesh(world)
  ex = ExpertExchange.from_mesh(mesh)
  dev = torch.device("cuda", torch.cuda.current_device())
  results = {}
  for name, (g, s, h, m, e, k, c) in {"el1": (4, 64, 128, 256, world, 2, 40),
                                        "el2": (3, 100, 64, 128, 2 * world, 2, 28)}.items():
    torch.manual_seed(100 + rank)
    el = e // world
    x = torch.randn(g, s, h, device=dev).bfloat16()
    res = torch.randn(g, s, h, device=dev).bfloat16()
    logits = torch.randn(g, s, e, device=dev)
    dy = torch.randn(g, s, h, device=dev).bfloat16()
    w1 = torch.randn(el, m, h, device=dev) * 0.05
    b1 = torch.randn(el, m, device=dev) * 0.1
    w2 = torch.randn(el, h, m, device=dev) * 0.05
    b2 = torch.randn(el, h, device=dev) * 0.1
    tensors = (x, res, logits, w1, b1, w2, b2, dy)
    ref = run(ex, False, tensors, k, c)
    got = run(ex, True, tensors, k, c)
    errs = []
    for a, b in zip(got, ref):
      scale = b.float().abs().max().item() + 1e-6
      errs.append((a.float() - b.float()).abs().max().item() / scale)
    results[name] = errs
  status = [int(cm.status.item()) for cm in moe_ops._LAYER_COMMS.values()]
  json.dump({"errs": results, "status": status}, open(os.path.join(outdir, f"p2p_r{rank}.json"), "w"))
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
