"""Worker (one process per GPU): the peer-memory expert-parallel MoE layer against a
single-process fp32 PyTorch formulation of the same layer over the gathered global batch
(indices dispatcher of ``vmoe_b200.moe``, plain matmuls, autograd), and against the NCCL path.

Cases: two toy geometries (one and two experts per rank) and, with ``--big``, the per-layer shape
of V-MoE B/16 training (1576-token groups, hidden 768, MLP 3072, capacity 416, 8 experts), which
exercises the rotated tile order, all destinations of the multi-destination store and the
fused push + GEMM launch at the sizes the benchmark runs.
"""
import json
import logging
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vmoe_b200 import moe as moe_core  # noqa: E402
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


def _gather(t, world):
  parts = [torch.empty_like(t) for _ in range(world)]
  dist.all_gather(parts, t.contiguous())
  return torch.cat(parts, dim=0)


def oracle(tensors, k, c, rank, world):
  """fp32 autograd evaluation over the global batch; returns this rank's slices."""
  x0, res0, logits0, w1, b1, w2, b2, dy0 = tensors
  g = x0.shape[0]
  X = _gather(x0, world).float().requires_grad_()
  R = _gather(res0, world).float().requires_grad_()
  L = _gather(logits0, world).float().requires_grad_()
  DY = _gather(dy0, world).float()
  W1 = _gather(w1, world).float().requires_grad_()   # (E, m, h): experts are rank-major
  B1 = _gather(b1, world).float().requires_grad_()
  W2 = _gather(w2, world).float().requires_grad_()
  B2 = _gather(b2, world).float().requires_grad_()
  gates = torch.softmax(L, -1)
  disp = moe_core.get_top_experts_per_item_dispatcher(
      gates, name="indices", num_selected_experts=k, batch_priority=True, capacity=c)
  xe = disp.dispatch(X)                                         # (E, G*C, h)
  hid = torch.nn.functional.gelu(torch.baddbmm(B1.unsqueeze(1), xe, W1.transpose(1, 2)),
                                 approximate="tanh")
  ye = torch.baddbmm(B2.unsqueeze(1), hid, W2.transpose(1, 2))
  Y = disp.combine(ye) + R
  Y.backward(DY)
  el = w1.shape[0]
  sl = slice(rank * g, (rank + 1) * g)
  es = slice(rank * el, (rank + 1) * el)
  return [Y.detach()[sl], X.grad[sl], R.grad[sl], L.grad[sl], W1.grad[es], B1.grad[es],
          W2.grad[es], B2.grad[es]]


def run_soft(exchange, tensors, e, c, steps=2):
  """Soft-MoE-style layer: real-valued dispatch / combine weights over every (expert, slot),
  slot rows exchanged over peer memory inside the expert GEMMs."""
  os.environ["VMOE_B200_P2P"] = "1"
  x0, wd0, wc0, w1, b1, w2, b2, dy = tensors
  mlp = Mlp()
  mlp.w1, mlp.b1, mlp.w2, mlp.b2 = [t.detach().clone().requires_grad_() for t in (w1, b1, w2, b2)]
  outs = []
  for _ in range(steps):
    x = x0.detach().clone().requires_grad_()
    wd = wd0.detach().clone().requires_grad_()
    wc = wc0.detach().clone().requires_grad_()
    for p in (mlp.w1, mlp.b1, mlp.w2, mlp.b2):
      p.grad = None
    disp = moe_core.Bfloat16Dispatcher(moe_core.EinsumDispatcher(
        combine_weights=wc, dispatch_weights=wd, exchange=exchange))
    y = disp.apply_experts(mlp, x)
    y.backward(dy)
    outs = [y.detach(), x.grad, wd.grad, wc.grad, mlp.w1.grad, mlp.b1.grad, mlp.w2.grad,
            mlp.b2.grad]
  torch.cuda.synchronize()
  return outs


def oracle_soft(tensors, rank, world):
  """fp32 einsum formulation over the global batch (weights rounded to bf16 like the kernels')."""
  x0, wd0, wc0, w1, b1, w2, b2, dy0 = tensors
  g = x0.shape[0]
  X = _gather(x0, world).float().requires_grad_()
  WD = _gather(wd0, world).float().requires_grad_()
  WC = _gather(wc0, world).float().requires_grad_()
  DY = _gather(dy0, world).float()
  W1 = _gather(w1, world).float().requires_grad_()
  B1 = _gather(b1, world).float().requires_grad_()
  W2 = _gather(w2, world).float().requires_grad_()
  B2 = _gather(b2, world).float().requires_grad_()
  G, S, E, C = WD.shape
  q = lambda t: t + (t.detach().bfloat16().float() - t.detach())   # bf16 value, fp32 gradient
  xs = torch.einsum("gsec,gsh->egch", q(WD), X).reshape(E, G * C, -1)
  hid = torch.nn.functional.gelu(torch.baddbmm(B1.unsqueeze(1), xs, W1.transpose(1, 2)),
                                 approximate="tanh")
  ye = torch.baddbmm(B2.unsqueeze(1), hid, W2.transpose(1, 2)).reshape(E, G, C, -1)
  Y = torch.einsum("gsec,egch->gsh", q(WC), ye)
  Y.backward(DY)
  el = w1.shape[0]
  sl = slice(rank * g, (rank + 1) * g)
  es = slice(rank * el, (rank + 1) * el)
  return [Y.detach()[sl], X.grad[sl], WD.grad[sl], WC.grad[sl], W1.grad[es], B1.grad[es],
          W2.grad[es], B2.grad[es]]


def rel_errs(got, ref):
  errs = []
  for a, b in zip(got, ref):
    scale = b.float().abs().max().item() + 1e-6
    errs.append((a.float() - b.float()).abs().max().item() / scale)
  return errs


def main():
  logging.disable(logging.WARNING)
  outdir = sys.argv[1]
  big = "--big" in sys.argv
  mesh_lib.init_distributed()
  rank, world = dist.get_rank(), dist.get_world_size()
  mesh = mesh_lib.get_auto_logical_mesh(world)
  ex = ExpertExchange.from_mesh(mesh)
  dev = torch.device("cuda", torch.cuda.current_device())
  torch.backends.cuda.matmul.allow_tf32 = False
  cases = {"el1": (4, 64, 128, 256, world, 2, 40), "el2": (3, 100, 64, 128, 2 * world, 2, 28)}
  if big and 8 % world == 0:
    cases["b16_layer"] = (32 if world >= 8 else 64, 1576, 768, 3072, 8, 2, 416)
  results, oracle_errs = {}, {}
  for name, (g, s, h, m, e, k, c) in cases.items():
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
    got = run(ex, True, tensors, k, c)
    # The kernels multiply bf16 copies of the weights: the oracle gets the same rounded values.
    want = oracle((x, res, logits, w1.bfloat16().float(), b1, w2.bfloat16().float(), b2, dy), k,
                  c, rank, world)
    oracle_errs[name] = rel_errs(got, want)
    del want
    torch.cuda.empty_cache()
    if name != "b16_layer":
      ref = run(ex, False, tensors, k, c)
      results[name] = rel_errs(got, ref)
  # Soft-MoE-style layers: (groups, tokens, hidden, mlp, experts, slots per expert)
  for name, (g, s, h, m, e, c) in {"soft_c1": (32, 49, 64, 128, 4 * world, 1),
                                     "soft_c2": (16, 40, 128, 256, 2 * world, 2)}.items():
    torch.manual_seed(200 + rank)
    el = e // world
    x = torch.randn(g, s, h, device=dev).bfloat16()
    logits = torch.randn(g, s, e, c, device=dev)
    wd = torch.softmax(logits, dim=1)
    wc = torch.softmax(logits.reshape(g, s, e * c), dim=-1).reshape(g, s, e, c)
    dy = torch.randn(g, s, h, device=dev).bfloat16()
    w1 = torch.randn(el, m, h, device=dev) * 0.05
    b1 = torch.randn(el, m, device=dev) * 0.1
    w2 = torch.randn(el, h, m, device=dev) * 0.05
    b2 = torch.randn(el, h, device=dev) * 0.1
    got = run_soft(ex, (x, wd, wc, w1, b1, w2, b2, dy), e, c)
    want = oracle_soft((x, wd, wc, w1.bfloat16().float(), b1, w2.bfloat16().float(), b2, dy),
                       rank, world)
    oracle_errs[name] = rel_errs(got, want)
  soft_comms = sum(1 for k in moe_ops._LAYER_COMMS)
  status = [int(cm.status.item()) for cm in moe_ops._LAYER_COMMS.values()]
  for cm in moe_ops._LAYER_COMMS.values():
    cm.check_guards()  # nothing was stored between or past the peer-written regions
  json.dump({"errs": results, "oracle_errs": oracle_errs, "status": status,
             "layer_comms": soft_comms},
            open(os.path.join(outdir, f"p2p_r{rank}.json"), "w"))
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
