"""Times one expert-parallel MoE layer (dispatch -> expert MLP -> combine) on N GPUs.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port 29533 -m vmoe_b200.ops.bench_moe_layer [--path p2p|nccl] [--iters 10]

Shapes follow V-MoE B/16 training with 512 images per GPU: 32 groups of 3152 tokens per GPU,
hidden 768, MLP 3072, 8 experts, K=2, capacity 832 per (group, expert). Times are CUDA-event
times, maximum over ranks. The roofline of each fused half (dispatch + GEMM1, GEMM2 + combine)
is the slower of its FLOPs at the measured GEMM peak and its bytes over NVLink at the measured
770 GB/s per direction; rank 0 prints achieved / roofline.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


class _Mlp:
  training = False
  dropout_rate = 0.0


def layer_phases(moe_ops, disp, mlp, x, res, dy, ex, c, iters):
  """The launches of the peer-memory layer (``moe_ops._P2PMoeFn``), forward then backward, with
  a CUDA event between them; returns mean milliseconds per phase on this rank."""
  from vmoe_b200.ops.functional import _wgrad_split, bf16_shadow, bias_grad, wgrad
  from vmoe_b200.ops.gemm import ACT_GELU, gemm
  g, s, h = x.shape
  e, k = disp.num_experts, disp.expert.shape[-1]
  r = g * c
  comm = moe_ops.layer_comm(mlp, ex, e, r, h, x.device)
  ep, el, rank = comm.ep, comm.el, comm.rank
  w1h, w2h = bf16_shadow(mlp.w1), bf16_shadow(mlp.w2)
  m = mlp.w1.shape[1]
  gate = disp.combine_weights.detach().float().contiguous()
  names = ["wait_free", "push+gemm1", "gemm2_to_peers", "wait_y", "combine",
           "push_dy+dgrad", "dx_to_peers", "bias+wgrads", "signal_free+wait_dx", "combine_dx"]
  total = {n: 0.0 for n in names}
  xd, dyd = x.detach(), dy.detach()
  with torch.no_grad():
    for it in range(iters + 2):
      ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
      ev[0].record()
      if comm.epoch["free"] > 0:
        moe_ops.wait_counters(comm.ffree, ep, comm.epoch["free"], comm.status)
      for key in ("x", "y", "dy", "dx"):
        comm.epoch[key] += 1
      ev[1].record()
      pre = torch.empty(el, ep * r, m, dtype=torch.bfloat16, device=x.device)
      pa = moe_ops.push_args(xd, disp.slot_pair, None, comm.push_x, comm.flag_x, None, None, g, s,
                             e, c, k, h, el, ep, rank)
      hid = gemm(comm.xe, w1h, bias=mlp.b1, act=ACT_GELU, out_pre=pre, out_pre_is_grad=True,
                 a_ready=comm.fx, a_ready_epoch=comm.epoch["x"], status=comm.status,
                 mt_offset=comm.mt_offset, push=pa)
      ev[2].record()
      gemm(hid, w2h, bias=mlp.b2, out_multi=[comm.home_out("YB", src) for src in range(ep)],
           mt_offset=comm.mt_offset, signal_flags=comm.done_flag_addrs("FY"),
           done_counter=comm.done[0:1])
      ev[3].record()
      moe_ops.wait_counters(comm.fy, ep, comm.epoch["y"], comm.status)
      ev[4].record()
      out = torch.empty_like(xd)
      moe_ops.combine_rows(comm.yb_table, disp.expert, disp.slot, gate, res, out, g, s, e, c, k, h)
      ev[5].record()
      # ---- backward
      dgate = torch.zeros(g, s, k, dtype=torch.float32, device=x.device)
      pa = moe_ops.push_args(dyd, disp.slot_pair, gate, comm.push_dy, comm.flag_dy, comm.yb_table,
                             dgate, g, s, e, c, k, h, el, ep, rank)
      db1 = torch.zeros(el, m, dtype=torch.float32, device=x.device)
      dpre = gemm(comm.dye, w2h, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True, colsum=db1,
                  a_ready=comm.fdy, a_ready_epoch=comm.epoch["dy"], status=comm.status,
                  mt_offset=comm.mt_offset, push=pa)
      ev[6].record()
      gemm(dpre, w1h, b_mn_major=True, out_multi=[comm.home_out("DXB", src) for src in range(ep)],
           mt_offset=comm.mt_offset, signal_flags=comm.done_flag_addrs("FDX"),
           done_counter=comm.done[1:2])
      ev[7].record()
      mlp.w1.grad = mlp.w2.grad = mlp.b2.grad = None
      bias_grad(comm.dye, mlp.b2)
      wgrad(comm.dye, hid, mlp.w2, split_k=_wgrad_split(h, m, ep * r) if el == 1 else 1)
      wgrad(dpre, comm.xe, mlp.w1, split_k=_wgrad_split(m, h, ep * r) if el == 1 else 1)
      ev[8].record()
      comm.epoch["free"] += 1
      moe_ops.signal_multi(comm.done_flag_addrs("FFREE"))
      moe_ops.wait_counters(comm.fdx, ep, comm.epoch["dx"], comm.status)
      ev[9].record()
      dx = torch.empty_like(xd)
      moe_ops.combine_rows(comm.dxb_table, disp.expert, disp.slot, None, None, dx, g, s, e, c, k, h)
      ev[10].record()
      torch.cuda.synchronize()
      if it >= 2:
        for i, n in enumerate(names):
          total[n] += ev[i].elapsed_time(ev[i + 1]) / iters
  return total


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--path", default="p2p", choices=["p2p", "nccl"])
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--groups", type=int, default=32)
  ap.add_argument("--group-size", type=int, default=3152)
  ap.add_argument("--hidden", type=int, default=768)
  ap.add_argument("--mlp", type=int, default=3072)
  ap.add_argument("--experts", type=int, default=8)
  ap.add_argument("--capacity", type=int, default=832)
  ap.add_argument("--gemm-tflops", type=float, default=1418.0,
                  help="measured sustained cuBLAS bf16 throughput used as the compute roof")
  ap.add_argument("--link-gbs", type=float, default=770.0)
  ap.add_argument("--phases", action="store_true",
                  help="also time the launches of the peer-memory layer one by one")
  ap.add_argument("--separate-push", action="store_true",
                  help="launch the row push as a kernel of its own in front of the GEMM")
  args = ap.parse_args()
  os.environ["VMOE_B200_P2P"] = "1" if args.path == "p2p" else "0"
  if args.separate_push:
    os.environ["VMOE_B200_FUSED_PUSH"] = "0"
  from vmoe_b200.ops import moe_ops
  from vmoe_b200.parallel import mesh as mesh_lib
  from vmoe_b200.parallel.exchange import ExpertExchange
  mesh_lib.init_distributed()
  rank, world = dist.get_rank(), dist.get_world_size()
  mesh = mesh_lib.get_auto_logical_mesh(min(world, args.experts))
  ex = ExpertExchange.from_mesh(mesh)
  dev = torch.device("cuda", torch.cuda.current_device())
  g, s, h, m, e, c, k = (args.groups, args.group_size, args.hidden, args.mlp, args.experts,
                         args.capacity, 2)
  el = e // ex.size
  torch.manual_seed(rank)
  x = torch.randn(g, s, h, device=dev).bfloat16().requires_grad_()
  res = torch.randn(g, s, h, device=dev).bfloat16()
  logits = torch.randn(g, s, e, device=dev)
  dy = torch.randn(g, s, h, device=dev).bfloat16()
  mlp = _Mlp()
  mlp.w1 = (torch.randn(el, m, h, device=dev) * 0.02).requires_grad_()
  mlp.b1 = torch.zeros(el, m, device=dev).requires_grad_()
  mlp.w2 = (torch.randn(el, h, m, device=dev) * 0.02).requires_grad_()
  mlp.b2 = torch.zeros(el, h, device=dev).requires_grad_()
  gates = torch.softmax(logits, -1).requires_grad_()
  disp = moe_ops.FusedTopKDispatcher(gates, k, c, True, exchange=ex)
  # A leaf, so that repeated backward passes stop here instead of re-entering a freed graph.
  disp.combine_weights = disp.combine_weights.detach().requires_grad_()

  def fwd():
    return disp.apply_experts(mlp, x, residual=res)

  def fwd_bwd():
    for p in (mlp.w1, mlp.b1, mlp.w2, mlp.b2, x, disp.combine_weights):
      p.grad = None
    fwd().backward(dy)

  def timed(fn):
    for _ in range(2):
      fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
      fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())

  if args.phases and args.path == "p2p" and ex.size > 1:
    phases = layer_phases(moe_ops, disp, mlp, x, res, dy, ex, c, args.iters)
    t = torch.tensor(list(phases.values()), device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
      print(json.dumps({"phases_ms_max_over_ranks":
                        dict(zip(phases.keys(), [round(v, 4) for v in t.tolist()]))}))
  with torch.no_grad():
    t_fwd = timed(fwd)
  t_both = timed(fwd_bwd)
  if rank == 0:
    rows = e * g * c                       # expert rows processed per GPU
    flops_half = 2.0 * rows * h * m        # one GEMM
    wire = rows * h * 2 * (ex.size - 1) / ex.size  # bytes leaving this GPU per all-to-all
    t_compute = flops_half / (args.gemm_tflops * 1e12) * 1e3
    t_wire = wire / (args.link_gbs * 1e9) * 1e3
    roof_half = max(t_compute, t_wire)
    out = {"path": args.path, "n_gpus": world, "fwd_ms": t_fwd, "fwd_bwd_ms": t_both,
           "roofline_fwd_ms": 2 * roof_half, "fwd_fraction_of_roofline": 2 * roof_half / t_fwd,
           # backward: 2 dgrad + 2 wgrad GEMMs and two more all-to-alls
           "roofline_fwd_bwd_ms": 6 * t_compute if t_compute >= t_wire else 4 * t_wire + 2 * t_compute,
           "compute_ms_per_gemm": t_compute, "wire_ms_per_all_to_all": t_wire}
    out["fwd_bwd_fraction_of_roofline"] = out["roofline_fwd_bwd_ms"] / t_both
    print(json.dumps(out))
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
