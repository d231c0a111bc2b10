"""Expert-parallel exchange of DENSE slot buffers over NVLink peer memory, fused with the expert
GEMMs: the all-to-alls around the experts of a Soft MoE layer (and of any dispatcher whose
dispatch is an einsum that fills every (expert, slot) row of every group).

The dispatch einsum leaves ``(G, E*C, H)`` slot rows on every rank. Their way to the experts'
owners and back is the one of the Top-K layer (``ops/moe_ops.py``) with an identity routing
table: two warps of every CTA of the first expert GEMM push this rank's slot rows into the
owners' buffers while the other warps multiply the tiles that have arrived; the second expert
GEMM stores its output tiles straight into the home ranks' buffers and signals them; the
combine einsum then runs at home. Backward mirrors it (slot gradients pushed under the
hidden-gradient GEMM, the input-gradient GEMM storing home while the weight gradients run).

Stands in for the two sharding constraints that XLA lowers to all-to-alls around the experts
(``vmoe/moe.py:488-519``) on the Soft MoE path (``vmoe/projects/soft_moe/router.py:91-100``).
"""
from __future__ import annotations

import torch

from vmoe_b200.ops import moe_ops
from vmoe_b200.ops.functional import (_grad_target, _wgrad_split, bf16_shadow, bias_grad, wgrad)
from vmoe_b200.ops.gemm import ACT_GELU, gemm

_IDENTITY: dict = {}


def _identity_slots(g: int, e: int, c: int, device) -> torch.Tensor:
  """``slot_pair[g, e, c] = e * c_total + c``: buffer slot (e, c) of group g holds row
  ``e*C + c`` of that group (one choice per row, so pair == row)."""
  key = (g, e, c, str(device))
  t = _IDENTITY.get(key)
  if t is None:
    if len(_IDENTITY) > 64:
      _IDENTITY.clear()
    t = torch.arange(e * c, dtype=torch.int32, device=device).reshape(1, e, c).expand(g, e, c)
    t = t.contiguous()
    _IDENTITY[key] = t
  return t


def applicable(exchange, mlp, groups: int, num_experts: int, capacity: int,
               data: torch.Tensor) -> bool:
  """Peer memory is available, the payload is bf16 on CUDA, every (expert, source rank) block
  of ``groups * capacity`` rows is a whole number of 32-row store boxes, at most 8 ranks, and
  the experts apply no dropout."""
  if not moe_ops.p2p_enabled(exchange):
    return False
  if mlp.training and getattr(mlp, "dropout_rate", 0.0) > 0:
    return False
  r = groups * capacity
  return (data.is_cuda and data.dtype == torch.bfloat16 and data.shape[-1] % 8 == 0 and
          r % 32 == 0 and exchange.size <= 8 and num_experts % exchange.size == 0 and
          all(hasattr(mlp, n) for n in ("w1", "b1", "w2", "b2")))


class _DenseP2PFn(torch.autograd.Function):
  """``xs (G, E*C, H)`` slot inputs on their home rank -> ``(G, E*C, H)`` slot outputs of the
  experts ``w1 (E_local, M, H)``, ``w2 (E_local, H, M)`` held by the ranks of the group."""

  @staticmethod
  def forward(ctx, xs, w1, b1, w2, b2, e, c, comm):
    g, n, h = xs.shape
    r = g * c
    ep, el, rank = comm.ep, comm.el, comm.rank
    xs = xs.contiguous()
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    m = w1.shape[1]
    ident = _identity_slots(g, e, c, xs.device)
    if comm.epoch["free"] > 0:
      moe_ops.wait_counters(comm.ffree, ep, comm.epoch["free"], comm.status)
    for key in ("x", "y"):
      comm.epoch[key] += 1
    need = any(ctx.needs_input_grad)
    pre = torch.empty(el, ep * r, m, dtype=torch.bfloat16, device=xs.device) if need else None
    pargs = moe_ops.push_args(xs, ident, None, comm.push_x, comm.flag_x, None, None, g, n, e, c,
                              1, h, el, ep, rank)
    hid = gemm(comm.xe, w1h, bias=b1, act=ACT_GELU, out_pre=pre, out_pre_is_grad=True,
               a_ready=comm.fx, a_ready_epoch=comm.epoch["x"], status=comm.status,
               mt_offset=comm.mt_offset, push=pargs)
    gemm(hid, w2h, bias=b2, out_multi=[comm.home_out("YB", src) for src in range(ep)],
         mt_offset=comm.mt_offset, signal_flags=comm.done_flag_addrs("FY"),
         done_counter=comm.done[0:1])
    moe_ops.wait_counters(comm.fy, ep, comm.epoch["y"], comm.status)
    # Home buffer (E, G*C, H) -> (G, E*C, H), the layout of the combine einsum.
    ys = comm.yb.reshape(e, g, c, h).permute(1, 0, 2, 3).reshape(g, n, h).contiguous()
    ctx.save_for_backward(w1, w2, pre, hid)
    ctx.dims = (g, n, e, c, h, m)
    ctx.comm = comm
    ctx.biases = (b1, b2)
    return ys

  @staticmethod
  def backward(ctx, dys):
    w1, w2, pre, hid = ctx.saved_tensors
    g, n, e, c, h, m = ctx.dims
    comm = ctx.comm
    ep, el, rank, r = comm.ep, comm.el, comm.rank, g * c
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    dys = dys.contiguous()
    dev = dys.device
    ident = _identity_slots(g, e, c, dev)
    for key in ("dy", "dx"):
      comm.epoch[key] += 1
    pargs = moe_ops.push_args(dys, ident, None, comm.push_dy, comm.flag_dy, None, None, g, n, e,
                              c, 1, h, el, ep, rank)
    b1, b2 = ctx.biases
    tgt = _grad_target(b1)
    db1 = tgt if tgt is not None else torch.zeros(el, m, dtype=torch.float32, device=dev)
    dpre = gemm(comm.dye, w2h, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True, colsum=db1,
                a_ready=comm.fdy, a_ready_epoch=comm.epoch["dy"], status=comm.status,
                mt_offset=comm.mt_offset, push=pargs)
    if tgt is not None:
      db1 = None
    gemm(dpre, w1h, b_mn_major=True,
         out_multi=[comm.home_out("DXB", src) for src in range(ep)], mt_offset=comm.mt_offset,
         signal_flags=comm.done_flag_addrs("FDX"), done_counter=comm.done[1:2])
    db2 = bias_grad(comm.dye, b2)
    dw2 = wgrad(comm.dye, hid, w2, split_k=_wgrad_split(h, m, ep * r) if el == 1 else 1)
    dw1 = wgrad(dpre, comm.xe, w1, split_k=_wgrad_split(m, h, ep * r) if el == 1 else 1)
    comm.epoch["free"] += 1
    moe_ops.signal_multi(comm.done_flag_addrs("FFREE"))
    moe_ops.wait_counters(comm.fdx, ep, comm.epoch["dx"], comm.status)
    dxs = comm.dxb.reshape(e, g, c, h).permute(1, 0, 2, 3).reshape(g, n, h).contiguous()
    return dxs, dw1, db1, dw2, db2, None, None, None


def expert_exchange_and_mlp(mlp, exchange, xs: torch.Tensor, num_experts: int,
                            capacity: int) -> torch.Tensor:
  """Slot rows ``xs (G, E*C, H)`` through the experts of the whole group and back."""
  g, n, h = xs.shape
  comm = moe_ops.layer_comm(mlp, exchange, num_experts, g * capacity, h, xs.device)
  return _DenseP2PFn.apply(xs, mlp.w1, mlp.b1, mlp.w2, mlp.b2, num_experts, capacity, comm)
