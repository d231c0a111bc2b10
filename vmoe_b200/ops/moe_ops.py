"""GPU Top-K MoE layer in indices form: routing-plan kernel, row gather/combine kernels and the
expert GEMMs, tied together by one autograd Function.

Forward:  plan -> gather rows into the expert buffers (local memory, or pushed into the peer
GPUs' buffers when experts are sharded) -> batched GEMM1 + bias + GELU -> batched GEMM2 + bias
-> gate-weighted combine (+ residual). Backward mirrors it: the backward of combine is a
gather (fused with the gate-gradient dot products) and the backward of dispatch is a combine
with unit weights.

Semantics are those of the reference's dispatchers (``vmoe/moe.py:148-209``) with the Top-K
plan of ``vmoe/moe.py:547-652``; tests compare against ``vmoe_b200.moe`` on CPU.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from vmoe_b200 import moe as moe_core
from vmoe_b200.ops import _lib
from vmoe_b200.ops.functional import (_grad_target, _wgrad_split, bf16_shadow, bias_grad,
                                       wgrad)
from vmoe_b200.ops.gemm import ACT_GELU, gemm
from vmoe_b200.parallel.exchange import ExpertExchange, LOCAL_EXCHANGE

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64


def routing_plan(gates: torch.Tensor, num_selected_experts: int, capacity: int,
                 batch_priority: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
  """Runs the routing-plan kernel on ``gates (G, S, E)`` fp32 (CUDA).

  Returns int32 tensors ``expert (G, S, K)``, ``slot (G, S, K)`` and ``slot_pair (G, E, C)``.
  """
  assert gates.is_cuda and gates.dtype == torch.float32 and gates.dim() == 3
  gates = gates.contiguous()
  g, s, e = gates.shape
  k = num_selected_experts
  expert = torch.empty(g, s, k, dtype=torch.int32, device=gates.device)
  slot = torch.empty(g, s, k, dtype=torch.int32, device=gates.device)
  slot_pair = torch.empty(g, e, capacity, dtype=torch.int32, device=gates.device)
  rc = _lib.lib().vmoe_routing_plan(
      _vp(gates.data_ptr()), _vp(expert.data_ptr()), _vp(slot.data_ptr()),
      _vp(slot_pair.data_ptr()), _i64(g), _i64(s), _i64(e), _i64(k), _i64(capacity),
      ctypes.c_int32(int(batch_priority)), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_routing_plan")
  _lib.count_launch()
  return expert, slot, slot_pair


def _base_table(buf: torch.Tensor) -> torch.Tensor:
  """Device table of per-expert base addresses for a local ``(E, rows, H)`` buffer."""
  e = buf.shape[0]
  addrs = [buf.data_ptr() + i * buf.stride(0) * buf.element_size() for i in range(e)]
  return torch.tensor(addrs, dtype=torch.int64, device=buf.device)


_TABLE_CACHE: dict = {}


def base_table(buf: torch.Tensor) -> torch.Tensor:
  key = (buf.data_ptr(), buf.shape[0], buf.stride(0), buf.device)
  t = _TABLE_CACHE.get(key)
  if t is None:
    if len(_TABLE_CACHE) > 4096:
      _TABLE_CACHE.clear()
    t = _base_table(buf)
    _TABLE_CACHE[key] = t
  return t


def gather_rows(x, slot_pair, weight, table, g, s, e, c, k, h):
  rc = _lib.lib().vmoe_moe_gather_rows(
      _vp(x.data_ptr()), _vp(slot_pair.data_ptr()), _vp(_lib.ptr(weight)), _vp(table.data_ptr()),
      _i64(g), _i64(s), _i64(e), _i64(c), _i64(k), _i64(h), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_gather_rows")
  _lib.count_launch()


def combine_rows(table, expert, slot, weight, residual, out, g, s, e, c, k, h, status=None):
  rc = _lib.lib().vmoe_moe_combine_rows(
      _vp(table.data_ptr()), _vp(expert.data_ptr()), _vp(slot.data_ptr()), _vp(_lib.ptr(weight)),
      _vp(_lib.ptr(residual)), _vp(out.data_ptr()), _i64(g), _i64(s), _i64(e), _i64(c), _i64(k),
      _i64(h), _vp(_lib.ptr(status)), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_combine_rows")
  _lib.count_launch()


def combine_bwd(dy, slot_pair, gate, ytable, dtable, dgate, g, s, e, c, k, h):
  rc = _lib.lib().vmoe_moe_combine_bwd(
      _vp(dy.data_ptr()), _vp(slot_pair.data_ptr()), _vp(gate.data_ptr()), _vp(ytable.data_ptr()),
      _vp(dtable.data_ptr()), _vp(dgate.data_ptr()), _i64(g), _i64(s), _i64(e), _i64(c), _i64(k),
      _i64(h), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_combine_bwd")
  _lib.count_launch()


def _a2a_to_experts(buf: torch.Tensor, ex: ExpertExchange) -> torch.Tensor:
  """NCCL baseline exchange ``(E, R, H) -> (E_local, ep*R, H)`` (no autograd)."""
  if ex.size == 1:
    return buf
  e, r, h = buf.shape
  el = e // ex.size
  recv = torch.empty_like(buf)
  dist.all_to_all_single(recv, buf, group=ex.group)
  if el == 1:
    return recv.reshape(1, ex.size * r, h)
  return recv.reshape(ex.size, el, r, h).transpose(0, 1).reshape(el, ex.size * r, h)


def _a2a_from_experts(buf: torch.Tensor, ex: ExpertExchange) -> torch.Tensor:
  """Inverse of ``_a2a_to_experts``: ``(E_local, ep*R, H) -> (E, R, H)``."""
  if ex.size == 1:
    return buf
  el, rows, h = buf.shape
  r = rows // ex.size
  send = buf if el == 1 else buf.reshape(el, ex.size, r, h).transpose(0, 1).contiguous()
  recv = torch.empty(ex.size * el, r, h, dtype=buf.dtype, device=buf.device)
  dist.all_to_all_single(recv, send.reshape(ex.size * el, r, h), group=ex.group)
  return recv


def push_rows(x, slot_pair, weight, dst_table, flag_table, ybuf_table, dgate, g, s, e, c, k, h,
              el, ep, rank):
  rc = _lib.lib().vmoe_moe_push_rows(
      _vp(x.data_ptr()), _vp(slot_pair.data_ptr()), _vp(_lib.ptr(weight)),
      _vp(dst_table.data_ptr()), _vp(_lib.ptr(flag_table)), _vp(_lib.ptr(ybuf_table)),
      _vp(_lib.ptr(dgate)), _i64(g), _i64(s), _i64(e), _i64(c), _i64(k), _i64(h), _i64(el),
      _i64(ep), _i64(rank), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_push_rows")
  _lib.count_launch()


def push_args(x, slot_pair, weight, dst_table, flag_table, ybuf_table, dgate, g, s, e, c, k, h,
              el, ep, rank) -> "_lib.PushArgs":
  """Arguments of the row push for the GEMM's push CTAs (``gemm(..., push=...)``) or for
  ``push_rows_bulk``. The tensors must stay alive until the launch that uses them is enqueued."""
  a = _lib.PushArgs()
  a.x, a.slot_pair, a.weight = x.data_ptr(), slot_pair.data_ptr(), _lib.ptr(weight)
  a.dst_base, a.flag_base = dst_table.data_ptr(), _lib.ptr(flag_table)
  a.ybuf_base, a.dgate = _lib.ptr(ybuf_table), _lib.ptr(dgate)
  a.groups, a.s, a.e, a.c, a.k, a.h = g, s, e, c, k, h
  a.experts_per_rank, a.ep, a.rank = el, ep, rank
  return a


def push_rows_bulk(args: "_lib.PushArgs", ctas: int = 37, status=None):
  """The bulk-copy row push as a launch of its own (``csrc/moe_push.cuh``)."""
  rc = _lib.lib().vmoe_moe_push_rows_bulk(ctypes.byref(args), ctypes.c_int32(ctas),
                                          _vp(_lib.ptr(status)), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_moe_push_rows_bulk")
  _lib.count_launch()


def signal_multi(addrs, value: int = 1):
  arr = (ctypes.c_uint64 * len(addrs))(*[int(a) for a in addrs])
  rc = _lib.lib().vmoe_signal_multi(arr, ctypes.c_int32(len(addrs)), ctypes.c_uint32(value),
                                    _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_signal_multi")
  _lib.count_launch()


def signal(addr: int, value: int = 1):
  rc = _lib.lib().vmoe_signal(_vp(addr), ctypes.c_uint32(value), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_signal")
  _lib.count_launch()


def wait_counters(counters: torch.Tensor, n: int, target: int, status=None, limit_cycles: int = 0):
  rc = _lib.lib().vmoe_wait_counters(_vp(counters.data_ptr()), ctypes.c_int32(n),
                                     ctypes.c_uint32(target & 0xFFFFFFFF), _vp(_lib.ptr(status)),
                                     _i64(limit_cycles), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_wait_counters")
  _lib.count_launch()


class LayerComm:
  """Symmetric buffers and address tables of one MoE layer for the peer-to-peer path.

  Per rank: XE / DYE ``(E_local, ep*R, H)`` receive the rows dispatched to the local experts
  (forward / backward), YB / DXB ``(E, R, H)`` receive the expert outputs coming home, plus
  per-tile arrival counters for XE / DYE and per-source completion counters for YB / DXB.
  ``R = G*C`` rows per (expert, source rank).
  """

  def __init__(self, exchange: ExpertExchange, e: int, r: int, h: int, device):
    from vmoe_b200.parallel import symm
    ep = exchange.size
    self.ep, self.e, self.el, self.r, self.h = ep, e, e // ep, r, h
    self.tiles = (ep * r + 127) // 128
    blk = e * r * h * 2
    fl_tiles = (self.el * self.tiles * 4 + 255) // 256 * 256
    fl_src = 256
    # Canary words before, between and after the four data regions and after the counters: a
    # peer's store that runs past its block lands in one of them (``check_guards``).
    gb = symm.GUARD_BYTES
    blk_g = blk + gb
    fl0 = gb + 4 * blk_g
    self.off = {"XE": gb, "YB": gb + blk_g, "DYE": gb + 2 * blk_g, "DXB": gb + 3 * blk_g,
                "FX": fl0, "FDY": fl0 + fl_tiles, "FY": fl0 + 2 * fl_tiles,
                "FDX": fl0 + 2 * fl_tiles + fl_src,
                "FFREE": fl0 + 2 * fl_tiles + 2 * fl_src}
    end = fl0 + 2 * fl_tiles + 3 * fl_src
    self.buf = symm.SymmetricBuffer(end + gb, exchange.group, device)
    self.buf.set_guards([0] + [self.off[k] + blk for k in ("XE", "YB", "DYE", "DXB")] + [end])
    self.rank = self.buf.rank
    b = self.buf
    self.xe = b.local(self.off["XE"], (self.el, ep * r, h), torch.bfloat16)
    self.dye = b.local(self.off["DYE"], (self.el, ep * r, h), torch.bfloat16)
    self.yb = b.local(self.off["YB"], (e, r, h), torch.bfloat16)
    self.dxb = b.local(self.off["DXB"], (e, r, h), torch.bfloat16)
    self.fx = b.local(self.off["FX"], (self.el * self.tiles,), torch.int32)
    self.fdy = b.local(self.off["FDY"], (self.el * self.tiles,), torch.int32)
    self.fy = b.local(self.off["FY"], (64,), torch.int32)
    self.fdx = b.local(self.off["FDX"], (64,), torch.int32)
    # ffree[src]: backward passes after which rank src no longer reads what this rank pushed
    # into its XE / DYE buffers; the next forward waits for it instead of a group barrier.
    self.ffree = b.local(self.off["FFREE"], (64,), torch.int32)
    self.status = torch.zeros(1, dtype=torch.int32, device=device)
    self.done = torch.zeros(2, dtype=torch.int32, device=device)  # GEMM completion tickets
    self.epoch = {"x": 0, "y": 0, "dy": 0, "dx": 0, "free": 0}

    def table(data_key, flag_key):
      dst, flg = [], []
      for ee in range(e):
        owner, loc = ee // self.el, ee % self.el
        dst.append(b.ptrs[owner] + self.off[data_key] + (loc * ep + self.rank) * r * h * 2)
        flg.append(b.ptrs[owner] + self.off[flag_key] + loc * self.tiles * 4)
      mk = lambda v: torch.tensor(v, dtype=torch.int64, device=device)
      return mk(dst), mk(flg)

    self.push_x, self.flag_x = table("XE", "FX")
    self.push_dy, self.flag_dy = table("DYE", "FDY")
    self.yb_table = _base_table(self.yb)
    self.dxb_table = _base_table(self.dxb)
    self.mt_offset = (self.rank * r) // 128

  def check_guards(self) -> None:
    """Raises ``symm.BufferOverrun`` if something wrote between or past the regions of this
    rank's buffer (synchronises with the device)."""
    self.buf.check_guards("expert exchange buffers")

  def home_out(self, key: str, src: int) -> torch.Tensor:
    """View of source rank ``src``'s YB/DXB slice that receives this rank's experts."""
    off = self.off[key] + self.rank * self.el * self.r * self.h * 2
    return self.buf.peer(src, off, (self.el, self.r, self.h), torch.bfloat16)

  def done_flag_addr(self, key: str, src: int) -> int:
    return self.buf.ptrs[src] + self.off[key] + self.rank * 4

  def done_flag_addrs(self, key: str):
    """This rank's completion flag on every rank of the group, own rank first: the flag whose
    owner is this GPU is bumped without crossing the link."""
    return [self.done_flag_addr(key, (self.rank + i) % self.ep) for i in range(self.ep)]


_LAYER_COMMS: dict = {}


def layer_comm(owner, exchange: ExpertExchange, e: int, r: int, h: int, device) -> LayerComm:
  """The ``LayerComm`` of a MoE layer (``owner`` identifies the layer), created on first use.
  Creation is a collective: all ranks of the expert group must reach it in the same order."""
  key = (id(owner), e, r, h)
  comm = _LAYER_COMMS.get(key)
  if comm is None:
    comm = LayerComm(exchange, e, r, h, device)
    _LAYER_COMMS[key] = comm
  return comm


def p2p_enabled(exchange: ExpertExchange) -> bool:
  import os
  from vmoe_b200.parallel import symm
  return (exchange.size > 1 and os.environ.get("VMOE_B200_P2P", "1") != "0" and symm.available()
          and dist.is_initialized() and dist.get_backend(exchange.group) == "nccl")


class _P2PMoeFn(torch.autograd.Function):
  """Expert-parallel MoE layer over NVLink peer memory (no NCCL all-to-all).

  Forward: push rows into the owners' XE buffers (arrival counters) -> GEMM1 consumes tiles as
  they arrive -> GEMM2 per source rank stores its output tiles into that rank's YB buffer and
  bumps its completion counter -> combine at home once all sources are complete.
  """

  @staticmethod
  def forward(ctx, x, gate, w1, b1, w2, b2, residual, expert, slot, slot_pair, capacity,
              exchange, comm):
    g, s, h = x.shape
    k = expert.shape[-1]
    e = slot_pair.shape[1]
    c = capacity
    r = g * c
    ep, el, rank = comm.ep, comm.el, comm.rank
    x = x.contiguous()
    gate = gate.contiguous().float()
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    m = w1.shape[1]
    # Every peer is past the reads of what this rank pushed last time (its previous backward
    # pass through this layer): a counter wait that is normally satisfied long before, instead
    # of a barrier over the group.
    if comm.epoch["free"] > 0:
      wait_counters(comm.ffree, ep, comm.epoch["free"], comm.status)
    for key in ("x", "y"):
      comm.epoch[key] += 1
    need = any(ctx.needs_input_grad)
    pre = torch.empty(el, ep * r, m, dtype=torch.bfloat16, device=x.device) if need else None
    pargs = push_args(x, slot_pair, None, comm.push_x, comm.flag_x, None, None, g, s, e, c, k, h,
                      el, ep, rank)
    # Dispatch + first expert GEMM in one launch: two warps of every CTA send this rank's rows
    # to the expert owners while the other warps multiply the tiles that have arrived.
    hid = gemm(comm.xe, w1h, bias=b1, act=ACT_GELU, out_pre=pre, out_pre_is_grad=True,
               a_ready=comm.fx, a_ready_epoch=comm.epoch["x"], status=comm.status,
               mt_offset=comm.mt_offset, push=pargs)
    if r % 32 == 0 and ep <= 8:
      # One GEMM over all rows; every 32-row output box is TMA-stored straight into the home
      # buffer of the rank its rows came from, and the last CTA to finish tells every home rank.
      # mt_offset: rank r starts with the rows of source r, so at any moment the ranks store to
      # different destinations instead of all converging on the same GPU's link.
      gemm(hid, w2h, bias=b2, out_multi=[comm.home_out("YB", src) for src in range(ep)],
           mt_offset=comm.mt_offset, signal_flags=comm.done_flag_addrs("FY"),
           done_counter=comm.done[0:1])
    else:
      for i in range(ep):
        src = (rank + i) % ep
        gemm(hid[:, src * r:(src + 1) * r], w2h, bias=b2, out=comm.home_out("YB", src))
        signal(comm.done_flag_addr("FY", src))
    wait_counters(comm.fy, ep, comm.epoch["y"], comm.status)
    out = torch.empty_like(x)
    combine_rows(comm.yb_table, expert, slot, gate, residual, out, g, s, e, c, k, h)
    ctx.save_for_backward(gate, w1, w2, expert, slot, slot_pair, pre, hid)
    ctx.dims = (g, s, e, c, k, h, m)
    ctx.comm = comm
    ctx.biases = (b1, b2)
    ctx.has_res = residual is not None
    return out

  @staticmethod
  def backward(ctx, dy):
    gate, w1, w2, expert, slot, slot_pair, pre, hid = ctx.saved_tensors
    g, s, e, c, k, h, m = ctx.dims
    comm = ctx.comm
    ep, el, rank, r = comm.ep, comm.el, comm.rank, g * c
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    dy = dy.contiguous()
    dev = dy.device
    for key in ("dy", "dx"):
      comm.epoch[key] += 1
    dgate = torch.zeros(g, s, k, dtype=torch.float32, device=dev)
    pargs = push_args(dy, slot_pair, gate, comm.push_dy, comm.flag_dy, comm.yb_table, dgate, g, s,
                      e, c, k, h, el, ep, rank)
    b1, b2 = ctx.biases
    tgt = _grad_target(b1)
    db1 = tgt if tgt is not None else torch.zeros(el, m, dtype=torch.float32, device=dev)
    # Backward of combine (gate-scaled dy rows and the gate gradients) pushed by two warps of
    # every CTA of the hidden-gradient GEMM, which consumes the rows as they arrive.
    dpre = gemm(comm.dye, w2h, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True, colsum=db1,
                a_ready=comm.fdy, a_ready_epoch=comm.epoch["dy"], status=comm.status,
                mt_offset=comm.mt_offset, push=pargs)
    if tgt is not None:
      db1 = None
    # dX first: its tiles travel home over NVLink while the weight-gradient GEMMs below run.
    if r % 32 == 0 and ep <= 8:
      gemm(dpre, w1h, b_mn_major=True,
           out_multi=[comm.home_out("DXB", src) for src in range(ep)], mt_offset=comm.mt_offset,
           signal_flags=comm.done_flag_addrs("FDX"), done_counter=comm.done[1:2])
    else:
      for i in range(ep):
        src = (rank + i) % ep
        gemm(dpre[:, src * r:(src + 1) * r], w1h, b_mn_major=True,
             out=comm.home_out("DXB", src))
        signal(comm.done_flag_addr("FDX", src))
    # Every tile of dye has arrived once the dpre GEMM above has run.
    db2 = bias_grad(comm.dye, b2)
    # One expert per GPU leaves only 72 output tiles: split the long contraction over two CTAs.
    dw2 = wgrad(comm.dye, hid, w2, split_k=_wgrad_split(h, m, ep * r) if el == 1 else 1)
    dw1 = wgrad(dpre, comm.xe, w1, split_k=_wgrad_split(m, h, ep * r) if el == 1 else 1)
    # The rows that the peers pushed into XE / DYE have been read for the last time.
    comm.epoch["free"] += 1
    signal_multi(comm.done_flag_addrs("FFREE"))
    wait_counters(comm.fdx, ep, comm.epoch["dx"], comm.status)
    dx = torch.empty(g, s, h, dtype=torch.bfloat16, device=dev)
    combine_rows(comm.dxb_table, expert, slot, None, None, dx, g, s, e, c, k, h)
    d_res = dy if ctx.has_res else None
    return dx, dgate, dw1, db1, dw2, db2, d_res, None, None, None, None, None, None


class _FusedMoeFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, gate, w1, b1, w2, b2, residual, expert, slot, slot_pair, capacity,
              exchange):
    g, s, h = x.shape
    k = expert.shape[-1]
    e = slot_pair.shape[1]
    c = capacity
    x = x.contiguous()
    gate = gate.contiguous().float()
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    m = w1.shape[1]
    # Dispatch: expert buffers (E, G*C, H), rows ordered (group, slot).
    xbuf = torch.empty(e, g * c, h, dtype=torch.bfloat16, device=x.device)
    gather_rows(x, slot_pair, None, base_table(xbuf), g, s, e, c, k, h)
    xe = _a2a_to_experts(xbuf, exchange)
    need = any(ctx.needs_input_grad)
    pre = torch.empty(xe.shape[0], xe.shape[1], m, dtype=torch.bfloat16,
                      device=x.device) if need else None
    hid = gemm(xe, w1h, bias=b1, act=ACT_GELU, out_pre=pre, out_pre_is_grad=True)
    ye = gemm(hid, w2h, bias=b2)
    ybuf = _a2a_from_experts(ye, exchange)
    out = torch.empty_like(x)
    combine_rows(base_table(ybuf), expert, slot, gate, residual, out, g, s, e, c, k, h)
    ctx.save_for_backward(gate, w1, w2, expert, slot, slot_pair, xe, pre, hid, ybuf)
    ctx.dims = (g, s, e, c, k, h, m)
    ctx.biases = (b1, b2)
    ctx.exchange = exchange
    ctx.has_res = residual is not None
    return out

  @staticmethod
  def backward(ctx, dy):
    gate, w1, w2, expert, slot, slot_pair, xe, pre, hid, ybuf = ctx.saved_tensors
    g, s, e, c, k, h, m = ctx.dims
    ex = ctx.exchange
    w1h, w2h = bf16_shadow(w1), bf16_shadow(w2)
    dy = dy.contiguous()
    dev = dy.device
    # Backward of combine: d(ybuf) rows and gate gradients in one pass.
    dybuf = torch.empty(e, g * c, h, dtype=torch.bfloat16, device=dev)
    dgate = torch.zeros(g, s, k, dtype=torch.float32, device=dev)
    combine_bwd(dy, slot_pair, gate, base_table(ybuf), base_table(dybuf), dgate, g, s, e, c, k, h)
    dye = _a2a_to_experts(dybuf, ex)
    el = dye.shape[0]
    b1, b2 = ctx.biases
    db2 = bias_grad(dye, b2)
    dw2 = wgrad(dye, hid, w2)
    tgt = _grad_target(b1)
    db1 = tgt if tgt is not None else torch.zeros(el, m, dtype=torch.float32, device=dev)
    dpre = gemm(dye, w2h, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True, colsum=db1)
    if tgt is not None:
      db1 = None
    dw1 = wgrad(dpre, xe, w1)
    dxe = gemm(dpre, w1h, b_mn_major=True)
    dxbuf = _a2a_from_experts(dxe, ex)
    # Backward of dispatch: unit-weight combine.
    dx = torch.empty(g, s, h, dtype=torch.bfloat16, device=dev)
    combine_rows(base_table(dxbuf), expert, slot, None, None, dx, g, s, e, c, k, h)
    d_res = dy if ctx.has_res else None
    return dx, dgate, dw1, db1, dw2, db2, d_res, None, None, None, None, None


class FusedTopKDispatcher(moe_core.BaseDispatcher):
  """Top-K dispatcher for CUDA bf16 activations backed by the kernels of this module.

  It also implements the generic ``dispatch`` / ``combine`` protocol (through the PyTorch
  indices dispatcher) so code written against ``BaseDispatcher`` keeps working, but the MoE
  block calls ``apply_experts`` which runs the whole layer in one autograd node.
  """

  def __init__(self, gates: torch.Tensor, num_selected_experts: int, capacity: int,
               batch_priority: bool, exchange: ExpertExchange = LOCAL_EXCHANGE):
    self.gates = gates
    self.capacity = capacity
    self.num_experts = gates.shape[-1]
    self.exchange = exchange
    self.expert, self.slot, self.slot_pair = routing_plan(
        gates.detach().float(), num_selected_experts, capacity, batch_priority)
    # Differentiable gate values of the selected experts (raw softmax, not renormalised).
    self.combine_weights = torch.gather(gates, -1, self.expert.long())

  @property
  def indices(self) -> torch.Tensor:
    return torch.stack([self.expert, self.slot], dim=-1)

  def _generic(self) -> moe_core.ExpertIndicesDispatcher:
    return moe_core.ExpertIndicesDispatcher(
        indices=self.indices, combine_weights=self.combine_weights,
        num_experts=self.num_experts, capacity=self.capacity, exchange=self.exchange)

  def dispatch(self, data):
    return self._generic().dispatch(data)

  def combine(self, data):
    return self._generic().combine(data)

  def apply_experts(self, mlp, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
    if mlp.training and getattr(mlp, "dropout_rate", 0.0) > 0:
      out = moe_core.sparse_moe_apply(mlp, self._generic(), x)
      return out if residual is None else out + residual
    if p2p_enabled(self.exchange):
      g, s, h = x.shape
      comm = layer_comm(mlp, self.exchange, self.num_experts, g * self.capacity, h, x.device)
      return _P2PMoeFn.apply(x, self.combine_weights, mlp.w1, mlp.b1, mlp.w2, mlp.b2, residual,
                             self.expert, self.slot, self.slot_pair, self.capacity,
                             self.exchange, comm)
    return _FusedMoeFn.apply(x, self.combine_weights, mlp.w1, mlp.b1, mlp.w2, mlp.b2, residual,
                             self.expert, self.slot, self.slot_pair, self.capacity,
                             self.exchange)


def experts_choose_plan(gates: torch.Tensor, capacity: int):
  """Runs the experts-choose plan kernel on ``gates (G, S, E)`` fp32 (CUDA, S <= 4096).

  Returns int32 ``slot (G, S, E)`` (rank of the item in the expert's order, ``capacity`` if the
  expert did not take it) and ``slot_pair (G, E, C)`` (``item * E + expert``, -1 for empty)."""
  assert gates.is_cuda and gates.dtype == torch.float32 and gates.dim() == 3
  gates = gates.contiguous()
  g, s, e = gates.shape
  slot = torch.empty(g, s, e, dtype=torch.int32, device=gates.device)
  slot_pair = torch.empty(g, e, capacity, dtype=torch.int32, device=gates.device)
  rc = _lib.lib().vmoe_experts_choose_plan(
      _vp(gates.data_ptr()), _vp(slot.data_ptr()), _vp(slot_pair.data_ptr()), _i64(g), _i64(s),
      _i64(e), _i64(capacity), _vp(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_experts_choose_plan")
  _lib.count_launch()
  return slot, slot_pair


EXPERTS_CHOOSE_MAX_ITEMS = 4096


class FusedTopItemsDispatcher(FusedTopKDispatcher):
  """"Experts choose" dispatcher (every expert takes its ``capacity`` best items of a group;
  ``vmoe/moe.py:655-694``) on the kernels of the Top-K layer: in indices form it is "every item
  has E choices, choice j is expert j, taken or not", so the plan kernel fills the same tables
  and the row movers, the peer-memory exchange and the combine kernels are shared."""

  def __init__(self, gates: torch.Tensor, capacity: int,
               exchange: ExpertExchange = LOCAL_EXCHANGE):
    self.gates = gates
    self.capacity = capacity
    self.num_experts = gates.shape[-1]
    self.exchange = exchange
    g, s, e = gates.shape
    self.slot, self.slot_pair = experts_choose_plan(gates.detach().float(), capacity)
    self.expert = torch.arange(e, dtype=torch.int32, device=gates.device).expand(g, s, e)
    self.expert = self.expert.contiguous()
    self.combine_weights = gates  # choice j of an item is weighted by its gate for expert j

  def metrics(self) -> dict:
    """Per-group monitoring values of the reference (``vmoe/moe.py:676-693``)."""
    g, s, e = self.gates.shape
    taken = self.slot < self.capacity                      # (G, S, E)
    per_item = taken.sum(dim=-1).to(torch.int32)           # (G, S)
    gates = self.gates.detach()
    sel = torch.where(taken, gates, torch.full_like(gates, float("inf")))
    sel_max = torch.where(taken, gates, torch.full_like(gates, float("-inf")))
    out = {
        "num_experts_per_item_min": per_item.min(dim=1).values,
        "num_experts_per_item_max": per_item.max(dim=1).values,
        "min_selected_gate": sel.amin(dim=(1, 2)),
        "max_selected_gate": sel_max.amax(dim=(1, 2)),
    }
    import math
    log2e = int(math.log2(e))
    for t in [2 ** i for i in range(log2e + 1)] + [e]:
      out[f"ratio_processed_items_by_at_least_{t}_experts"] = (
          (per_item >= t).sum(dim=1).to(gates.dtype) / s)
    return out
