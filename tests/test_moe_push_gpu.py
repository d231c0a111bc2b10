"""The bulk-copy row push (``csrc/moe_push.cuh``) alone and as the push warps inside the CTAs
of the expert GEMM, on one GPU: the destination tables point at local buffers laid out as the expert owners' buffers
would be, so the row movement, the zero rows of empty slots, the tile counters, the gate scaling
and the gate gradients can be compared with the plain gather formulation in PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
  pytest.skip("needs a GPU", allow_module_level=True)

from vmoe_b200.ops import gemm as G  # noqa: E402
from vmoe_b200.ops import moe_ops  # noqa: E402


def _setup(g, s, e, k, c, h, ep, rank, seed=0):
  """Routing plan and the buffers of a fake expert group of ``ep`` ranks seen from ``rank``:
  every owner's (el, ep * R, h) row buffer and tile counters live on this GPU."""
  torch.manual_seed(seed)
  dev = "cuda"
  el, r = e // ep, g * c
  x = torch.randn(g, s, h, device=dev).bfloat16()
  gates = torch.softmax(torch.randn(g, s, e, device=dev), -1)
  expert, slot, slot_pair = moe_ops.routing_plan(gates, k, c, True)
  tiles = (ep * r + 127) // 128
  bufs = [torch.full((el, ep * r, h), 7.0, device=dev, dtype=torch.bfloat16) for _ in range(ep)]
  flags = [torch.zeros(el * tiles, device=dev, dtype=torch.int32) for _ in range(ep)]
  dst, flg = [], []
  for ee in range(e):
    owner, loc = ee // el, ee % el
    dst.append(bufs[owner].data_ptr() + (loc * ep + rank) * r * h * 2)
    flg.append(flags[owner].data_ptr() + loc * tiles * 4)
  mk = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)
  return x, gates, expert, slot, slot_pair, bufs, flags, mk(dst), mk(flg), tiles


def _expected_rows(x, slot_pair, k, weight=None):
  """(g, e, c, h) rows that the push must deliver (zeros for empty slots)."""
  g, e, c = slot_pair.shape
  h = x.shape[-1]
  sp = slot_pair.long()
  item = (sp.clamp(min=0) // k)
  rows = torch.gather(x.float().unsqueeze(1).expand(g, e, -1, h), 2,
                      item.unsqueeze(-1).expand(g, e, c, h))
  if weight is not None:
    w = torch.gather(weight.reshape(g, 1, -1).expand(g, e, -1), 2, sp.clamp(min=0))
    rows = rows * w.unsqueeze(-1)
  return rows * (sp >= 0).unsqueeze(-1)


@pytest.mark.parametrize("h", [128, 768, 1280])
@pytest.mark.parametrize("ep,rank", [(1, 0), (2, 1), (4, 2)])
def test_bulk_push_delivers_rows_and_counters(h, ep, rank):
  g, s, e, k, c = 3, 150, 8, 2, 44          # block of 132 rows: one full chunk and a short one
  x, gates, expert, slot, slot_pair, bufs, flags, dst, flg, tiles = _setup(g, s, e, k, c, h, ep, rank)
  el, r = e // ep, g * c
  status = torch.zeros(1, dtype=torch.int32, device="cuda")
  args = moe_ops.push_args(x, slot_pair, None, dst, flg, None, None, g, s, e, c, k, h, el, ep, rank)
  moe_ops.push_rows_bulk(args, ctas=3, status=status)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  want = _expected_rows(x, slot_pair, k)      # (g, e, c, h)
  for ee in range(e):
    owner, loc = ee // el, ee % el
    got = bufs[owner][loc, rank * r:(rank + 1) * r].float().reshape(g, c, h)
    torch.testing.assert_close(got, want[:, ee], rtol=0, atol=0)
    # rows of other source ranks are untouched
    if ep > 1:
      other = (rank + 1) % ep
      assert bool((bufs[owner][loc, other * r:(other + 1) * r] == 7.0).all())
    # counters: every tile received exactly the rows of this rank's block that fall into it
    cnt = flags[owner][loc * tiles:(loc + 1) * tiles].cpu()
    for t in range(tiles):
      lo, hi = max(rank * r, t * 128), min((rank + 1) * r, (t + 1) * 128)
      assert int(cnt[t]) == max(0, hi - lo), (ee, t, int(cnt[t]))


def test_bulk_push_scales_rows_and_returns_gate_gradients():
  g, s, e, k, c, h = 2, 120, 4, 2, 70, 256
  x, gates, expert, slot, slot_pair, bufs, flags, dst, flg, tiles = _setup(g, s, e, k, c, h, 1, 0, 3)
  dev = "cuda"
  gate = torch.rand(g, s, k, device=dev)
  ybuf = torch.randn(e, g * c, h, device=dev).bfloat16()
  dgate = torch.zeros(g, s, k, device=dev)
  args = moe_ops.push_args(x, slot_pair, gate, dst, flg, moe_ops.base_table(ybuf), dgate, g, s, e,
                           c, k, h, e, 1, 0)
  moe_ops.push_rows_bulk(args, ctas=2)
  torch.cuda.synchronize()
  want = _expected_rows(x, slot_pair, k, weight=gate)
  got = bufs[0].float().reshape(e, g, c, h).transpose(0, 1)
  torch.testing.assert_close(got, want.bfloat16().float(), rtol=1e-2, atol=1e-2)
  # dgate[g, item, choice] = <x[g, item], ybuf row of that pair>; dropped pairs stay zero
  yrows = ybuf.float().reshape(e, g, c, h)
  want_dg = torch.zeros_like(dgate)
  sp = slot_pair.cpu()
  xf = x.float().cpu()
  yr = yrows.cpu()
  for gi in range(g):
    for ee in range(e):
      for ci in range(c):
        p = int(sp[gi, ee, ci])
        if p >= 0:
          want_dg[gi, p // k, p % k] = float((xf[gi, p // k] * yr[ee, gi, ci]).sum())
  torch.testing.assert_close(dgate.cpu(), want_dg.cpu(), rtol=2e-2, atol=0.3)


@pytest.mark.parametrize("h,m,g,c", [(128, 256, 4, 100), (768, 512, 8, 160)])
def test_gemm_with_fused_push_matches_gemm_on_pushed_rows(h, m, g, c):
  """Dispatch + first expert GEMM through one call: on the larger case the push runs in two
  warps of every GEMM CTA, on the small one (too few tiles for CTA pairs) as a launch of its
  own in front of the GEMM; both must deliver the same rows and the same product."""
  s, e, k = 4 * c, 4, 2
  x, gates, expert, slot, slot_pair, bufs, flags, dst, flg, tiles = _setup(g, s, e, k, c, h, 1, 0, 5)
  dev = "cuda"
  w1 = (torch.randn(e, m, h, device=dev) * 0.05).bfloat16()
  b1 = torch.randn(e, m, device=dev) * 0.1
  status = torch.zeros(1, dtype=torch.int32, device=dev)
  args = moe_ops.push_args(x, slot_pair, None, dst, flg, None, None, g, s, e, c, k, h, e, 1, 0)
  for epoch in (1, 2):   # the counters are cumulative: a second pass waits for 2 x rows
    bufs[0].fill_(7.0)
    hid = G.gemm(bufs[0], w1, bias=b1, act=G.ACT_GELU, a_ready=flags[0], a_ready_epoch=epoch,
                 status=status, push=args)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rows = _expected_rows(x, slot_pair, k).transpose(0, 1).reshape(e, g * c, h).bfloat16()
    torch.testing.assert_close(bufs[0], rows, rtol=0, atol=0)
    want = G.gemm_reference(rows, w1, bias=b1, act=G.ACT_GELU)
    torch.testing.assert_close(hid.float(), want.float(), rtol=2e-2, atol=2e-2)


def test_hidden_gradient_gemm_with_fused_scaled_push():
  """Backward of combine fused into the hidden-gradient GEMM: gate-scaled dy rows, gate
  gradients from the expert outputs, GELU' multiply and bias-gradient column sums."""
  g, c, h, m = 8, 160, 768, 512
  s, e, k = 4 * c, 4, 2
  x, gates, expert, slot, slot_pair, bufs, flags, dst, flg, tiles = _setup(g, s, e, k, c, h, 1, 0, 9)
  dev = "cuda"
  gate = torch.rand(g, s, k, device=dev)
  ybuf = torch.randn(e, g * c, h, device=dev).bfloat16()
  dgate = torch.zeros(g, s, k, device=dev)
  w2 = (torch.randn(e, h, m, device=dev) * 0.05).bfloat16()
  pre = torch.rand(e, g * c, m, device=dev).bfloat16()
  db1 = torch.zeros(e, m, device=dev)
  status = torch.zeros(1, dtype=torch.int32, device=dev)
  args = moe_ops.push_args(x, slot_pair, gate, dst, flg, moe_ops.base_table(ybuf), dgate, g, s, e,
                           c, k, h, e, 1, 0)
  dpre = G.gemm(bufs[0], w2, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True, colsum=db1,
                a_ready=flags[0], a_ready_epoch=1, status=status, push=args)
  torch.cuda.synchronize()
  assert int(status.item()) == 0
  rows = _expected_rows(x, slot_pair, k, weight=gate).transpose(0, 1).reshape(e, g * c, h)
  torch.testing.assert_close(bufs[0].float(), rows.bfloat16().float(), rtol=1e-2, atol=1e-2)
  want_cs = torch.zeros_like(db1)
  want = G.gemm_reference(bufs[0], w2, b_mn_major=True, gelu_pre=pre, gelu_pre_is_grad=True,
                          colsum=want_cs)
  torch.testing.assert_close(dpre.float(), want.float(), rtol=2e-2, atol=2e-2)
  torch.testing.assert_close(db1, want_cs, rtol=2e-2, atol=0.5)
  # gate gradients: <dy row, expert output row> for every kept pair
  sp = slot_pair.long()
  valid = sp >= 0
  item = sp.clamp(min=0) // k
  xr = torch.gather(x.float().unsqueeze(1).expand(g, e, -1, h), 2,
                    item.unsqueeze(-1).expand(g, e, c, h))
  dots = (xr * ybuf.float().reshape(e, g, c, h).transpose(0, 1)).sum(-1)   # (g, e, c)
  want_dg = torch.zeros(g, s * k, device=dev)
  want_dg.scatter_(1, sp.clamp(min=0).reshape(g, -1), (dots * valid).reshape(g, -1))
  # slots that hold no pair scattered a zero into entry 0: restore that entry from its own slot
  got = dgate.reshape(g, -1)
  mask = torch.zeros_like(want_dg, dtype=torch.bool)
  mask.scatter_(1, sp.clamp(min=0).reshape(g, -1), valid.reshape(g, -1))
  torch.testing.assert_close(got[mask], want_dg[mask], rtol=2e-2, atol=0.3)
  assert bool((got[~mask] == 0).all())


def test_gemm_completion_signal_fires_once_per_launch():
  dev = "cuda"
  a = torch.randn(1000, 256, device=dev).bfloat16()
  b = torch.randn(512, 256, device=dev).bfloat16()
  flags = torch.zeros(4, dtype=torch.int32, device=dev)
  done = torch.zeros(1, dtype=torch.int32, device=dev)
  for i in range(3):
    for pair in (1, 2):
      G.gemm(a, b, cta_pair=pair, signal_flags=[flags.data_ptr() + 4 * j for j in (0, 2)],
             done_counter=done)
  torch.cuda.synchronize()
  assert flags.tolist() == [6, 0, 6, 0] and int(done.item()) == 0
