"""tcgen05 GEMM kernel vs an fp32 PyTorch reference of the same contract."""
import pytest
import torch

from vmoe_b200.ops import gemm as G

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape):
  return torch.randn(*shape, device=DEV).bfloat16()


def _check(out, ref, tol=2e-2):
  """Largest error relative to the largest reference value, and the relative L2 error over the
  whole tensor (which a wrong tile or a missing edge moves even when no element is far off)."""
  err = (out.float() - ref.float()).abs().max().item()
  scale = ref.float().abs().max().item() + 1e-6
  assert err / scale < tol, (err, scale)
  rel_l2 = ((out.float() - ref.float()).norm() / (ref.float().norm() + 1e-12)).item()
  assert rel_l2 < tol, ("relative L2", rel_l2)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (512, 768, 768), (200, 304, 136), (1000, 21843, 192)])
@pytest.mark.parametrize("amn,bmn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("pair", [1, 2])
def test_gemm_majors(m, n, k, amn, bmn, pair):
  if n % 8 and bmn:
    pytest.skip("MN-major B needs a 16-byte aligned leading dimension")
  torch.manual_seed(0)
  a = _rand(k, m) if amn else _rand(m, k)
  b = _rand(k, n) if bmn else _rand(n, k)
  status = torch.zeros(1, dtype=torch.int32, device=DEV)
  out = G.gemm(a, b, a_mn_major=amn, b_mn_major=bmn, status=status, out_dtype=torch.float32,
               cta_pair=pair)
  ref = G.gemm_reference(a, b, a_mn_major=amn, b_mn_major=bmn, out_dtype=torch.float32)
  _check(out, ref, 1e-3)
  assert status.item() == 0


@pytest.mark.parametrize("pair", [1, 2])
def test_gemm_batched_and_epilogue(pair):
  torch.manual_seed(1)
  e, m, n, k = 3, 300, 520, 192
  a, b = _rand(e, m, k), _rand(e, n, k)
  bias = torch.randn(e, n, device=DEV)
  res = _rand(e, m, n)
  pre = torch.empty(e, m, n, device=DEV, dtype=torch.bfloat16)
  cs = torch.zeros(e, n, device=DEV)
  out = G.gemm(a, b, bias=bias, act=G.ACT_GELU, residual=res, out_pre=pre, colsum=cs,
               cta_pair=pair)
  pre_r = torch.empty_like(pre)
  cs_r = torch.zeros_like(cs)
  ref = G.gemm_reference(a, b, bias=bias, act=G.ACT_GELU, residual=res, out_pre=pre_r, colsum=cs_r,
                         out_dtype=torch.float32)
  _check(out, ref)
  _check(pre, pre_r)
  _check(cs, cs_r, 5e-3)


@pytest.mark.parametrize("pair", [1, 2])
def test_gemm_gelu_grad_and_splitk(pair):
  torch.manual_seed(2)
  m, n, k = 300, 520, 1000
  a, b = _rand(m, k), _rand(n, k)
  gp = _rand(m, n)
  out = G.gemm(a, b, gelu_pre=gp, cta_pair=pair)
  _check(out, G.gemm_reference(a, b, gelu_pre=gp, out_dtype=torch.float32))
  o32 = torch.zeros(m, n, device=DEV)
  G.gemm(a, b, out=o32, accumulate=True, split_k=3, cta_pair=pair)
  G.gemm(a, b, out=o32, accumulate=True, cta_pair=pair)
  _check(o32, 2 * G.gemm_reference(a, b, out_dtype=torch.float32), 1e-3)


def test_gemm_ready_flag_timeout_sets_status():
  """A flag that nothing sets must time out, report through the status word and return."""
  import os
  a, b = _rand(128, 64), _rand(256, 64)
  flags = torch.zeros(1, dtype=torch.int32, device=DEV)
  status = torch.zeros(1, dtype=torch.int32, device=DEV)
  out = G.gemm(a, b, a_ready=flags, a_ready_epoch=1, status=status)
  torch.cuda.synchronize()
  assert status.item() & 8  # kStatusTimeoutFlag
  # The context stays usable and a signalled flag lets the same call complete.
  flags.fill_(128)
  status.zero_()
  out = G.gemm(a, b, a_ready=flags, a_ready_epoch=1, status=status, out_dtype=torch.float32)
  _check(out, G.gemm_reference(a, b, out_dtype=torch.float32), 1e-3)
  assert status.item() == 0


def test_gemm_pair_large_matches_single():
  """A full-size problem (many tiles per CTA pair, several pipeline wraps) in both modes."""
  torch.manual_seed(3)
  m, n, k = 4096 + 128, 2304, 768
  a, b = _rand(m, k), _rand(n, k)
  bias = torch.randn(n, device=DEV)
  status = torch.zeros(1, dtype=torch.int32, device=DEV)
  one = G.gemm(a, b, bias=bias, cta_pair=1, status=status)
  two = G.gemm(a, b, bias=bias, cta_pair=2, status=status)
  assert status.item() == 0
  assert torch.equal(one, two)
  _check(two, G.gemm_reference(a, b, bias=bias, out_dtype=torch.float32))


@pytest.mark.parametrize("pair", [1, 2])
def test_gemm_multi_destination_output(pair):
  """Row blocks of the output go to separate tensors (stand-ins for peer buffers)."""
  torch.manual_seed(4)
  e, rows, dests, n, k = 2, 96, 3, 200, 128
  a, b = _rand(e, rows * dests, k), _rand(e, n, k)
  bias = torch.randn(e, n, device=DEV)
  outs = [torch.zeros(e, rows, n, device=DEV, dtype=torch.bfloat16) for _ in range(dests)]
  G.gemm(a, b, bias=bias, out_multi=outs, cta_pair=pair)
  ref = G.gemm_reference(a, b, bias=bias, out_dtype=torch.float32)
  for j, o in enumerate(outs):
    _check(o, ref[:, j * rows:(j + 1) * rows])
