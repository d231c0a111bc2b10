"""The no-allocation LayerNorm backward entry point, called through its exported C symbol,
must agree with the regular entry point (which takes a caller-provided scratch buffer)."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "vmoe_b200",
                    "libvmoe_b200.so")
_vp = ctypes.c_void_p


def _lib():
  lib = ctypes.CDLL(_LIB)
  lib.vmoe_layernorm_bwd_scratch_bytes.restype = ctypes.c_int64
  lib.vmoe_layernorm_bwd_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
  lib.vmoe_last_error.restype = ctypes.c_char_p
  common = [_vp] * 9
  lib.vmoe_layernorm_bwd.argtypes = common + [_vp, ctypes.c_int64, ctypes.c_int64, _vp]
  lib.vmoe_layernorm_bwd_static.argtypes = common + [ctypes.c_int64, ctypes.c_int64, _vp]
  lib.vmoe_layernorm_fwd.argtypes = [_vp] * 6 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_float, _vp]
  return lib


def _case(lib, rows, h, seed):
  torch.manual_seed(seed)
  dev = "cuda"
  stream = torch.cuda.current_stream().cuda_stream
  x = (torch.randn(rows, h, device=dev) * 1.5 + 0.3).bfloat16()
  dy = torch.randn(rows, h, device=dev).bfloat16()
  gamma = torch.randn(h, device=dev)
  beta = torch.randn(h, device=dev)
  y = torch.empty_like(x)
  mean = torch.empty(rows, device=dev)
  rstd = torch.empty(rows, device=dev)
  rc = lib.vmoe_layernorm_fwd(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(),
                              mean.data_ptr(), rstd.data_ptr(), rows, h, 1e-6, stream)
  assert rc == 0, lib.vmoe_last_error()
  outs = []
  for static in (False, True):
    dx = torch.empty_like(x)
    dgamma = torch.zeros(h, device=dev)
    dbeta = torch.zeros(h, device=dev)
    args = [dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), None,
            dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr()]
    if static:
      rc = lib.vmoe_layernorm_bwd_static(*args, rows, h, stream)
    else:
      nbytes = lib.vmoe_layernorm_bwd_scratch_bytes(rows, h)
      scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=dev)
      rc = lib.vmoe_layernorm_bwd(*args, scratch.data_ptr(), rows, h, stream)
    assert rc == 0, lib.vmoe_last_error()
    torch.cuda.synchronize()
    outs.append((dx.float().cpu(), dgamma.cpu(), dbeta.cpu()))
  (dx0, dg0, db0), (dx1, dg1, db1) = outs
  assert torch.equal(dx0, dx1)
  assert torch.equal(dg0, dg1) and torch.equal(db0, db1)
  # and both agree with an fp32 PyTorch reference
  xf = x.float().requires_grad_()
  gf = gamma.clone().requires_grad_()
  bf = beta.clone().requires_grad_()
  torch.nn.functional.layer_norm(xf, (h,), gf, bf, 1e-6).backward(dy.float())
  scale = xf.grad.abs().max().item()
  assert (dx1.cuda() - xf.grad).abs().max().item() / scale < 2e-2
  assert (dg1.cuda() - gf.grad).abs().max().item() / gf.grad.abs().max().item() < 1e-2
  assert (db1.cuda() - bf.grad).abs().max().item() / bf.grad.abs().max().item() < 1e-2


def test_static_scratch_layernorm_bwd_two_calls_in_a_row():
  lib = _lib()
  _case(lib, rows=5000, h=768, seed=0)   # first call: resolves the static array's address
  _case(lib, rows=777, h=1024, seed=1)   # second call reuses the array with other sizes


def test_static_scratch_rejects_large_hidden():
  lib = _lib()
  rc = lib.vmoe_layernorm_bwd_static(None, None, None, None, None, None, None, None, None, 16, 2048,
                                     None)
  assert rc == -1
  assert b"1024" in lib.vmoe_last_error()
