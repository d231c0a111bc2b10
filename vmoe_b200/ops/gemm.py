"""bf16 GEMM on the tcgen05 kernel (``csrc/gemm_tcgen05.cu``) with fused epilogues.

``gemm(a, b)`` computes ``a @ b^T`` for ``a: [.., M, K]`` and ``b: [.., N, K]``; with
``a_mn_major`` / ``b_mn_major`` the operand is stored transposed (``[.., K, M]`` /
``[.., K, N]``), which is how the backward matmuls read activations and weights in place.
On CPU tensors the same contract is evaluated with PyTorch in fp32 (test oracle and CPU path).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from vmoe_b200.ops import _lib

ACT_NONE, ACT_GELU = 0, 1


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
  return torch.nn.functional.gelu(x, approximate="tanh")


def gelu_tanh_grad(x: torch.Tensor) -> torch.Tensor:
  k0, k1 = 0.7978845608028654, 0.044715
  u = k0 * (x + k1 * x ** 3)
  t = torch.tanh(u)
  return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def _as3d(t: torch.Tensor) -> torch.Tensor:
  return t.unsqueeze(0) if t.dim() == 2 else t


def gemm_reference(a, b, *, a_mn_major=False, b_mn_major=False, bias=None, act=ACT_NONE,
                   residual=None, gelu_pre=None, out=None, out_pre=None, colsum=None,
                   out_dtype=torch.bfloat16, accumulate=False, out_pre_is_grad=False,
                   gelu_pre_is_grad=False):
  """fp32 PyTorch evaluation of the kernel's contract (any device)."""
  a3, b3 = _as3d(a).float(), _as3d(b).float()
  if a_mn_major:
    a3 = a3.transpose(1, 2)
  if b_mn_major:
    b3 = b3.transpose(1, 2)
  v = torch.matmul(a3, b3.transpose(1, 2))
  if bias is not None:
    v = v + bias.float().reshape(v.shape[0], 1, -1)
  if out_pre is not None:
    pv = gelu_tanh_grad(v) if out_pre_is_grad else v
    out_pre.copy_(pv.reshape(out_pre.shape).to(out_pre.dtype))
  if act == ACT_GELU:
    v = gelu_tanh(v)
  if gelu_pre is not None:
    gp = _as3d(gelu_pre).float()
    v = v * (gp if gelu_pre_is_grad else gelu_tanh_grad(gp))
  if residual is not None:
    v = v + _as3d(residual).float()
  if colsum is not None:
    colsum.add_(v.sum(dim=1).reshape(colsum.shape))
  if a.dim() == 2:
    v = v[0]
  if out is None:
    return v.to(out_dtype)
  if accumulate:
    out.add_(v.to(out.dtype))
  else:
    out.copy_(v.to(out.dtype))
  return out


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False,
         b_mn_major: bool = False, bias: Optional[torch.Tensor] = None, act: int = ACT_NONE,
         residual: Optional[torch.Tensor] = None, gelu_pre: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, out_pre: Optional[torch.Tensor] = None,
         colsum: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, split_k: int = 1, a_ready: Optional[torch.Tensor] = None,
         a_ready_epoch: int = 0, status: Optional[torch.Tensor] = None,
         num_sms: int = 0, out_pre_is_grad: bool = False,
         gelu_pre_is_grad: bool = False, mt_offset: int = 0,
         cta_pair: int = 0, out_multi=None, push=None,
         signal_flags=None, done_counter: Optional[torch.Tensor] = None) -> torch.Tensor:
  """``out = epilogue(a @ b^T)``; see ``csrc/vmoe_api.h`` for the epilogue order."""
  if not a.is_cuda:
    return gemm_reference(a, b, a_mn_major=a_mn_major, b_mn_major=b_mn_major, bias=bias,
                          act=act, residual=residual, gelu_pre=gelu_pre, out=out,
                          out_pre=out_pre, colsum=colsum, out_dtype=out_dtype,
                          accumulate=accumulate, out_pre_is_grad=out_pre_is_grad,
                          gelu_pre_is_grad=gelu_pre_is_grad)
  assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, (a.dtype, b.dtype)
  a3, b3 = _as3d(a), _as3d(b)
  assert a3.stride(-1) == 1 and b3.stride(-1) == 1, "innermost dim must be contiguous"
  batch = a3.shape[0]
  assert b3.shape[0] == batch
  if a_mn_major:
    K, M = a3.shape[1], a3.shape[2]
  else:
    M, K = a3.shape[1], a3.shape[2]
  if b_mn_major:
    Kb, N = b3.shape[1], b3.shape[2]
  else:
    N, Kb = b3.shape[1], b3.shape[2]
  assert K == Kb, (a.shape, b.shape, a_mn_major, b_mn_major)
  if out_multi:
    out = out_multi[0]  # layout and dtype of every destination
  elif out is None:
    shape = (M, N) if a.dim() == 2 else (batch, M, N)
    out = torch.empty(shape, dtype=out_dtype, device=a.device)
    assert not accumulate
  o3 = _as3d(out)
  assert o3.stride(-1) == 1 and (out_multi or o3.shape[-2:] == (M, N)), (o3.shape, M, N)
  args = _lib.GemmArgs()
  args.A, args.B, args.C = a3.data_ptr(), b3.data_ptr(), o3.data_ptr()
  args.M, args.N, args.K, args.batch = M, N, K, batch
  args.lda, args.ldb, args.ldc = a3.stride(1), b3.stride(1), o3.stride(1)
  args.a_batch_stride = a3.stride(0) if batch > 1 else 0
  args.b_batch_stride = b3.stride(0) if batch > 1 else 0
  args.c_batch_stride = o3.stride(0) if batch > 1 else 0
  args.a_mn_major, args.b_mn_major = int(a_mn_major), int(b_mn_major)
  args.c_fp32 = int(out.dtype == torch.float32)
  assert out.dtype in (torch.float32, torch.bfloat16)
  args.c_atomic = int(accumulate or split_k > 1)
  if args.c_atomic:
    assert out.dtype == torch.float32, "accumulating output must be fp32"
  args.act, args.split_k = act, max(1, split_k)
  if bias is not None:
    assert bias.dtype == torch.float32 and bias.is_contiguous()
    args.bias = bias.data_ptr()
    args.bias_batch_stride = N if batch > 1 else 0
  if colsum is not None:
    assert colsum.dtype == torch.float32 and colsum.is_contiguous()
    args.colsum = colsum.data_ptr()
    args.bias_batch_stride = N if batch > 1 else 0
  if out_pre is not None:
    p3 = _as3d(out_pre)
    assert out_pre.dtype == torch.bfloat16 and p3.stride() == o3.stride() and out.dtype == torch.bfloat16
    args.C2 = p3.data_ptr()
  r_batch = None
  if residual is not None:
    r3 = _as3d(residual)
    assert residual.dtype == torch.bfloat16 and r3.stride(-1) == 1
    args.residual, args.ldr = r3.data_ptr(), r3.stride(1)
    r_batch = r3.stride(0) if batch > 1 else 0
  if gelu_pre is not None:
    g3 = _as3d(gelu_pre)
    assert gelu_pre.dtype == torch.bfloat16 and g3.stride(-1) == 1
    args.gelu_pre, args.ldr2 = g3.data_ptr(), g3.stride(1)
    gb = g3.stride(0) if batch > 1 else 0
    assert r_batch is None or r_batch == gb
    r_batch = gb
  args.r_batch_stride = r_batch or 0
  if a_ready is not None:
    args.a_ready, args.a_ready_epoch = a_ready.data_ptr(), a_ready_epoch
  if status is not None:
    args.status = status.data_ptr()
  args.num_sms = num_sms
  args.c2_gelu_grad = int(out_pre_is_grad)
  args.pre_is_grad = int(gelu_pre_is_grad)
  args.mt_offset = int(mt_offset)
  args.cta_pair = int(cta_pair)
  if out_multi:
    # Row block j of every batch goes to out_multi[j] (all of shape (batch, rows, N), same
    # strides as ``out``, which only provides the layout and is not written).
    d0 = _as3d(out_multi[0])
    assert len(out_multi) <= 8 and d0.dtype == torch.bfloat16
    assert d0.shape[0] == batch and d0.shape[2] == N and d0.shape[1] * len(out_multi) >= M
    for j, d in enumerate(out_multi):
      dj = _as3d(d)
      assert dj.shape == d0.shape and dj.stride() == d0.stride()
      args.c_multi[j] = dj.data_ptr()
    args.c_multi_count = len(out_multi)
    args.c_multi_rows = d0.shape[1]
    args.ldc = d0.stride(1)
    args.c_batch_stride = d0.stride(0) if batch > 1 else 0
  if push is not None:
    # ``push``: a ``_lib.PushArgs``; two warps of every CTA of the launch deliver rows to the
    # expert owners while the others consume arrived tiles (``a_ready``). Where the fused form
    # does not apply the library runs the push as a launch of its own first.
    args.push = ctypes.cast(ctypes.pointer(push), ctypes.c_void_p)
  if signal_flags:
    # Device addresses (local or peer) that receive +1 once every output tile is stored.
    assert len(signal_flags) <= 8 and done_counter is not None
    for j, addr in enumerate(signal_flags):
      args.signal_flags[j] = int(addr)
    args.signal_count = len(signal_flags)
    args.done_counter = done_counter.data_ptr()
  rc = _lib.lib().vmoe_gemm_bf16(ctypes.byref(args), ctypes.c_void_p(_lib.stream_ptr()))
  _lib.check(rc, "vmoe_gemm_bf16")
  _lib.count_launch()
  return out
