"""Micro-benchmarks of single kernels on ViT-B/16 training shapes (one GPU).

  python -m vmoe_b200.ops.bench_kernels <case> [--rows 100864] [--iters 10]

Cases: ``gemm_dense`` (qkv, fc1 with GELU and two outputs, out-projection with residual),
``gemm_dgrad`` (hidden-gradient GEMM with / without GELU' and column sums in the epilogue),
``gemm_multi_dest`` (second expert GEMM storing row blocks into eight destination buffers),
``gemm_expert_wgrad`` (weight gradients of batched experts, accumulating and not),
``gemm_dense_wgrad`` (weight gradients of the dense layers over split-K factors),
``gemm_library`` (the same shapes through ``torch.matmul`` / ``torch.addmm``, i.e. cuBLAS: the
comparator of the two cases above), ``colsum`` (bias gradients), ``layernorm`` (forward and backward), ``attention``
(packed-QKV forward and backward at the B/16 shape: 12 heads of 64, 197 tokens),
``attention_trace`` (in-kernel timeline, diagnostic build), ``attention_h14`` (16 heads of 80, 257 tokens: the key-blocked kernels, with PyTorch's fused
attention as the comparator), ``attention_dropout`` (the B/16 shape with dropout 0.1),
``router`` (gating logits, noisy softmax, auxiliary losses, forward and backward),
``soft_router`` (Soft MoE dispatch / combine softmaxes, forward and backward).
Every case runs one warm-up pass, then times ``iters`` passes with CUDA events; inputs are
larger than the L2 cache. The same commands are the workloads of the profiler summaries kept
under ``profiles/``.
"""
from __future__ import annotations

import argparse
import os

import torch


def _timed(fn, iters):
  fn()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(iters):
    fn()
  e1.record()
  torch.cuda.synchronize()
  return e0.elapsed_time(e1) * 1e3 / iters  # microseconds


def gemm_dense(rows: int, iters: int):
  from vmoe_b200.ops import gemm as G
  dev = "cuda"
  x = torch.randn(rows, 768, device=dev).bfloat16()
  wqkv = torch.randn(2304, 768, device=dev).bfloat16()
  bqkv = torch.randn(2304, device=dev)
  w1 = torch.randn(3072, 768, device=dev).bfloat16()
  b1 = torch.randn(3072, device=dev)
  wo = torch.randn(768, 768, device=dev).bfloat16()
  bo = torch.randn(768, device=dev)
  res = torch.randn(rows, 768, device=dev).bfloat16()
  pre = torch.empty(rows, 3072, device=dev, dtype=torch.bfloat16)
  cases = {
      "qkv": (lambda: G.gemm(x, wqkv, bias=bqkv), 2 * rows * 768 * 2304),
      "fc1_gelu": (lambda: G.gemm(x, w1, bias=b1, act=G.ACT_GELU, out_pre=pre),
                   2 * rows * 768 * 3072),
      "out_proj_residual": (lambda: G.gemm(x, wo, bias=bo, residual=res), 2 * rows * 768 * 768),
  }
  for name, (fn, flops) in cases.items():
    us = _timed(fn, iters)
    print(f"{name}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s")


def gemm_dgrad(rows: int, iters: int):
  """The MLP's hidden-gradient GEMM: dy (rows x 768) x W2 -> rows x 3072, with and without the
  GELU' multiply and the bias-gradient column sums in the epilogue."""
  from vmoe_b200.ops import gemm as G
  from vmoe_b200.ops import reduce
  dev = "cuda"
  dy = torch.randn(rows, 768, device=dev).bfloat16()
  w2 = torch.randn(768, 3072, device=dev).bfloat16()
  gp = torch.rand(rows, 3072, device=dev).bfloat16()
  cs = torch.zeros(3072, device=dev)
  flops = 2 * rows * 768 * 3072
  out = G.gemm(dy, w2, b_mn_major=True)
  cases = {
      "plain": lambda: G.gemm(dy, w2, b_mn_major=True),
      "gelu_grad": lambda: G.gemm(dy, w2, b_mn_major=True, gelu_pre=gp, gelu_pre_is_grad=True),
      "colsum": lambda: G.gemm(dy, w2, b_mn_major=True, colsum=cs),
      "gelu_grad+colsum": lambda: G.gemm(dy, w2, b_mn_major=True, gelu_pre=gp,
                                         gelu_pre_is_grad=True, colsum=cs),
      "separate colsum kernel": lambda: reduce.colsum(out, out=cs),
  }
  for name, fn in cases.items():
    us = _timed(fn, iters)
    print(f"{name}: {us:.1f} us" + (f", {flops / us / 1e6:.0f} TFLOP/s" if "kernel" not in name else ""))


def gemm_multi_dest(rows: int, iters: int):
  """The second expert GEMM as the expert-parallel path runs it: (experts x rows, 3072) x
  (3072, 768) with every block of rows / 8 output rows stored into its own destination buffer
  (here all local; on several GPUs seven of the eight are peers' buffers), against the same
  GEMM with one ordinary output."""
  from vmoe_b200.ops import gemm as G
  dev = "cuda"
  dests = 8
  block = (rows // dests) // 256 * 256
  m = block * dests
  hid = torch.randn(1, m, 3072, device=dev).bfloat16()
  w2 = torch.randn(1, 768, 3072, device=dev).bfloat16()
  b2 = torch.randn(1, 768, device=dev)
  outs = [torch.empty(1, block, 768, device=dev, dtype=torch.bfloat16) for _ in range(dests)]
  flops = 2 * m * 3072 * 768
  for name, fn in {
      "one output": lambda: G.gemm(hid, w2, bias=b2),
      "eight destinations": lambda: G.gemm(hid, w2, bias=b2, out_multi=outs, mt_offset=block // 128),
  }.items():
    us = _timed(fn, iters)
    print(f"{name}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s")


def colsum(rows: int, iters: int):
  """Bias gradients: column sums of (rows, n) bf16 matrices into fp32."""
  from vmoe_b200.ops import reduce
  for n in (768, 2304, 3072):
    x = torch.randn(rows, n, device="cuda").bfloat16()
    out = torch.zeros(n, device="cuda")
    us = _timed(lambda: reduce.colsum(x, out=out), iters)
    print(f"colsum rows x {n}: {us:.1f} us ({rows * n * 2 / us / 1e3:.0f} GB/s)")


def layernorm(rows: int, iters: int):
  from vmoe_b200 import ops
  x = torch.randn(rows, 768, device="cuda").bfloat16().requires_grad_()
  w = torch.ones(768, device="cuda", requires_grad=True)
  b = torch.zeros(768, device="cuda", requires_grad=True)
  y = ops.layer_norm(x, w, b, 1e-6)
  g = torch.randn_like(y)
  us_f = _timed(lambda: ops.layer_norm(x, w, b, 1e-6), iters)

  nbytes = rows * 768 * 2
  us_b = _timed(lambda: torch.autograd.grad(y, x, g, retain_graph=True), iters)
  y2, xr = ops.layer_norm_fork(x, w, b, 1e-6)
  us_bf = _timed(lambda: torch.autograd.grad([y2, xr], x, [g, g], retain_graph=True), iters)
  print(f"layernorm fwd: {us_f:.1f} us ({2 * nbytes / us_f / 1e3:.0f} GB/s); "
        f"bwd: {us_b:.1f} us ({3 * nbytes / us_b / 1e3:.0f} GB/s); "
        f"bwd with residual gradient: {us_bf:.1f} us ({4 * nbytes / us_bf / 1e3:.0f} GB/s)")


def attention(rows: int, iters: int):
  from vmoe_b200 import ops
  batch = max(rows // 197, 1)
  qkv = torch.randn(batch, 197, 3, 12, 64, device="cuda").bfloat16().requires_grad_()
  out = ops.attention_packed(qkv)
  g = torch.randn_like(out)
  us_f = _timed(lambda: ops.attention_packed(qkv), iters)

  us_b = _timed(lambda: torch.autograd.grad(out, qkv, g, retain_graph=True), iters)
  flops = 4 * batch * 12 * 197 * 197 * 64
  print(f"attention fwd: {us_f:.1f} us ({flops / us_f / 1e6:.0f} TFLOP/s useful); "
        f"bwd: {us_b:.1f} us ({2.5 * flops / us_b / 1e6:.0f} TFLOP/s useful)")


def gemm_expert_wgrad(rows: int, iters: int):
  """Weight-gradient GEMMs of batched experts, dW[e] = dy[e]^T x[e], adding into an fp32 buffer
  (``accumulate=True``, as the backward pass does) and as a plain store: many small experts
  (Soft MoE B/16: 128 x 256 and 128 x 512 rows, V-MoE L/16: 32 x 832 rows) and the 8 large
  experts of V-MoE B/16."""
  from vmoe_b200.ops import gemm as G
  for e, r, h, m in ((128, 256, 768, 3072), (128, 512, 768, 3072), (32, 832, 1024, 4096),
                     (8, 26624, 768, 3072)):
    dy = torch.randn(e, r, m, device="cuda").bfloat16()
    x = torch.randn(e, r, h, device="cuda").bfloat16()
    dw = torch.zeros(e, m, h, device="cuda")
    flops = 2.0 * e * r * h * m
    for acc in (True, False):
      us = _timed(lambda: G.gemm(dy, x, a_mn_major=True, b_mn_major=True, out=dw, accumulate=acc),
                  iters)
      print(f"experts={e} rows={r} weight {m}x{h} accumulate={acc}: {us:.0f} us, "
            f"{flops / us / 1e6:.0f} TFLOP/s")


def gemm_dense_wgrad(rows: int, iters: int):
  """Weight gradients of the dense layers of ViT-B, dW = dy^T x over ``rows`` tokens, adding
  into an fp32 buffer with the split-K factor the backward pass picks
  (``ops/functional.py:_wgrad_split``) and with factors 1, 2, 4 and 8 for comparison."""
  from vmoe_b200.ops import gemm as G
  from vmoe_b200.ops.functional import _wgrad_split
  for name, n, k in (("qkv", 2304, 768), ("out_proj", 768, 768), ("fc1", 3072, 768),
                     ("fc2", 768, 3072)):
    dy = torch.randn(rows, n, device="cuda").bfloat16()
    x = torch.randn(rows, k, device="cuda").bfloat16()
    dw = torch.zeros(n, k, device="cuda")
    picked = _wgrad_split(n, k, rows)
    parts = []
    for split in sorted({picked, 1, 2, 4, 8}):
      us = _timed(lambda: G.gemm(dy, x, a_mn_major=True, b_mn_major=True, out=dw,
                                 accumulate=True, split_k=split), iters)
      parts.append(f"split {split}{' (picked)' if split == picked else ''}: {us:.0f} us")
    print(f"{name} weight gradient {n}x{k}: " + ", ".join(parts))


def gemm_library(rows: int, iters: int):
  """The shapes of ``gemm_dense`` / ``gemm_dgrad`` through cuBLAS (``torch.matmul``, and
  ``torch.addmm`` for the bias): the rate a library GEMM reaches WITHOUT the GELU, the second
  output, the residual add or the column sums that our epilogues carry."""
  dev = "cuda"
  x = torch.randn(rows, 768, device=dev).bfloat16()
  for name, n in (("qkv", 2304), ("fc1", 3072), ("out_proj", 768)):
    w = torch.randn(n, 768, device=dev).bfloat16()
    b = torch.randn(n, device=dev).bfloat16()
    out = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
    flops = 2 * rows * 768 * n
    us = _timed(lambda: torch.matmul(x, w.t(), out=out), iters)
    us_b = _timed(lambda: torch.addmm(b, x, w.t(), out=out), iters)
    print(f"library {name}: matmul {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s; with bias "
          f"{us_b:.1f} us, {flops / us_b / 1e6:.0f} TFLOP/s")
  w2 = torch.randn(768, 3072, device=dev).bfloat16()
  out = torch.empty(rows, 3072, device=dev, dtype=torch.bfloat16)
  us = _timed(lambda: torch.matmul(x, w2, out=out), iters)
  print(f"library dgrad (rows x 768) x (768 x 3072): {us:.1f} us, "
        f"{2 * rows * 768 * 3072 / us / 1e6:.0f} TFLOP/s")


def _attention_case(batch, t, h, d, iters, dropout=0.0, library=True):
  from vmoe_b200 import ops
  import torch.nn.functional as F
  qkv = torch.randn(batch, t, 3, h, d, device="cuda").bfloat16().requires_grad_()
  run = lambda: ops.attention_packed(qkv, dropout_p=dropout, training=dropout > 0)
  out = run()
  g = torch.randn_like(out)
  us_f = _timed(run, iters)
  us_b = _timed(lambda: torch.autograd.grad(out, qkv, g, retain_graph=True), iters)
  flops = 4 * batch * h * t * t * d
  line = (f"attention B={batch} T={t} H={h} D={d} dropout={dropout}: fwd {us_f:.1f} us "
          f"({flops / us_f / 1e6:.0f} TFLOP/s useful); bwd {us_b:.1f} us "
          f"({2.5 * flops / us_b / 1e6:.0f} TFLOP/s useful)")
  if library:
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
    lib = lambda: F.scaled_dot_product_attention(q, k, v, dropout_p=dropout)
    out2 = lib()
    g2 = torch.randn_like(out2)
    us_lf = _timed(lib, iters)
    us_lb = _timed(lambda: torch.autograd.grad(out2, qkv, g2, retain_graph=True), iters)
    line += f"; PyTorch fused attention fwd {us_lf:.1f} us, bwd {us_lb:.1f} us"
  print(line)


def attention_trace(rows: int, iters: int):
  """In-kernel timeline of one CTA of the general attention kernels (needs a library built with
  ``python -m vmoe_b200.build --define ATT_TRACE=1 --output <path>`` and loaded through
  ``VMOE_B200_LIB=<path>``): mean cycles between consecutive probes, by (tag, next tag), for the
  forward pass and for the backward pass; the tags are listed beside ``ATT_STAMP`` in
  ``csrc/attention_tcgen05.cu``. With ``VMOE_B200_ATTN_GENERAL=1`` the D = 64 shape runs on the
  general kernels; without it, on the one-shot kernels, whose backward pass carries probes of
  its own (``csrc/attention_d64_tcgen05.cu``)."""
  import collections
  import ctypes
  from vmoe_b200.ops import _lib, attention_ops
  lib = _lib.lib()
  if not hasattr(lib, "vmoe_attention_trace_read"):
    raise SystemExit("this library was built without -DATT_TRACE")
  batch = max(rows // 197, 1)
  qkv = torch.randn(batch, 197, 3, 12, 64, device="cuda").bfloat16().requires_grad_()
  buf = (ctypes.c_longlong * 4096)()

  general = os.environ.get("VMOE_B200_ATTN_GENERAL") == "1"
  reader = lib.vmoe_attention_trace_read if general else lib.vmoe_attention_d64_trace_read

  def report(title):
    for who, name in ((0, "softmax warp"), (1, "MMA thread")):
      n = reader(buf, who)
      ev = [(buf[2 * i], buf[2 * i + 1]) for i in range(n)]
      if not ev:
        continue
      print(f"{title}, {name}: {n} stamps over {ev[-1][1] - ev[0][1]} cycles")
      acc = collections.defaultdict(list)
      for (t0, c0), (t1, c1) in zip(ev, ev[1:]):
        acc[t0, t1].append(c1 - c0)
      for (t0, t1), v in sorted(acc.items()):
        v = v[2:] if len(v) > 4 else v
        print(f"  {t0} -> {t1}: n={len(v)} mean={sum(v) / len(v):.0f} min={min(v)} max={max(v)}")

  out = attention_ops.packed_attention(qkv)
  g = torch.randn_like(out)
  torch.cuda.synchronize()
  for who in (0, 1):
    reader(buf, who)
  out = attention_ops.packed_attention(qkv)
  torch.cuda.synchronize()
  report("forward")
  out.backward(g)
  torch.cuda.synchronize()
  report("backward")


def attention_h14(rows: int, iters: int):
  """ViT-H/14 at 224 px: 16 heads of 80, 257 tokens (two key blocks, head dimension not 64)."""
  _attention_case(max(rows // 257 // 4, 1), 257, 16, 80, iters)


def attention_dropout(rows: int, iters: int):
  _attention_case(max(rows // 197, 1), 197, 12, 64, iters, dropout=0.1)


def router(rows: int, iters: int):
  from vmoe_b200.models import routing
  groups = 32
  x = torch.randn(groups, rows // groups, 768, device="cuda").bfloat16().requires_grad_()
  r = routing.NoisyTopExpertsPerItemRouter(
      num_experts=8, hidden_size=768, num_selected_experts=2, noise_std=1.0,
      importance_loss_weight=0.005, load_loss_weight=0.005,
      dispatcher=dict(name="einsum", capacity_factor=1.05, batch_priority=True)).cuda()
  r.train()

  def fwd():
    return r._compute_gates_softmax_and_metrics(x, 8)

  def both():
    gates, metrics = fwd()
    (gates.square().sum() + metrics["auxiliary_loss"].sum()).backward()

  print(f"router fwd: {_timed(fwd, iters):.1f} us; fwd+bwd: {_timed(both, iters):.1f} us")


def soft_router(rows: int, iters: int):
  """Soft MoE routing weights of ``rows // 196`` groups of 196 tokens x 128 slots: both
  softmaxes in one kernel, and the fused backward, against the two PyTorch softmaxes."""
  from vmoe_b200.ops import router_ops
  groups = max(rows // 196, 1)
  logits = (torch.randn(groups, 196, 128, device="cuda") * 3).requires_grad_()
  d, c = router_ops.soft_router_weights(logits)
  gd, gc = torch.randn_like(d), torch.randn_like(c)
  nbytes = logits.numel() * 4
  us_f = _timed(lambda: router_ops.soft_router_weights(logits), iters)
  us_b = _timed(lambda: torch.autograd.grad([d, c], logits, [gd, gc], retain_graph=True), iters)

  def torch_fwd():
    return torch.softmax(logits, dim=1), torch.softmax(logits, dim=2)

  d2, c2 = torch_fwd()
  us_tf = _timed(torch_fwd, iters)
  us_tb = _timed(lambda: torch.autograd.grad([d2, c2], logits, [gd, gc], retain_graph=True), iters)
  print(f"soft router weights fwd: {us_f:.1f} us ({3 * nbytes / us_f / 1e3:.0f} GB/s; PyTorch "
        f"{us_tf:.1f} us); bwd: {us_b:.1f} us ({5 * nbytes / us_b / 1e3:.0f} GB/s; PyTorch "
        f"{us_tb:.1f} us)")


CASES = {"soft_router": soft_router, "gemm_dense": gemm_dense, "gemm_dgrad": gemm_dgrad,
         "gemm_multi_dest": gemm_multi_dest, "gemm_library": gemm_library, "gemm_expert_wgrad": gemm_expert_wgrad, "gemm_dense_wgrad": gemm_dense_wgrad, "colsum": colsum, "layernorm": layernorm,
         "attention": attention, "attention_trace": attention_trace, "attention_h14": attention_h14,
         "attention_dropout": attention_dropout, "router": router}


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("case", choices=sorted(CASES))
  ap.add_argument("--rows", type=int, default=100864)
  ap.add_argument("--iters", type=int, default=10)
  args = ap.parse_args()
  CASES[args.case](args.rows, args.iters)


if __name__ == "__main__":
  main()
