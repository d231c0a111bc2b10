"""Soft MoE router (https://arxiv.org/abs/2308.00951).

Tokens are L2-normalised; each of the ``E x slots`` slots has a learned unit-norm vector
``mu``; ``logits[g, m, n, p] = <x_gm, mu_np>`` (times a learned scalar ``scale``). Slot inputs
are convex combinations of tokens (softmax over tokens) and token outputs are convex
combinations of slot outputs (softmax over all slots): a dense einsum dispatcher with real
weights and bf16 payloads (reference: ``vmoe/projects/soft_moe/router.py:36-182``).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import nn

from vmoe_b200 import moe
from vmoe_b200.models import routing
from vmoe_b200.parallel.exchange import ExpertExchange, LOCAL_EXCHANGE

Tensor = torch.Tensor


def normalize(x: Tensor, axis: int = -1, eps: float = 1e-6) -> Tensor:
  return x * torch.rsqrt(x.square().sum(dim=axis, keepdim=True) + eps)


def cosine_psim(x: Tensor, batch_axes: Tuple[int, ...], contract_axes: Tuple[int, ...],
                eps: float = 1e-9) -> Tensor:
  """Pairwise cosine similarity over the non-batch, non-contracted axes of ``x``: the result
  has shape ``batch + free + free``."""
  x = x * torch.rsqrt(x.square().sum(dim=contract_axes, keepdim=True) + eps)
  free = [a for a in range(x.dim()) if a not in batch_axes and a not in contract_axes]
  perm = list(batch_axes) + free + list(contract_axes)
  xp = x.permute(perm)
  bshape = [x.shape[a] for a in batch_axes]
  fshape = [x.shape[a] for a in free]
  flat = xp.reshape(*bshape, int(torch.tensor(fshape).prod()) if fshape else 1, -1)
  sim = flat @ flat.transpose(-1, -2)
  return sim.reshape(*bshape, *fshape, *fshape)


class SoftRouter(nn.Module):

  def __init__(self, num_experts: int, hidden_size: int, num_slots: Optional[int] = None,
               capacity_factor: Optional[float] = 1.0, noise_std: float = 0.0,
               deterministic: Optional[bool] = None, dtype: Optional[torch.dtype] = None,
               compute_similarity_metrics: bool = True, group_size: Optional[int] = None,
               exchange: ExpertExchange = LOCAL_EXCHANGE, partition_spec=None, precision=None):
    super().__init__()
    self.num_experts = num_experts
    self.num_slots = num_slots
    self.capacity_factor = capacity_factor
    self.noise_std = noise_std
    self.deterministic = deterministic
    self.dtype = dtype
    self.compute_similarity_metrics = compute_similarity_metrics
    self.exchange = exchange
    self._hidden = hidden_size
    self.scale = nn.Parameter(torch.ones(()))
    self.mu: Optional[nn.Parameter] = None
    slots = num_slots
    if slots is None and group_size is not None:
      slots = moe.compute_capacity(group_size, num_experts, capacity_factor,
                                   ceil_or_round="round", multiple_of=1)
    if slots is not None:
      self._create_mu(slots)

  def _create_mu(self, slots: int):
    mu = torch.empty(self._hidden, self.num_experts, slots)
    # lecun-normal with fan_in = hidden * ... as Flax computes it for a (d, n, p) kernel
    routing.lecun_normal_(mu, self._hidden * 1)
    self.mu = nn.Parameter(mu.to(self.scale.device))

  def is_deterministic(self) -> bool:
    return (not self.training) if self.deterministic is None else self.deterministic

  def forward(self, inputs: Tensor):
    dtype = self.dtype or inputs.dtype
    if dtype == torch.bfloat16:
      dtype = torch.float32  # routing statistics in fp32; payloads travel in bf16
    _, group_size, dim = inputs.shape
    if self.num_slots is None:
      slots = moe.compute_capacity(group_size, self.num_experts, self.capacity_factor,
                                   ceil_or_round="round", multiple_of=1)
    else:
      slots = self.num_slots
    if self.mu is None:
      self._create_mu(slots)
    elif self.mu.shape[2] != slots:
      raise ValueError(f"mu was created for {self.mu.shape[2]} slots but {slots} are needed")
    mu = normalize(self.mu.to(dtype), axis=0)
    scale = self.scale.to(dtype)
    logits = self._fast_logits(inputs, mu, scale)
    if logits is None:
      x = normalize(inputs.to(dtype), axis=-1)
      if x.numel() < mu.numel():
        x = x * scale
      else:
        mu = mu * scale
      logits = torch.einsum("gmd,dnp->gmnp", x, mu)
    if not self.is_deterministic() and self.noise_std > 0:
      logits = logits + self.noise_std * torch.randn_like(logits)
    g, m, n, p = logits.shape
    from vmoe_b200.ops import router_ops
    flat = logits.reshape(g, m, n * p)
    if router_ops.soft_router_weights_supported(flat):
      dispatch_weights, combine_weights = router_ops.soft_router_weights(flat)
      dispatch_weights = dispatch_weights.reshape(g, m, n, p)
      combine_weights = combine_weights.reshape(g, m, n, p)
    else:
      dispatch_weights = torch.softmax(logits, dim=1)
      combine_weights = torch.softmax(flat, dim=-1).reshape(g, m, n, p)
    dispatcher = moe.Bfloat16Dispatcher(moe.EinsumDispatcher(
        combine_weights=combine_weights, dispatch_weights=dispatch_weights,
        exchange=self.exchange))
    return dispatcher, self.get_metrics(combine_weights, dispatch_weights, mu)

  def _fast_logits(self, inputs: Tensor, mu: Tensor, scale: Tensor) -> Optional[Tensor]:
    """``<normalize(x), mu> * scale`` for bf16 CUDA activations without materialising the
    normalised tokens: the raw ``x @ mu`` runs on the tensor-core GEMM (fp32 accumulation and
    output) and the per-token ``rsqrt(|x|^2 + eps)`` scales the rows of the (much smaller)
    logits afterwards. Returns None when the fast path does not apply."""
    from vmoe_b200.ops import router_ops
    d, n, p = mu.shape
    if not (inputs.is_cuda and inputs.dtype == torch.bfloat16 and (n * p) % 8 == 0 and d % 8 == 0
            and router_ops.gating_logits_supported(inputs, mu.reshape(d, n * p).t())):
      return None
    w = mu.reshape(d, n * p).t().contiguous()  # (slots, hidden)
    raw = router_ops.gating_logits(inputs, w)  # (G, S, n * p) fp32
    norm = torch.linalg.vector_norm(inputs, ord=2, dim=-1, keepdim=True, dtype=torch.float32)
    inv = torch.rsqrt(norm * norm + 1e-6)
    return (raw * (inv * scale)).reshape(*raw.shape[:2], n, p)

  def get_metrics(self, combine_weights: Tensor, dispatch_weights: Tensor, mu: Tensor):
    g, m, n, p = combine_weights.shape
    metrics: Dict[str, Tensor] = {
        "auxiliary_loss": torch.zeros((), dtype=torch.float32, device=combine_weights.device),
        "combine_weights_min_mean": combine_weights.amin(dim=(2, 3)).mean(),
        "combine_weights_max_mean": combine_weights.amax(dim=(2, 3)).mean(),
        "dispatch_weights_min_mean": dispatch_weights.amin(dim=1).mean(),
        "dispatch_weights_max_mean": dispatch_weights.amax(dim=1).mean(),
    }
    if not self.compute_similarity_metrics:
      return metrics
    with torch.no_grad():
      def stats(sim, eye, count, pairs):
        masked = (1 - eye) * sim
        masked = masked + eye * masked.max()
        return masked.min(), masked.max(), (sim.sum() - count) / pairs
      cw = cosine_psim(combine_weights, (0,), (2, 3))  # (g, m, m)
      lo, hi, mean = stats(cw, torch.eye(m, device=cw.device)[None], g * m, g * m * max(m - 1, 1))
      metrics.update(combine_weights_similarity_min=lo, combine_weights_similarity_max=hi,
                     combine_weights_similarity_mean=mean)
      dw = cosine_psim(dispatch_weights, (0,), (1,))  # (g, n, p, n, p)
      eye = torch.eye(n * p, device=dw.device).reshape(1, n, p, n, p)
      lo, hi, mean = stats(dw, eye, g * n * p, g * n * p * max(n * p - 1, 1))
      metrics.update(dispatch_weights_similarity_min=lo, dispatch_weights_similarity_max=hi,
                     dispatch_weights_similarity_mean=mean)
      ms = cosine_psim(mu, (), (0,))  # (n, p, n, p)
      eye = torch.eye(n * p, device=ms.device).reshape(n, p, n, p)
      lo, hi, mean = stats(ms, eye, n * p, n * p * max(n * p - 1, 1))
      metrics.update(mu_similarity_min=lo, mu_similarity_max=hi, mu_similarity_mean=mean)
    return metrics


def _register():
  from vmoe_b200.models import vit_moe
  vit_moe.register_router("SoftRouter", SoftRouter)


_register()
