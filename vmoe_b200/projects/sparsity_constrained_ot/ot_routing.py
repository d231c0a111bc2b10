"""Routers that turn gating logits into a (possibly sparse) optimal-transport plan between
the S tokens of a group and the E experts — rows sum to 1, columns to S/E — and then reuse
Top-K ("tokens choose") or Top-C ("experts choose") dispatch on that plan, optionally with
the plain softmax gates as combine weights.

Plans: entropic (Sinkhorn with epsilon = 1 and a fixed number of iterations, or the same KL
projection solved with L-BFGS on the dual), k-sparse (semi-dual of the quadratically
regularised problem whose columns/rows are projected on the k-sparse simplex) and
quadratically regularised without the sparsity constraint. The reference builds them on
jaxopt/ott (``vmoe/projects/sparsity_constrained_ot/*.py``); here the solvers are a few lines
of PyTorch: Sinkhorn is unrolled (differentiable), the dual solvers run without gradient and
the plan is then re-evaluated from the dual potentials so that gradients reach the logits.
"""
from __future__ import annotations

from typing import Optional

import torch

from vmoe_b200 import moe
from vmoe_b200.models import routing

Tensor = torch.Tensor


def _weighted_sum(*pairs):
  total = 0.0
  for w, x in pairs:
    if w > 0:
      total = total + x * w
  return total


def _replace_combine_weights(dispatcher, gates: Tensor):
  if not isinstance(dispatcher, moe.EinsumDispatcher):
    raise TypeError(f"Unsupported dispatcher: {type(dispatcher)}")
  dw = dispatcher._dispatch_w()
  dispatcher.dispatch_weights = dw
  dispatcher.combine_weights = dw.to(gates.dtype) * gates.unsqueeze(-1)
  return dispatcher


# ----------------------------------------------------------------------------- plans
def sinkhorn_plan(sim: Tensor, maxiter: int = 20) -> Tensor:
  """Entropic OT (epsilon 1) for ``sim (G, S, E)``: ``diag(u) exp(sim) diag(v)``."""
  g, s, e = sim.shape
  k = torch.exp(sim - sim.amax(dim=(1, 2), keepdim=True))
  a = sim.new_ones(g, s)
  b = sim.new_full((g, e), s / e)
  u, v = torch.ones_like(a), torch.ones_like(b)
  for _ in range(maxiter):
    v = b / (torch.einsum("gse,gs->ge", k, u) + 1e-30)
    u = a / (torch.einsum("gse,ge->gs", k, v) + 1e-30)
  return u.unsqueeze(-1) * k * v.unsqueeze(1)


def kl_projection_lbfgs_plan(sim: Tensor, maxiter: int = 20) -> Tensor:
  """The same KL projection solved on the dual potentials with L-BFGS."""
  g, s, e = sim.shape
  a = sim.new_ones(g, s)
  b = sim.new_full((g, e), s / e)
  shift = sim.detach().amax(dim=(1, 2), keepdim=True)
  f = torch.zeros(g, s, device=sim.device, dtype=sim.dtype, requires_grad=True)
  h = torch.zeros(g, e, device=sim.device, dtype=sim.dtype, requires_grad=True)
  opt = torch.optim.LBFGS([f, h], max_iter=maxiter, tolerance_grad=1e-3,
                          line_search_fn="strong_wolfe")
  sd = sim.detach() - shift
  def closure():
    opt.zero_grad()
    plan = torch.exp(sd + f.unsqueeze(-1) + h.unsqueeze(1))
    loss = plan.sum() - (f * a).sum() - (h * b).sum()
    loss.backward()
    return loss
  with torch.enable_grad():
    opt.step(closure)
  return torch.exp(sim - shift + f.detach().unsqueeze(-1) + h.detach().unsqueeze(1))


def projection_simplex(x: Tensor, dim: int = -1) -> Tensor:
  """Euclidean projection of every vector along ``dim`` onto the probability simplex."""
  x = x.movedim(dim, -1)
  srt = torch.sort(x, dim=-1, descending=True).values
  css = srt.cumsum(-1) - 1.0
  idx = torch.arange(1, x.shape[-1] + 1, device=x.device, dtype=x.dtype)
  cond = srt - css / idx > 0
  rho = cond.to(x.dtype).cumsum(-1).argmax(-1, keepdim=True)
  tau = css.gather(-1, rho) / (rho.to(x.dtype) + 1.0)
  return torch.clamp(x - tau, min=0).movedim(-1, dim)


def projection_sparse_simplex(x: Tensor, k: int, dim: int = -1) -> Tensor:
  """Projection onto the simplex restricted to at most ``k`` non-zeros (the k largest)."""
  x = x.movedim(dim, -1)
  top, idx = torch.topk(x, min(k, x.shape[-1]), dim=-1)
  out = torch.zeros_like(x).scatter(-1, idx, projection_simplex(top, -1))
  return out.movedim(-1, dim)


def regularized_semi_dual_plan(sim: Tensor, *, nnz_k: Optional[int], row_sparse: bool,
                               maxiter: int = 20, lr: float = 0.5) -> Tensor:
  """Quadratically regularised OT through its semi-dual, maximised with Adam.

  With ``nnz_k`` every column of the plan (every row if ``row_sparse``) has at most ``nnz_k``
  non-zeros; without it the plain simplex projection is used (dense quadratic OT).
  """
  g, s, e = sim.shape
  if row_sparse:  # transpose the problem: "columns" are tokens
    cost = -sim.transpose(1, 2)          # (G, E, S)
    marg_a = sim.new_full((g, e), s / e)  # potentials live on the experts
    marg_b = sim.new_ones(g, s)
  else:
    cost = -sim                           # (G, S, E)
    marg_a = sim.new_ones(g, s)
    marg_b = sim.new_full((g, e), s / e)
  proj = (lambda z: projection_sparse_simplex(z, nnz_k, dim=1)) if nnz_k else \
      (lambda z: projection_simplex(z, dim=1))

  def columns(alpha, c):
    # Column j: b_j * proj((alpha - C_j) / b_j) over the rows (gamma = 1).
    z = (alpha.unsqueeze(-1) - c) / marg_b.unsqueeze(1)
    return proj(z) * marg_b.unsqueeze(1)

  alpha = torch.zeros_like(marg_a, requires_grad=True)
  opt = torch.optim.Adam([alpha], lr=lr)
  cd = cost.detach()
  with torch.enable_grad():
    for _ in range(maxiter):
      opt.zero_grad()
      plan = columns(alpha, cd).detach()
      # Gradient of the semi-dual w.r.t. alpha: a - row sums of the plan (ascent).
      alpha.grad = -(marg_a - plan.sum(-1))
      opt.step()
  plan = columns(alpha.detach(), cost)
  return plan.transpose(1, 2) if row_sparse else plan


# ----------------------------------------------------------------------------- routers
class BaseOTNoisyTopExpertsPerItemRouter(routing.NoisyTopExpertsPerItemRouter):
  """Tokens-choose routers dispatching on a transport plan."""

  def __init__(self, *args, maxiter: int = 20, use_softmax_combine_weights: bool = True, **kw):
    super().__init__(*args, **kw)
    self.maxiter = maxiter
    self.use_softmax_combine_weights = use_softmax_combine_weights

  def plan(self, logits: Tensor) -> Tensor:
    raise NotImplementedError

  def forward(self, inputs: Tensor):
    if inputs.dim() != 3:
      raise ValueError(f"inputs.ndim must be 3, but it is {inputs.dim()}")
    e = self.num_experts
    if not e >= self.num_selected_experts >= 1:
      raise ValueError(
          "num_experts >= num_selected_experts >= 1, but got "
          f"num_experts = {e} and num_selected_experts = {self.num_selected_experts}.")
    logits = self.gating_logits(inputs)
    gates_softmax = torch.softmax(logits, dim=-1)
    importance = (self._importance_auxiliary_loss(gates_softmax)
                  if self.importance_loss_weight else 0.0)
    if self.is_deterministic() or self.noise_std == 0.0:
      plan = self.plan(logits)
      metrics = {"auxiliary_loss": _weighted_sum((self.importance_loss_weight, importance)),
                 "importance_loss": importance}
    else:
      std = self.noise_std / e
      noisy = logits + self.sample_noise(logits)
      plan = self.plan(noisy)
      load = (self._load_auxiliary_loss(logits, noisy, std, self.num_selected_experts)
              if self.load_loss_weight else 0.0)
      metrics = {"auxiliary_loss": _weighted_sum((self.importance_loss_weight, importance),
                                                 (self.load_loss_weight, load)),
                 "importance_loss": importance, "load_loss": load}
    kwargs = dict(self.dispatcher_kwargs)
    use_bf16 = kwargs.pop("bfloat16", False)
    d = moe.get_top_experts_per_item_dispatcher(
        plan, num_selected_experts=self.num_selected_experts, exchange=self.exchange, **kwargs)
    if self.use_softmax_combine_weights:
      d = _replace_combine_weights(d, gates_softmax)
    return (moe.Bfloat16Dispatcher(d) if use_bf16 else d), metrics


class BaseOTNoisyTopItemsPerExpertRouter(routing.NoisyTopItemsPerExpertRouter):
  """Experts-choose routers dispatching on a transport plan."""

  def __init__(self, *args, maxiter: int = 20, use_softmax_combine_weights: bool = True, **kw):
    super().__init__(*args, **kw)
    self.maxiter = maxiter
    self.use_softmax_combine_weights = use_softmax_combine_weights

  def plan(self, logits: Tensor) -> Tensor:
    raise NotImplementedError

  def forward(self, inputs: Tensor):
    logits = self.gating_logits(inputs)
    gates_softmax = torch.softmax(logits, dim=-1)
    if not (self.is_deterministic() or self.noise_std == 0.0):
      logits = logits + self.sample_noise(logits)
    plan = self.plan(logits)
    kwargs = dict(self.dispatcher_kwargs)
    use_bf16 = kwargs.pop("bfloat16", False)
    d, metrics = moe.get_top_items_per_expert_dispatcher(plan, exchange=self.exchange, **kwargs)
    if self.use_softmax_combine_weights:
      d = _replace_combine_weights(d, gates_softmax)
    metrics["auxiliary_loss"] = torch.zeros(plan.shape[0], dtype=plan.dtype, device=plan.device)
    return (moe.Bfloat16Dispatcher(d) if use_bf16 else d), metrics


def _kl_plan(self, logits):
  if getattr(self, "use_lbfgs", False):
    return kl_projection_lbfgs_plan(logits, self.maxiter)
  return sinkhorn_plan(logits, self.maxiter)


class KLProjectionNoisyTopExpertsPerItemRouter(BaseOTNoisyTopExpertsPerItemRouter):
  def __init__(self, *args, use_lbfgs: bool = False, use_implicit_differentiation: bool = False, **kw):
    super().__init__(*args, **kw)
    self.use_lbfgs = use_lbfgs
  plan = _kl_plan


class KLProjectionNoisyTopItemsPerExpertRouter(BaseOTNoisyTopItemsPerExpertRouter):
  def __init__(self, *args, use_lbfgs: bool = False, use_implicit_differentiation: bool = False, **kw):
    super().__init__(*args, **kw)
    self.use_lbfgs = use_lbfgs
  plan = _kl_plan


class KSparseProjectionTransportTopExpertsPerItemRouter(BaseOTNoisyTopExpertsPerItemRouter):
  """Rows (tokens) of the plan have at most ``num_selected_experts`` non-zeros."""
  def plan(self, logits):
    return regularized_semi_dual_plan(logits, nnz_k=self.num_selected_experts, row_sparse=True,
                                      maxiter=self.maxiter)


class KSparseProjectionTransportTopItemsPerExpertRouter(BaseOTNoisyTopItemsPerExpertRouter):
  """Columns (experts) of the plan have at most ``capacity`` non-zeros."""
  def plan(self, logits):
    s, e = logits.shape[1], logits.shape[2]
    kw = self.dispatcher_kwargs
    cap = kw.get("capacity") or moe.compute_capacity(
        s, e, kw.get("capacity_factor", 1.0), kw.get("capacity_ceil_or_round", "ceil"),
        kw.get("capacity_multiple_of", 4))
    return regularized_semi_dual_plan(logits, nnz_k=int(cap), row_sparse=False,
                                      maxiter=self.maxiter)


class SparseProjectionTransportTopItemsPerExpertRouter(BaseOTNoisyTopItemsPerExpertRouter):
  """Quadratically regularised OT (sparse by nature, no explicit sparsity constraint)."""
  def plan(self, logits):
    return regularized_semi_dual_plan(logits, nnz_k=None, row_sparse=False, maxiter=self.maxiter)


def _register():
  from vmoe_b200.models import vit_moe
  for cls in (KLProjectionNoisyTopExpertsPerItemRouter, KLProjectionNoisyTopItemsPerExpertRouter,
              KSparseProjectionTransportTopExpertsPerItemRouter,
              KSparseProjectionTransportTopItemsPerExpertRouter,
              SparseProjectionTransportTopItemsPerExpertRouter):
    vit_moe.register_router(cls.__name__, cls)


_register()
