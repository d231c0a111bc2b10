"""Vision Transformer with sparse Mixture-of-Experts MLP blocks (V-MoE).

Module tree and parameter names mirror the reference's Flax model so that checkpoints map
one to one (``vmoe_b200/checkpoints/flax_layout.py`` does the layout conversion):
``embedding`` -> ``cls`` -> ``Encoder/{posembed_input, encoderblock_N/{LayerNorm_0,
SelfAttention, LayerNorm_1, Mlp | Moe/{Router, Mlp}}, encoder_norm}`` -> ``MapHead`` ->
``pre_logits`` -> ``head``. Every model returns ``(output, metrics)`` where
``metrics['auxiliary_loss']`` is the per-group sum over all MoE blocks.

Reference: ``vmoe/nn/vit_moe.py`` (MlpMoeBlock :48-124, MapHead :127-148, EncoderBlock
:151-183, EncoderMoe :186-308, VisionTransformerMoe :311-383).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Iterable, Mapping, Optional, Sequence, Union

import torch
import torch.nn.functional as F
from torch import nn

from vmoe_b200 import moe
from vmoe_b200 import ops
from vmoe_b200.models import routing
from vmoe_b200.parallel import grad_allreduce
from vmoe_b200.parallel import mesh as mesh_lib
from vmoe_b200.parallel.exchange import ExpertExchange
from vmoe_b200.utils.misc import parse_call

Tensor = torch.Tensor
KwArgs = Mapping[str, Any]

LN_EPS = 1e-6


def parse_dtype(dtype) -> Optional[torch.dtype]:
  if dtype is None or isinstance(dtype, torch.dtype):
    return dtype
  table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "float16": torch.float16, "float64": torch.float64}
  if str(dtype) in table:
    return table[str(dtype)]
  raise ValueError(f"Unsupported dtype {dtype!r}")


def xavier_uniform_(w: Tensor, fan_in: int, fan_out: int) -> Tensor:
  bound = math.sqrt(6.0 / (fan_in + fan_out))
  with torch.no_grad():
    return w.uniform_(-bound, bound)


class LayerNorm(nn.Module):
  """LayerNorm over the last dim, eps 1e-6 (the Flax default used by the reference)."""

  def __init__(self, dim: int, use_bias: bool = True, eps: float = LN_EPS):
    super().__init__()
    self.eps = eps
    self.scale = nn.Parameter(torch.ones(dim))
    self.bias = nn.Parameter(torch.zeros(dim)) if use_bias else None

  def forward(self, x: Tensor) -> Tensor:
    return ops.layer_norm(x, self.scale, self.bias, self.eps)

  def fork(self, x: Tensor):
    """``(self(x), x)`` with the residual branch's gradient fused into the backward kernel."""
    return ops.layer_norm_fork(x, self.scale, self.bias, self.eps)


class Dense(nn.Module):
  """``y = x W^T + b`` with ``weight: [out, in]`` (fp32 master, bf16 tensor-core compute)."""

  def __init__(self, in_features: int, out_features: int, use_bias: bool = True,
               kernel_init: str = "lecun_normal", bias_init: float = 0.0):
    super().__init__()
    self.weight = nn.Parameter(torch.empty(out_features, in_features))
    self.bias = nn.Parameter(torch.full((out_features,), float(bias_init))) if use_bias else None
    if kernel_init == "zeros":
      nn.init.zeros_(self.weight)
    elif kernel_init == "xavier_uniform":
      xavier_uniform_(self.weight, in_features, out_features)
    else:
      routing.lecun_normal_(self.weight, in_features)

  def forward(self, x: Tensor, act: Optional[str] = None, residual: Optional[Tensor] = None):
    return ops.linear(x, self.weight, self.bias, act=act, residual=residual)


class MlpBlock(nn.Module):
  """Dense -> GELU(tanh) -> dropout -> Dense -> dropout (``vit_jax`` MlpBlock semantics)."""

  def __init__(self, hidden_size: int, mlp_dim: int, out_dim: Optional[int] = None,
               dropout_rate: float = 0.0):
    super().__init__()
    out_dim = out_dim or hidden_size
    self.dropout_rate = dropout_rate
    # Stored with a leading expert axis of 1 so that dense and expert MLPs share kernels.
    self.w1 = nn.Parameter(torch.empty(1, mlp_dim, hidden_size))
    self.b1 = nn.Parameter(torch.empty(1, mlp_dim))
    self.w2 = nn.Parameter(torch.empty(1, out_dim, mlp_dim))
    self.b2 = nn.Parameter(torch.empty(1, out_dim))
    xavier_uniform_(self.w1, hidden_size, mlp_dim)
    xavier_uniform_(self.w2, mlp_dim, out_dim)
    nn.init.normal_(self.b1, std=1e-6)
    nn.init.normal_(self.b2, std=1e-6)

  def forward(self, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
    shape = x.shape
    x3 = x.reshape(1, -1, shape[-1])
    if self.training and self.dropout_rate > 0:
      h = ops.linear(x3[0], self.w1[0], self.b1[0], act="gelu")
      h = F.dropout(h, self.dropout_rate, True)
      y = F.dropout(ops.linear(h, self.w2[0], self.b2[0]), self.dropout_rate, True)
      y = y.reshape(*shape[:-1], -1)
      return y if residual is None else y + residual
    res3 = None if residual is None else residual.reshape(1, -1, residual.shape[-1])
    y = ops.expert_mlp(x3, self.w1, self.b1, self.w2, self.b2, residual=res3)
    return y.reshape(*shape[:-1], -1)


class ExpertMlp(nn.Module):
  """The MLPs of the experts held by this rank, batched over the leading expert axis."""

  def __init__(self, num_local_experts: int, hidden_size: int, mlp_dim: int,
               dropout_rate: float = 0.0, num_experts: Optional[int] = None,
               first_expert: int = 0, split_rngs: bool = False):
    super().__init__()
    self.dropout_rate = dropout_rate
    e_total = num_experts or num_local_experts
    n_init = e_total if split_rngs else 1
    w1 = torch.empty(n_init, mlp_dim, hidden_size)
    w2 = torch.empty(n_init, hidden_size, mlp_dim)
    b1 = torch.empty(n_init, mlp_dim)
    b2 = torch.empty(n_init, hidden_size)
    xavier_uniform_(w1, hidden_size, mlp_dim)
    xavier_uniform_(w2, mlp_dim, hidden_size)
    nn.init.normal_(b1, std=1e-6)
    nn.init.normal_(b2, std=1e-6)
    sl = slice(first_expert, first_expert + num_local_experts)

    def pick(t):
      # Without split RNGs every expert starts from the same weights (the reference
      # broadcasts one RNG through its vmap, vmoe/nn/vit_moe.py:90-99).
      return (t[sl] if split_rngs else t.expand(num_local_experts, *t.shape[1:])).clone()

    self.w1, self.b1 = nn.Parameter(pick(w1)), nn.Parameter(pick(b1))
    self.w2, self.b2 = nn.Parameter(pick(w2)), nn.Parameter(pick(b2))
    for p in (self.w1, self.b1, self.w2, self.b2):
      p.expert_sharded = True  # sharded over the 'expert' mesh axis (dim 0)

  def forward(self, x: Tensor) -> Tensor:
    if self.training and self.dropout_rate > 0:
      dt = x.dtype
      h = torch.baddbmm(self.b1.to(dt).unsqueeze(1), x, self.w1.to(dt).transpose(1, 2))
      h = F.dropout(F.gelu(h, approximate="tanh"), self.dropout_rate, True)
      y = torch.baddbmm(self.b2.to(dt).unsqueeze(1), h, self.w2.to(dt).transpose(1, 2))
      return F.dropout(y, self.dropout_rate, True)
    return ops.expert_mlp(x, self.w1, self.b1, self.w2, self.b2)


class MlpMoeBlock(nn.Module):
  """Sparse MoE of MLPs: tokens are regrouped into groups of ``group_size`` and each group is
  routed independently; experts are sharded over the 'expert' axis of the mesh."""

  def __init__(self, hidden_size: int, mlp_dim: int, num_experts: int, group_size: int,
               dropout_rate: float = 0.0, router: Optional[KwArgs] = None,
               dtype: Optional[torch.dtype] = None,
               split_rngs: Union[bool, Iterable[str]] = False,
               mesh: Optional[mesh_lib.Mesh] = None):
    super().__init__()
    self.group_size = group_size
    self.num_experts = num_experts
    mesh = mesh or mesh_lib.get_mesh()
    self.mesh = mesh
    ep = mesh.num_partitions
    if num_experts % ep:
      raise ValueError(f"num_experts={num_experts} is not divisible by the expert axis ({ep})")
    self.num_local_experts = num_experts // ep
    self.exchange = ExpertExchange.from_mesh(mesh)
    if isinstance(split_rngs, bool):
      split_params = split_rngs
    else:
      split_params = "params" in set(split_rngs)
    self.Router = self.create_router(hidden_size, num_experts, router, dtype)
    self.Mlp = ExpertMlp(self.num_local_experts, hidden_size, mlp_dim, dropout_rate,
                         num_experts=num_experts,
                         first_expert=mesh.expert_rank * self.num_local_experts,
                         split_rngs=split_params)

  def create_router(self, hidden_size, num_experts, router, dtype) -> nn.Module:
    kwargs = dict(num_experts=num_experts, **(router or {}))
    name = kwargs.pop("name", "NoisyTopExpertsPerItemRouter")
    _load_project_routers()
    cls, args, kwargs2 = parse_call(name, default_module=ROUTERS)
    merged = {**kwargs2, **kwargs}
    return cls(*args, hidden_size=hidden_size, dtype=dtype, exchange=self.exchange, **merged)

  def forward(self, inputs: Tensor, residual: Optional[Tensor] = None):
    assert inputs.dim() == 3, f"Expected ndim = 3, but got shape {tuple(inputs.shape)}"
    shape = inputs.shape
    total = shape[0] * shape[1]
    if total % self.group_size:
      raise ValueError(f"{total} tokens cannot be split in groups of {self.group_size}")
    x = inputs.reshape(-1, self.group_size, shape[-1])
    dispatcher, metrics = self.Router(x)
    fused = getattr(dispatcher, "apply_experts", None)
    if fused is not None:
      res = None if residual is None else residual.reshape(x.shape)
      out = fused(self.Mlp, x, residual=res)
      return out.reshape(*shape[:-1], out.shape[-1]), metrics
    out = moe.sparse_moe_apply(self.Mlp, dispatcher, x)
    out = out.reshape(*shape[:-1], out.shape[-1])
    if residual is not None:
      out = out + residual
    return out, metrics


class MultiHeadDotProductAttention(nn.Module):
  """Multi-head attention with separate query / key-value inputs and optional QK LayerNorm.

  Self-attention uses one fused QKV projection (a single GEMM with N = 3*hidden).
  """

  def __init__(self, hidden_size: int, num_heads: int, dropout_rate: float = 0.0,
               normalize_qk: bool = False, out_features: Optional[int] = None):
    super().__init__()
    assert hidden_size % num_heads == 0
    self.num_heads = num_heads
    self.head_dim = hidden_size // num_heads
    self.dropout_rate = dropout_rate
    self.qkv = Dense(hidden_size, 3 * hidden_size, kernel_init="zeros")
    for i in range(3):  # query, key, value kernels are initialised independently
      xavier_uniform_(self.qkv.weight[i * hidden_size:(i + 1) * hidden_size], hidden_size,
                      hidden_size)
    self.out = Dense(hidden_size, out_features or hidden_size, kernel_init="xavier_uniform")
    self.query_ln = LayerNorm(self.head_dim, use_bias=False) if normalize_qk else None
    self.key_ln = LayerNorm(self.head_dim, use_bias=False) if normalize_qk else None

  def forward(self, inputs_q: Tensor, inputs_kv: Optional[Tensor] = None,
              residual: Optional[Tensor] = None) -> Tensor:
    b, tq, hdim = inputs_q.shape
    h, d = self.num_heads, self.head_dim
    if inputs_kv is None or inputs_kv is inputs_q:
      qkv = self.qkv(inputs_q).reshape(b, tq, 3, h, d)
      if self.query_ln is None:
        a = ops.attention_packed(qkv, dropout_p=self.dropout_rate, training=self.training)
        return self.out(a.reshape(b, tq, h * d), residual=residual)
      # QK-norm: normalise the query and key slices, re-pack and use the fused kernel.
      from vmoe_b200.ops import norm as norm_ops
      if (ops.cuda_kernels_enabled() and norm_ops.qk_norm_packed_supported(
          qkv, self.query_ln.scale, self.key_ln.scale, self.query_ln.bias, self.key_ln.bias)):
        packed = norm_ops.qk_norm_packed(qkv, self.query_ln.scale, self.key_ln.scale,
                                         self.query_ln.eps)
      else:
        qn, kn = self.query_ln(qkv[:, :, 0]), self.key_ln(qkv[:, :, 1])
        packed = torch.stack([qn, kn, qkv[:, :, 2]], dim=2)
      a = ops.attention_packed(packed, dropout_p=self.dropout_rate, training=self.training)
      return self.out(a.reshape(b, tq, h * d), residual=residual)
    else:
      w, bias = self.qkv.weight, self.qkv.bias
      q = ops.linear(inputs_q, w[:hdim], bias[:hdim]).reshape(b, tq, h, d)
      kv = ops.linear(inputs_kv, w[hdim:], bias[hdim:]).reshape(b, inputs_kv.shape[1], 2, h, d)
      k, v = kv[:, :, 0], kv[:, :, 1]
    if self.query_ln is not None:
      q, k = self.query_ln(q), self.key_ln(k)
    a = ops.attention(q, k, v, dropout_p=self.dropout_rate, training=self.training)
    return self.out(a.reshape(b, tq, h * d), residual=residual)


class MapHead(nn.Module):
  """Multihead attention pooling: a learned probe attends over the tokens."""

  def __init__(self, hidden_size: int, mlp_dim: int, num_heads: int, qk_norm: bool = False):
    super().__init__()
    self.probe = nn.Parameter(torch.empty(1, 1, hidden_size))
    xavier_uniform_(self.probe, hidden_size, hidden_size)
    self.MultiHeadDotProductAttention = MultiHeadDotProductAttention(
        hidden_size, num_heads, normalize_qk=qk_norm)
    self.LayerNorm = LayerNorm(hidden_size)
    self.Mlp = MlpBlock(hidden_size, mlp_dim)

  def forward(self, x: Tensor) -> Tensor:
    probe = self.probe.to(x.dtype).expand(x.shape[0], -1, -1)
    x = self.MultiHeadDotProductAttention(probe, x)
    y = self.Mlp(self.LayerNorm(x))
    return (x + y)[:, 0, :]


class EncoderBlock(nn.Module):
  """Pre-LN transformer block whose MLP is dense or a sparse MoE."""

  def __init__(self, hidden_size: int, num_heads: int, mlp: nn.Module, is_moe: bool,
               dropout_rate: float = 0.0, attention_dropout_rate: float = 0.0,
               attention_qk_norm: bool = False):
    super().__init__()
    self.dropout_rate = dropout_rate
    self.is_moe = is_moe
    self.LayerNorm_0 = LayerNorm(hidden_size)
    self.SelfAttention = MultiHeadDotProductAttention(
        hidden_size, num_heads, dropout_rate=attention_dropout_rate,
        normalize_qk=attention_qk_norm)
    self.LayerNorm_1 = LayerNorm(hidden_size)
    if is_moe:
      self.Moe = mlp
    else:
      self.Mlp = mlp

  def forward(self, inputs: Tensor):
    x, inputs = self.LayerNorm_0.fork(inputs)
    if self.training and self.dropout_rate > 0:
      x = F.dropout(self.SelfAttention(x), self.dropout_rate, True) + inputs
    else:
      x = self.SelfAttention(x, residual=inputs)  # residual add fused in the GEMM epilogue
    y, x = self.LayerNorm_1.fork(x)
    if self.is_moe:
      return self.Moe(y, residual=x)
    return self.Mlp(y, residual=x)


def sincos2d_position_embedding(h: int, w: int, c: int, temperature: float = 10_000.0,
                                dtype=torch.float32, device=None) -> Tensor:
  """MoCo-v3 style fixed 2-D embedding ``(1, h*w, c)``: [sin x, cos x, sin y, cos y]."""
  if c % 4 != 0 or c < 8:
    raise ValueError(f"The hidden_size={c} must be multiple of 4 and >= 8.")
  yy, xx = torch.meshgrid(torch.arange(h, dtype=dtype, device=device),
                          torch.arange(w, dtype=dtype, device=device), indexing="ij")
  yy, xx = yy.flatten(), xx.flatten()
  omega = torch.arange(c // 4, dtype=dtype, device=device) / (c // 4 - 1)
  omega = 1.0 / (temperature ** omega)
  x = xx[:, None] * omega[None, :]
  y = yy[:, None] * omega[None, :]
  return torch.cat([x.sin(), x.cos(), y.sin(), y.cos()], dim=-1)[None]


class AddPositionEmbs(nn.Module):
  """Learned position embedding ``pos_embedding (1, T, H)``, N(0, 0.02) init."""

  def __init__(self, seq_len: int, hidden_size: int):
    super().__init__()
    self.pos_embedding = nn.Parameter(torch.empty(1, seq_len, hidden_size))
    nn.init.normal_(self.pos_embedding, std=0.02)

  def forward(self, x: Tensor) -> Tensor:
    if x.shape[1] != self.pos_embedding.shape[1]:
      raise ValueError(
          f"sequence length {x.shape[1]} != position embedding {self.pos_embedding.shape[1]}")
    return x + self.pos_embedding.to(x.dtype)


class EncoderMoe(nn.Module):
  """Transformer encoder; blocks listed in ``moe['layers']`` use a sparse MoE of MLPs."""

  DEFAULT_SINCOS2D_TEMPERATURE = 10_000.0

  def __init__(self, hidden_size: int, seq_len: int, num_layers: int, mlp_dim: int,
               num_heads: int, dropout_rate: float = 0.0, attention_dropout_rate: float = 0.0,
               attention_qk_norm: bool = False, moe: Optional[KwArgs] = None,
               dtype=None, position_emb: Optional[KwArgs] = None,
               mesh: Optional[mesh_lib.Mesh] = None, moe_block_cls=None):
    super().__init__()
    self.dropout_rate = dropout_rate
    self.dtype = parse_dtype(dtype)
    self.position_emb = dict(position_emb or {})
    name = self.position_emb.get("name", "learned")
    if name == "learned":
      self.posembed_input = AddPositionEmbs(seq_len, hidden_size)
    elif name not in ("none", "sincos2d"):
      raise ValueError(f"Unsupported position embedding: {position_emb}")
    moe_params = {"mlp_dim": mlp_dim, "dropout_rate": dropout_rate, **dict(moe or {})}
    moe_layers = tuple(moe_params.pop("layers", ()))
    self.moe_layers = moe_layers
    self.num_layers = num_layers
    moe_block_cls = moe_block_cls or MlpMoeBlock
    for block in range(num_layers):
      is_moe = block in moe_layers
      if is_moe:
        mlp = moe_block_cls(hidden_size=hidden_size, dtype=self.dtype, mesh=mesh, **moe_params)
      else:
        mlp = MlpBlock(hidden_size, mlp_dim, dropout_rate=dropout_rate)
      self.add_module(
          f"encoderblock_{block}",
          EncoderBlock(hidden_size, num_heads, mlp, is_moe, dropout_rate,
                       attention_dropout_rate, attention_qk_norm))
    self.encoder_norm = LayerNorm(hidden_size)

  def add_position_emb(self, inputs: Tensor) -> Tensor:
    name = self.position_emb.get("name", "learned")
    if name == "none":
      return inputs
    if name == "learned":
      return self.posembed_input(inputs)
    _, n, c = inputs.shape
    h, w = self.position_emb["h"], self.position_emb["w"]
    temperature = self.position_emb.get("temperature", self.DEFAULT_SINCOS2D_TEMPERATURE)
    pe = sincos2d_position_embedding(h, w, c, temperature, device=inputs.device).to(inputs.dtype)
    if n == h * w:
      return inputs + pe
    if n == h * w + 1:
      return torch.cat([inputs[:, :1], inputs[:, 1:] + pe], dim=1)
    raise ValueError(f"Unsupported sequence length n={n} for the given h={h} and w={w}.")

  def forward(self, inputs: Tensor, first_block: int = 0, last_block: Optional[int] = None,
              add_pos: bool = True, final_norm: bool = True):
    assert inputs.dim() == 3, f"Expected ndim = 3, but got shape {tuple(inputs.shape)}"
    x = inputs
    if add_pos:
      x = self.add_position_emb(x)
      if self.training and self.dropout_rate > 0:
        x = F.dropout(x, self.dropout_rate, True)
    metrics: Dict[str, Any] = {}
    last_block = self.num_layers if last_block is None else last_block
    for block in range(first_block, last_block):
      # In backward, the gradient of this tensor means blocks >= `block` have their parameter
      # gradients: the data-parallel reducer starts all-reducing them right away.
      x = grad_allreduce.grad_marker(x, block)
      out = getattr(self, f"encoderblock_{block}")(x)
      if isinstance(out, tuple):
        x, metrics[f"encoderblock_{block}"] = out
      else:
        x = out
    x = grad_allreduce.grad_marker(x, last_block)
    encoded = self.encoder_norm(x) if final_norm else x
    aux = [m["auxiliary_loss"] for m in metrics.values()]
    metrics["auxiliary_loss"] = sum(aux) if aux else torch.zeros((), device=x.device)
    return encoded, metrics


class VisionTransformerMoe(nn.Module):
  """ViT with sparse MoE layers (https://arxiv.org/abs/2106.05974).

  ``image_size`` fixes the token grid (PyTorch parameters are created eagerly); images are
  NHWC ``(B, H, W, C)`` as in the reference's input pipeline.
  """

  encoder_cls = EncoderMoe

  def __init__(self, num_classes: Optional[int], patch_size: Sequence[int], hidden_size: int,
               encoder: KwArgs, classifier: str = "token",
               representation_size: Optional[int] = None, deterministic: bool = False,
               head_bias_init: float = 0.0, head_kernel_zero_init: bool = True,
               image_size: Union[int, Sequence[int]] = 224, num_channels: int = 3,
               mesh: Optional[mesh_lib.Mesh] = None):
    super().__init__()
    if isinstance(image_size, int):
      image_size = (image_size, image_size)
    if isinstance(patch_size, int):
      patch_size = (patch_size, patch_size)
    self.patch_size = tuple(patch_size)
    self.image_size = tuple(image_size)
    self.num_channels = num_channels
    self.hidden_size = hidden_size
    self.classifier = classifier
    self.num_classes = num_classes
    self.deterministic = deterministic
    gh, gw = image_size[0] // patch_size[0], image_size[1] // patch_size[1]
    self.grid = (gh, gw)
    if classifier not in ("token", "0", "gap", "map"):
      raise ValueError(f"Unknown classifier: {classifier!r}")
    seq_len = gh * gw + (1 if classifier == "token" else 0)
    patch_dim = patch_size[0] * patch_size[1] * num_channels
    # Conv with kernel = stride = patch is a GEMM over flattened (ph, pw, c) patches.
    self.embedding = Dense(patch_dim, hidden_size, kernel_init="lecun_normal")
    if classifier == "token":
      self.cls = nn.Parameter(torch.zeros(1, 1, hidden_size))
    encoder_kwargs = dict(encoder)
    self.dtype = parse_dtype(encoder_kwargs.get("dtype"))
    if dict(encoder_kwargs.get("position_emb") or {}).get("name") == "sincos2d":
      pe = dict(encoder_kwargs["position_emb"])
      pe["h"], pe["w"] = gh, gw
      encoder_kwargs["position_emb"] = pe
    self.Encoder = self.encoder_cls(hidden_size=hidden_size, seq_len=seq_len, mesh=mesh,
                                    **encoder_kwargs)
    if classifier == "map":
      self.MapHead = MapHead(hidden_size, encoder["mlp_dim"], encoder["num_heads"],
                             qk_norm=encoder.get("attention_qk_norm", False))
    feat = hidden_size
    if representation_size is not None:
      self.pre_logits = Dense(hidden_size, representation_size)
      feat = representation_size
    else:
      self.pre_logits = None
    if num_classes:
      self.head = Dense(feat, num_classes,
                        kernel_init="zeros" if head_kernel_zero_init else "lecun_normal",
                        bias_init=head_bias_init)
    else:
      self.head = None
    if deterministic:
      self.eval()

  def train(self, mode: bool = True):
    # A model built with deterministic=True never leaves inference mode.
    return super().train(mode and not self.deterministic)

  def patchify(self, images: Tensor) -> Tensor:
    """``(B, H, W, C) -> (B, gh*gw, ph*pw*C)`` in the compute dtype."""
    b, hh, ww, c = images.shape
    ph, pw = self.patch_size
    gh, gw = hh // ph, ww // pw
    if images.is_cuda and self.dtype == torch.bfloat16 and ops.cuda_kernels_enabled():
      from vmoe_b200.ops import elementwise
      return elementwise.patchify(images, ph, pw)
    x = images[:, :gh * ph, :gw * pw].reshape(b, gh, ph, gw, pw, c).permute(0, 1, 3, 2, 4, 5)
    x = x.reshape(b, gh * gw, ph * pw * c)
    return x.to(self.dtype) if self.dtype is not None else x

  def embed(self, images: Tensor) -> Tensor:
    x = self.embedding(self.patchify(images))
    if self.classifier == "token":
      cls = self.cls.to(x.dtype).expand(x.shape[0], -1, -1)
      x = torch.cat([cls, x], dim=1)
    return x

  def pool_and_head(self, x: Tensor) -> Tensor:
    if self.classifier in ("token", "0"):
      x = x[:, 0]
    elif self.classifier == "gap":
      x = x.mean(dim=1)
    else:
      x = self.MapHead(x)
    if self.pre_logits is not None:
      x = torch.tanh(self.pre_logits(x))
    if self.head is not None:
      return self.head(x)
    return x

  def _fused_embed(self, images: Tensor) -> Optional[Tensor]:
    """Patch embedding, class token and learned position embedding with the concat + add done
    by one kernel; None when that path does not apply (then ``embed`` + the encoder's own
    position embedding are used)."""
    enc = self.Encoder
    if not (images.is_cuda and self.dtype == torch.bfloat16 and ops.cuda_kernels_enabled()
            and type(enc).forward is EncoderMoe.forward  # subclasses place pos-emb themselves
            and self.classifier in ("token", "gap", "map", "0")
            and enc.position_emb.get("name", "learned") == "learned"
            and not (self.training and enc.dropout_rate > 0)):
      return None
    from vmoe_b200.ops import elementwise
    x = self.embedding(self.patchify(images))
    has_cls = self.classifier == "token"
    pos = enc.posembed_input.pos_embedding
    if x.shape[-1] % 8 or pos.shape[1] != x.shape[1] + int(has_cls):
      return None
    return elementwise.embed_finalize(x, self.cls if has_cls else None, pos)

  def forward(self, images: Tensor):
    x = self._fused_embed(images)
    if x is not None:
      x, metrics = self.Encoder(x, add_pos=False)
      return self.pool_and_head(x), metrics
    x = self.embed(images)
    x, metrics = self.Encoder(x)
    return self.pool_and_head(x), metrics


ROUTERS: Dict[str, Any] = {
    "NoisyTopExpertsPerItemRouter": routing.NoisyTopExpertsPerItemRouter,
    "NoisyTopItemsPerExpertRouter": routing.NoisyTopItemsPerExpertRouter,
}


def _load_project_routers() -> None:
  """Imports the router modules that live under ``vmoe_b200.projects`` (they register
  themselves), so that configs can name e.g. ``'SoftRouter'`` without a module path."""
  import importlib
  for mod in ("vmoe_b200.projects.soft_moe.router",
              "vmoe_b200.projects.sparsity_constrained_ot.ot_routing"):
    try:
      importlib.import_module(mod)
    except ImportError:
      pass


def register_router(name: str, cls) -> None:
  """Adds a router class to the name registry used by ``MlpMoeBlock``."""
  ROUTERS[name] = cls
