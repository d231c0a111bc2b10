"""Schedules, optimizer, tree summarizer, mixup, utils, config dict (CPU)."""
import math

import numpy as np
import pytest
import torch

from vmoe_b200.train import optimizer as optim
from vmoe_b200.train import schedule, trainer
from vmoe_b200.train.tree_summarizer import TreeSummarizer
from vmoe_b200 import utils


def test_warmup_polynomial_decay_schedule():
  fn = schedule.warmup_polynomial_decay_schedule(peak_value=0.1, end_value=0.01, power=0.5,
                                                 warmup_steps=5, decay_steps=10)
  got = [fn(i) for i in range(15)]
  exp = [0.0, 0.02, 0.04, 0.06, 0.08, 0.1] + [(0.1 - 0.01) * (1 - i / 5) ** 0.5 + 0.01 for i in (1, 2, 3, 4)] + [0.01] * 5
  np.testing.assert_allclose(got, exp, rtol=1e-5)


def test_big_vision_rsqrt_schedule():
  fn = schedule.big_vision_rsqrt_schedule(peak_value=0.1, decay_steps=12, warmup_steps=4,
                                          cooldown_steps=3, timescale=2)
  exp = [0.0, 0.025, 0.05, 0.075, 0.1] + [0.1 / math.sqrt(1 + i / 2) for i in (1, 2, 3, 4)] + \
        [0.1 / math.sqrt(1 + 5 / 2) * (1 - i / 3) for i in (0, 1, 2)]
  np.testing.assert_allclose([fn(i) for i in range(12)], exp, rtol=1e-5)


def test_create_learning_rate_schedule():
  fn = schedule.create_learning_rate_schedule(schedule="warmup_exponential_decay", total_steps=10,
                                              peak_value=0.1, warmup_steps=4, transition_steps=1,
                                              decay_rate=0.9)
  v = [fn(i) for i in range(10)]
  assert abs(v[0]) < 1e-6 and abs(v[4] - 0.1) < 1e-6 and abs(v[8] - 0.1 * 0.9 ** 4) < 1e-6
  fn = schedule.create_learning_rate_schedule(schedule="warmup_cosine_decay", total_steps=10,
                                              peak_value=1.0, warmup_steps=2)
  assert abs(fn(2) - 1.0) < 1e-6 and abs(fn(10)) < 1e-6 and abs(fn(6) - 0.5) < 1e-6
  assert schedule.create_learning_rate_schedule(schedule="constant", total_steps=3, value=0.3)(2) == 0.3
  with pytest.raises(ValueError, match="Unknown learning rate schedule"):
    schedule.create_learning_rate_schedule(schedule="foo_bar", total_steps=10)


def _mccormick(x):
  a, b = x[0], x[1]
  return torch.sin(a + b) + (a - b) ** 2 - 1.5 * a + 2.5 * b + 1


@pytest.mark.parametrize("name,kw,lr,steps", [("adam", {}, 0.1, 200), ("sgd", {"momentum": 0.9}, 0.01, 200),
                                              ("big_vision_adafactor", {}, 0.05, 400)])
def test_optimizers_minimise_mccormick(name, kw, lr, steps):
  x = torch.nn.Parameter(torch.zeros(2))
  opt = optim.create_optimizer([("params/x", x)], name=name, total_steps=steps, learning_rate=lr, **kw)
  for _ in range(steps):
    opt.zero_grad()
    _mccormick(x).backward()
    opt.step()
  np.testing.assert_allclose(x.detach().numpy(), [-0.54719, -1.54719], atol=2e-3)


def test_optimizer_weight_decay_freeze_scale_and_clip():
  a = torch.nn.Parameter(torch.ones(3)); b = torch.nn.Parameter(torch.ones(3)); c = torch.nn.Parameter(torch.ones(3))
  opt = optim.create_optimizer(
      [("params/a/kernel", a), ("params/b/bias", b), ("params/c/kernel", c)], name="sgd",
      total_steps=1, learning_rate=0.5, weight_decay=[("a/kernel", 0.1)], frozen_pattern="c/",
      gradient_scale=[("b/", 2.0)], gradient_clip={"absolute_value": 1.5})
  opt.zero_grad()
  for p in (a, b, c):
    p.grad.add_(1.0)
  norms = opt.step()
  np.testing.assert_allclose(a.detach().numpy(), 1 - 0.5 * (1 + 0.1), rtol=1e-6)
  np.testing.assert_allclose(b.detach().numpy(), 1 - 0.5 * 1.5, rtol=1e-6)  # scaled to 2, clipped to 1.5
  np.testing.assert_allclose(c.detach().numpy(), 1.0)
  assert set(norms) == {"grads", "updates", "params"}
  with pytest.raises(ValueError, match="cannot specify both"):
    optim.make_frozen_fn("a", "b")
  with pytest.raises(ValueError, match="but not both"):
    optim.check_gradient_clip(1.0, 1.0)
  with pytest.raises(ValueError, match="Unknown optimizer"):
    optim.create_optimizer([("x", a)], name="foo", total_steps=1, learning_rate=0.1)


def test_global_norm_clip():
  a = torch.nn.Parameter(torch.zeros(4))
  opt = optim.create_optimizer([("params/a", a)], name="sgd", total_steps=1, learning_rate=1.0,
                               gradient_clip={"global_norm": 1.0})
  opt.zero_grad(); a.grad.add_(torch.tensor([3., 0., 4., 0.]))
  norms = opt.step()
  np.testing.assert_allclose(a.detach().numpy(), [-0.6, 0, -0.8, 0], atol=1e-6)
  assert abs(float(norms["grads"]) - 5.0) < 1e-5


@pytest.mark.parametrize("transforms,suffix,expected", [
    ((), "", [[1], [2], [3]]), (("sum",), "_sum", 6), (("std",), "_std", math.sqrt(2 / 3)),
    (("norm",), "_norm", math.sqrt(14)), ((("norm", (1, 0)),), "_norm(1, 0)", math.sqrt(14))])
def test_tree_summarizer_transform(transforms, suffix, expected):
  value = torch.tensor([[1.], [2.], [3.]])
  got_suffix, out = TreeSummarizer._transform(value, transforms)
  assert got_suffix == suffix
  np.testing.assert_allclose(out.numpy().squeeze(), np.asarray(expected, np.float32).squeeze(), rtol=1e-6)


def test_tree_summarizer_rules():
  tree = {"params": {"dense": {"w": torch.tensor([[1., 2., 3., 4.]])},
                     "moe": {"w": torch.tensor([[1., 2.], [3., 4.]])}},
          "opt_state": {"learning_rate": torch.tensor(1.0)}}
  s = TreeSummarizer(rules=[".*/learning_rate", (".*/dense/w", "norm"), (".*/moe/w", ("norm", (1,)))],
                     max_summary_values=2)
  out = {k: float(v) for k, v in s(tree)}
  exp = {"params/dense/w_norm": math.sqrt(30), "params/moe/w_norm(1,)[0]": math.sqrt(5),
         "params/moe/w_norm(1,)[1]": 5.0, "opt_state/learning_rate": 1.0}
  assert out.keys() == exp.keys()
  for k in exp:
    assert abs(out[k] - exp[k]) < 1e-5
  with pytest.raises(ValueError, match="Operation op='foo'"):
    TreeSummarizer._transform(torch.zeros(5), ("foo",))
  with pytest.raises(ValueError, match="generates 4 > 1"):
    dict(TreeSummarizer(rules=[(".*/moe/w",)])(tree))


def test_mixup_keeps_largest_weight_on_own_example():
  x = torch.eye(4).reshape(1, 4, 4)
  out = trainer.mixup(torch.Generator().manual_seed(0), (x,), concentration=1.0, shape=(1, 1, 2),
                      roll_axis=1)[0][0]
  assert torch.allclose(out.sum(-1), torch.ones(4))
  assert (out.diagonal() >= 0.5).all()
  with pytest.raises(ValueError, match="must be greater than 0"):
    trainer.mixup(None, (x,), concentration=0.0)
  with pytest.raises(ValueError, match="length >= 2"):
    trainer.mixup(None, (x,), concentration=1.0, shape=(2,))


def test_get_train_steps_and_epochs():
  assert trainer.get_train_steps_and_epochs(train_batch_size=10, train_examples=100, train_epochs=2) == (20, 2.0)
  assert trainer.get_train_steps_and_epochs(train_batch_size=10, train_examples=100, train_steps=5) == (5, 0.5)
  with pytest.raises(ValueError):
    trainer.get_train_steps_and_epochs(train_batch_size=1, train_examples=1)


def test_parse_call_and_friends():
  fn, args, kwargs = utils.parse_call("sqrt(4)", math)
  assert fn is math.sqrt and args == (4,) and kwargs == {}
  fn, args, kwargs = utils.parse_call("math.floor", None)
  assert fn is math.floor and args == ()
  fn, args, kwargs = utils.parse_call("foo(1, k='v')", {"foo": len})
  assert fn is len and args == (1,) and kwargs == {"k": "v"}
  with pytest.raises(ValueError):
    utils.parse_call("foo.bar().baz", None)
  cls = utils.partialclass(dict, a=1)
  assert cls(b=2) == {"a": 1, "b": 2}
  assert list(utils.safe_zip([1, 2], [3, 4])) == [(1, 3), (2, 4)]
  with pytest.raises(utils.SafeZipIteratorError):
    list(utils.safe_zip([1, 2], [3]))
  fn = utils.make_match_fn_from_regex_list(["a.c", "^x"])
  assert fn("zabc") and fn("xy") and not fn("yx")
  assert utils.make_match_fn_from_regex_list(None) is None
  out = utils.multiply_no_nan(torch.tensor([0., 2.]), torch.tensor([float("inf"), 3.]))
  assert out.tolist() == [0.0, 6.0]
  assert sorted(["a_11", "a_2", "a_0"], key=utils.natural_sort_key) == ["a_0", "a_2", "a_11"]


def test_config_dict():
  c = utils.ConfigDict({"a": {"b": 1}, "c": 2.0})
  c.a.b = 3
  c.lock()
  with pytest.raises(KeyError):
    c.z = 1
  with c.unlocked():
    c.z = 1
  assert c.to_dict() == {"a": {"b": 3}, "c": 2.0, "z": 1} and "a.b" in c
  with pytest.raises(TypeError):
    c.c = "x"
  c["a.b"] = 5
  assert c.get("a").b == 5 and c.get("nope", 7) == 7
  ref = utils.placeholder(int)
  d = utils.ConfigDict({"x": ref, "y": ref})
  d.x = 4
  assert d.y == 4 and d.copy_and_resolve_references().to_dict() == {"x": 4, "y": 4}


def test_hardware_and_logical_mesh_views():
  import numpy as np
  from vmoe_b200.parallel import mesh as mesh_lib
  from vmoe_b200.parallel import partitioning
  hw = partitioning.get_hardware_mesh(16, 8)
  assert hw.shape == (8, 2) and hw[3, 1] == 11
  lm = partitioning.get_logical_mesh(8, hw)     # 8 expert partitions, 2 replicas
  assert lm.shape == (8, 2)
  assert sorted(lm[:, 0]) == list(range(8))     # one expert group = the GPUs of node 0
  assert partitioning.processes_have_contiguous_device_slices(lm, 8)
  # Same assignment as the mesh every process builds for itself.
  assert np.array_equal(lm, np.asarray(mesh_lib.mesh_layout(16, 8)))
  lm4 = partitioning.get_logical_mesh(4, hw)    # two expert groups per node
  assert np.array_equal(lm4, np.asarray(mesh_lib.mesh_layout(16, 4)))
  x = object()
  assert partitioning.with_sharding_constraint(x, ("expert",)) is x


def test_weight_gradient_split_factor_fills_whole_rounds_of_cta_pairs():
  """``_wgrad_split`` cuts the contraction of a weight-gradient GEMM so that tiles x pieces fill
  whole rounds of the 74 CTA pairs: 27 tiles (qkv of ViT-B) take 5 pieces (135 items, two rounds),
  9 tiles (out-projection) take 8, 36 tiles (fc1 / fc2) take 2 (72 of 74 pairs); large outputs
  and short contractions are not split."""
  from vmoe_b200.ops.functional import _wgrad_split
  rows = 512 * 197
  assert _wgrad_split(2304, 768, rows) == 5
  assert _wgrad_split(768, 768, rows) == 8
  assert _wgrad_split(3072, 768, rows) == 2 and _wgrad_split(768, 3072, rows) == 2
  assert _wgrad_split(21843, 768, rows) == 1      # 258 tiles: more than two rounds already
  assert _wgrad_split(2304, 768, 2048) == 1       # too few rows to be worth cutting
  for n, k in ((1024, 1024), (3840, 1280), (512, 512)):
    s = _wgrad_split(n, k, rows)
    assert 1 <= s <= 16 and s <= rows // 2048
