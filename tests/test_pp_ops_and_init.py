"""Pre-processing ops not covered elsewhere, checkpoint file removal, RNG streams, train-state
norms and initialization from ViT ``.npz`` / Orbax-zarr checkpoints.

Counterparts in the reference: ``vmoe/data/pp_ops_test.py``, ``vmoe/checkpoints/base_test.py``,
``vmoe/utils_test.py``, ``vmoe/train/train_state_test.py``,
``vmoe/initialization/initialization_test.py:98-300``.
"""
import json
import os
import zlib

import numpy as np
import pytest
import torch

from vmoe_b200.checkpoints import base as ckpt_base
from vmoe_b200.data import pp_ops
from vmoe_b200.initialization import initialization
from vmoe_b200.utils import misc


@pytest.fixture(autouse=True)
def _seed_pp_ops():
  pp_ops.set_rng(np.random.default_rng(0))


def _image(h=32, w=48):
  rng = np.random.default_rng(1)
  return rng.integers(0, 256, size=(h, w, 3), dtype=np.uint8)


# ----------------------------------------------------------------------------- pp ops
def test_inception_crop_resizes_and_stays_inside_the_image():
  out = pp_ops.inception_crop(16)({"image": _image()})["image"]
  assert out.shape == (16, 16, 3)
  crop = pp_ops.inception_crop(area_min=20, area_max=60)({"image": _image()})["image"]
  h, w = crop.shape[:2]
  assert 0 < h <= 32 and 0 < w <= 48
  assert 0.15 * 32 * 48 <= h * w <= 0.65 * 32 * 48
  assert 0.7 <= w / h <= 1.4


def test_inception_crop_depends_on_the_rng():
  img = _image()
  pp_ops.set_rng(np.random.default_rng(0))
  a = pp_ops.inception_crop()({"image": img})["image"]
  pp_ops.set_rng(np.random.default_rng(0))
  b = pp_ops.inception_crop()({"image": img})["image"]
  pp_ops.set_rng(np.random.default_rng(5))
  c = pp_ops.inception_crop()({"image": img})["image"]
  assert a.shape == b.shape and np.array_equal(a, b)
  assert a.shape != c.shape or not np.array_equal(a, c)


@pytest.mark.parametrize("h, w, expected", [(32, 48, (16, 24)), (48, 32, (24, 16)),
                                            (8, 8, (16, 16))])
def test_resize_small_keeps_the_aspect_ratio(h, w, expected):
  out = pp_ops.resize_small(16)({"image": _image(h, w)})["image"]
  assert out.shape == expected + (3,)


def test_in_and_out_keys():
  data = {"image": _image(), "other": 1}
  out = pp_ops.resize(8, inkey="image", outkey="small")(dict(data))
  assert out["small"].shape == (8, 8, 3) and out["image"].shape == (32, 48, 3)
  out = pp_ops.resize(8, key="image")(dict(data))
  assert out["image"].shape == (8, 8, 3)


def test_ignore_no_labels_marks_examples_invalid():
  op = pp_ops.ignore_no_labels()
  assert op({"labels": np.array([0.0, 1.0])})["__valid__"]
  assert not op({"labels": np.zeros(3)})["__valid__"]
  assert not op({"labels": np.array([1.0]), "__valid__": False})["__valid__"]


def test_onehot_multi_hot_and_errors():
  out = pp_ops.onehot(5)({"labels": [1, 3]})["labels"]
  assert out.tolist() == [0, 1, 0, 1, 0]
  out = pp_ops.onehot(3, on=0.9, off=0.05)({"labels": 2})["labels"]
  np.testing.assert_allclose(out, [0.05, 0.05, 0.9])
  with pytest.raises(ValueError):
    pp_ops.onehot(5, multi=False)({"labels": [1, 3]})


def test_randaug_keeps_shape_and_dtype_and_changes_pixels():
  img = _image()
  out = pp_ops.randaug(2, 15)({"image": img.copy()})["image"]
  assert out.shape == img.shape and out.dtype == img.dtype
  changed = any(
      not np.array_equal(pp_ops.randaug(2, 15)({"image": img.copy()})["image"], img)
      for _ in range(5))
  assert changed


def test_tokenize_needs_a_model_file_and_pads(tmp_path):
  with pytest.raises(NotImplementedError):
    pp_ops.tokenize(8, model="c4_en")
  spm = pytest.importorskip("sentencepiece")
  corpus = tmp_path / "corpus.txt"
  corpus.write_text("\n".join(["a photo of a cat", "a photo of a dog", "the dog runs fast",
                               "the cat sleeps all day"] * 20))
  prefix = str(tmp_path / "tok")
  spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=40,
                                 model_type="bpe", minloglevel=2)
  op = pp_ops.tokenize(12, model=prefix + ".model", eos="yes")
  ids = op({"text": "a photo of a dog"})["text"]
  assert ids.shape == (12,) and ids.dtype == np.int32
  sp = spm.SentencePieceProcessor(model_file=prefix + ".model")
  n = len(sp.encode("a photo of a dog"))
  assert ids[n] == sp.eos_id() and not ids[n + 1:].any()
  multi = op({"text": np.array([b"the cat sleeps all day", b"the dog runs fast"])})["text"]
  assert multi.shape == (12,)


# ----------------------------------------------------------------------------- checkpoint files
def test_remove_checkpoints_removes_only_matching_files(tmp_path):
  names = ["ckpt_1", "ckpt_2", "ckpt_3.index", "other_1"]
  for name in names:
    (tmp_path / name).write_text("x")
  ckpt_base.remove_checkpoints([str(tmp_path / n) for n in names],
                               lambda fp: os.path.basename(fp) in ("ckpt_1", "ckpt_3.index"))
  assert sorted(os.listdir(tmp_path)) == ["ckpt_2", "other_1"]


def test_latest_complete_checkpoint_ignores_unfinished_steps(tmp_path):
  prefix = str(tmp_path / "ckpt")
  for name in ("ckpt_1", "ckpt_2", ".tmp.ckpt_3", "ckpt_3"):
    (tmp_path / name).write_text("x")
  assert ckpt_base.find_latest_complete_checkpoint_for_prefix(prefix) == prefix + "_2"
  assert list(ckpt_base.iterate_complete_steps_for_prefix(prefix)) == [1, 2]
  assert ckpt_base.find_latest_complete_checkpoint_for_prefix(str(tmp_path / "none")) is None


def test_shard_suffix_round_trip():
  path = ckpt_base.add_shard_suffix("/a/ckpt_1", 3, 16)
  assert path == "/a/ckpt_1-00003-of-00016"
  assert ckpt_base.remove_shard_suffix(path) == "/a/ckpt_1"


# ----------------------------------------------------------------------------- RNG streams
def test_named_rng_streams_are_reproducible_and_independent():
  a = misc.make_rngs(("params", "gating"), seed=3)
  b = misc.make_rngs(("params", "gating"), seed=3)
  c = misc.make_rngs(("params", "gating"), seed=4)
  draw = lambda g: torch.rand(4, generator=g)
  pa, ga = draw(a["params"]), draw(a["gating"])
  assert torch.equal(pa, draw(b["params"])) and torch.equal(ga, draw(b["gating"]))
  assert not torch.equal(pa, ga)
  assert not torch.equal(pa, draw(c["params"]))


def test_rng_split_gives_distinct_children():
  rngs = misc.make_rngs(("dropout", "gating"), seed=0)
  first, second, third = misc.tree_rngs_split(rngs, 3)
  assert set(first) == set(second) == set(third) == {"dropout", "gating"}
  draws = [torch.rand(4, generator=r["dropout"]) for r in (first, second, third)]
  assert not torch.equal(draws[0], draws[1]) and not torch.equal(draws[1], draws[2])
  again = misc.tree_rngs_split(misc.make_rngs(("dropout", "gating"), seed=0), 3)
  assert torch.equal(torch.rand(4, generator=again[0]["dropout"]), draws[0])


# ----------------------------------------------------------------------------- train state
def test_train_state_reports_global_norms_and_counts_steps():
  from vmoe_b200.parallel import mesh as mesh_lib
  from vmoe_b200.train import optimizer as optim
  from vmoe_b200.train import train_state
  model = torch.nn.Linear(2, 1, bias=False)
  with torch.no_grad():
    model.weight.copy_(torch.tensor([[3.0, 4.0]]))
  opt = optim.create_optimizer([("params/kernel", model.weight)], name="sgd", total_steps=10,
                               learning_rate=0.1, momentum=None)
  mesh = mesh_lib.get_auto_logical_mesh(1)
  state = train_state.TrainState(model=model, optimizer=opt, mesh=mesh)
  model.weight.grad.copy_(torch.tensor([[0.6, 0.8]])) if model.weight.grad is not None else \
      setattr(model.weight, "grad", torch.tensor([[0.6, 0.8]]))
  norms = state.apply_gradients_and_compute_global_norms()
  assert state.step == 1
  assert float(norms["grads"]) == pytest.approx(1.0, rel=1e-5)
  assert float(norms["updates"]) == pytest.approx(0.1, rel=1e-5)
  torch.testing.assert_close(model.weight.detach(), torch.tensor([[2.94, 3.92]]))
  assert float(norms["params"]) == pytest.approx(4.9, rel=1e-5)
  saved = state.state_dict()
  assert saved["step"] == 1 and set(saved) >= {"step", "params", "opt_state"}


# ----------------------------------------------------------------------------- initialization
def _target():
  return {"params": {"encoder": {"kernel": np.zeros((4, 3), np.float32),
                                 "bias": np.zeros((3,), np.float32)},
                     "head": {"kernel": np.zeros((3, 2), np.float32)}}}


def test_initialize_from_vit_npz(tmp_path):
  path = str(tmp_path / "vit.npz")
  np.savez(path, **{"Transformer/kernel": np.arange(12, dtype=np.float32).reshape(4, 3),
                    "Transformer/bias": np.ones(3, np.float32),
                    "head/kernel": np.full((3, 5), 7.0, np.float32)})
  rules = [(r"head/.*", None), (r"^Transformer/(.*)$", r"params/encoder/\1")]
  out = initialization.initialize_from_vit(target=_target(), filepath=path, rules=rules,
                                           raise_if_target_unmatched=False)
  np.testing.assert_array_equal(out["params"]["encoder"]["kernel"],
                                np.arange(12, dtype=np.float32).reshape(4, 3))
  np.testing.assert_array_equal(out["params"]["encoder"]["bias"], np.ones(3, np.float32))
  np.testing.assert_array_equal(out["params"]["head"]["kernel"], np.zeros((3, 2), np.float32))
  with pytest.raises(ValueError):
    initialization.initialize_from_vit(target=_target(), filepath=path, rules=rules)


def _write_zarr(directory, name, array, chunks, compressor=None):
  path = os.path.join(directory, name)
  os.makedirs(path)
  meta = {"shape": list(array.shape), "chunks": list(chunks), "dtype": array.dtype.str,
          "order": "C", "compressor": compressor, "fill_value": 0, "zarr_format": 2,
          "filters": None}
  with open(os.path.join(path, ".zarray"), "w") as fp:
    json.dump(meta, fp)
  grid = [range(-(-s // c)) for s, c in zip(array.shape, chunks)]
  import itertools
  for idx in itertools.product(*grid):
    chunk = np.zeros(chunks, array.dtype)
    sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, array.shape))
    part = array[sl]
    chunk[tuple(slice(0, n) for n in part.shape)] = part
    raw = chunk.tobytes()
    if compressor is not None:
      raw = zlib.compress(raw)
    with open(os.path.join(path, ".".join(str(i) for i in idx)), "wb") as fp:
      fp.write(raw)


def test_initialize_from_orbax_reads_chunked_zarr_arrays(tmp_path):
  directory = str(tmp_path / "orbax")
  os.makedirs(directory)
  kernel = np.arange(12, dtype=np.float32).reshape(4, 3)
  _write_zarr(directory, "params.Transformer.kernel", kernel, (3, 2))
  _write_zarr(directory, "params.Transformer.bias", np.ones(3, np.float32), (3,),
              compressor={"id": "zlib", "level": 1})
  structure = initialization.read_orbax_structure(directory)
  assert set(structure["params"]["Transformer"]) == {"kernel", "bias"}
  rules = [(r"^params/Transformer/(.*)$", r"params/encoder/\1")]
  out = initialization.initialize_from_orbax(target=_target(), directory=directory, rules=rules,
                                             raise_if_target_unmatched=False)
  np.testing.assert_array_equal(out["params"]["encoder"]["kernel"], kernel)
  np.testing.assert_array_equal(out["params"]["encoder"]["bias"], np.ones(3, np.float32))
  with pytest.raises(FileNotFoundError):
    initialization.initialize_from_orbax(target=_target(), directory=str(tmp_path / "empty"),
                                         rules=rules)
