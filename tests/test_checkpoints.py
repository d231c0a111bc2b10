"""Checkpoint format: types, serialization, base discovery, partitioned save/restore, rules."""
import os

import numpy as np
import pytest
import torch

from vmoe_b200.checkpoints import base, flax_layout, partitioned, serialization
from vmoe_b200.checkpoints.types import (ArrayChunks, IndexInfo, LazyArrayChunks, ShapedArray, Slice,
                                         SliceNd, SliceNdArray)
from vmoe_b200.initialization import mapping, rules
from vmoe_b200.parallel.mesh import Mesh


def test_slice_types():
  assert Slice(1, 5) == slice(1, 5) and Slice(1, 5) < Slice(2, 3) and hash(Slice(3)) == hash(Slice(None, 3))
  assert repr(Slice()) == "Slice()" and repr(Slice(3)) == "Slice(3)" and repr(Slice(1, 2, 3)) == "Slice(1, 2, 3)"
  s = SliceNd(Slice(0, 2), Slice(1, 3))
  assert s.chunk(np.arange(12).reshape(3, 4)).tolist() == [[1, 2], [5, 6]]
  assert SliceNd([slice(0, 2)]) == SliceNd(Slice(0, 2))
  arr = SliceNdArray.create([[slice(0, 1)], [slice(1, 2)]], shape=(2,), tile=(2,))
  assert arr.shape == (4,) and arr[2] == SliceNd(Slice(0, 1))
  with pytest.raises(ValueError):
    SliceNd(1, 2)


def test_serialization_roundtrip_of_custom_types():
  import ml_dtypes
  tree = {
      "a": np.arange(6, dtype=np.float32).reshape(2, 3), "b": np.float32(1.5), "c": 3 + 4j, "d": 7,
      "bf": np.arange(4).astype(ml_dtypes.bfloat16),
      "s": Slice(1, 2), "nd": SliceNd(Slice(0, 2), Slice(2, 4)),
      "nda": SliceNdArray.create([[slice(0, 1)], [slice(1, 2)]], shape=(2,)),
      "ii": IndexInfo(ShapedArray((4, 6), np.float32), [SliceNd(Slice(0, 4), Slice(0, 6))], [0]),
      "sa": ShapedArray((2,), "bfloat16", False),
  }
  out = serialization.msgpack_restore(serialization.msgpack_serialize(tree))
  np.testing.assert_array_equal(out["a"], tree["a"])
  assert out["b"] == np.float32(1.5) and out["c"] == 3 + 4j and out["d"] == 7
  assert out["bf"].dtype.name == "bfloat16" and out["s"] == Slice(1, 2) and out["nd"] == tree["nd"]
  assert out["nda"].shape == (2,) and out["ii"].global_shape.shape == (4, 6) and out["ii"].shards == (0,)
  assert out["sa"].dtype.name == "bfloat16"
  lac = LazyArrayChunks()
  lac.add(3, np.arange(12.).reshape(3, 4), SliceNd(Slice(0, 2), Slice(0, 4)), SliceNd(Slice(4, 6), Slice(0, 4)))
  chunks = serialization.msgpack_restore(serialization.msgpack_serialize(lac))
  assert isinstance(chunks, ArrayChunks)
  (chunk, gs), = list(chunks.iter_chunks(3))
  assert chunk.shape == (2, 4) and gs == SliceNd(Slice(4, 6), Slice(0, 4))


def test_ndarray_wire_layout():
  """ndarray ext payload is msgpack (shape, dtype name, C-order bytes)."""
  import msgpack
  raw = serialization._ndarray_to_bytes(np.arange(3, dtype=np.int16))
  shape, name, buf = msgpack.unpackb(raw, raw=True)
  assert shape == [3] and name == b"int16" and buf == np.arange(3, dtype=np.int16).tobytes()


def test_base_save_restore_and_discovery(tmp_path):
  p = str(tmp_path / "ckpt_3")
  base.save_checkpoint(p, {"x": np.ones(3)})
  assert base.restore_checkpoint(p)["x"].tolist() == [1, 1, 1]
  assert base.add_shard_suffix("a", 1, 3) == "a-00001-of-00003"
  assert base.remove_shard_suffix("ckpt_1.data-00000-of-00010") == "ckpt_1.data"
  d = str(tmp_path / "dd")
  os.makedirs(d)
  for f in ["ckpt_1.index", "ckpt_1.data", "ckpt_2.index", ".tmp.ckpt_2.data", "ckpt_3.data"]:
    open(os.path.join(d, f), "w").close()
  prefix = os.path.join(d, "ckpt")
  assert list(base.iterate_complete_steps_for_prefix(prefix, suffixes=[".index", ".data"])) == [1]
  assert base.find_latest_complete_checkpoint_for_prefix(prefix, [".index", ".data"]) == prefix + "_1"
  res = base.save_multiple_checkpoints_async({str(tmp_path / "m_1"): {"a": np.zeros(2)},
                                              str(tmp_path / "m_2"): {"a": np.ones(2)}})
  res.get()
  out = base.restore_multiple_checkpoints({str(tmp_path / "m_1"): None, str(tmp_path / "m_2"): None})
  assert out[str(tmp_path / "m_2")]["a"].tolist() == [1, 1]


@pytest.mark.parametrize("slicend,max_items,expected", [
    ((), None, [()]),
    (((0, 5),), 3, [((i, i + 1),) for i in range(5)]),
    (((0, 2), (4, 8)), None, [((0, 2), (4, 8))]),
    (((0, 2), (4, 8)), 4, [((0, 1), (4, 8)), ((1, 2), (4, 8))]),
    (((0, 2), (4, 8)), 2, [((0, 1), (4, 6)), ((0, 1), (6, 8)), ((1, 2), (4, 6)), ((1, 2), (6, 8))]),
    (((0, 2), (4, 8)), 1, [((i, i + 1), (j, j + 1)) for i in range(2) for j in range(4, 8)])])
def test_split_slicend(slicend, max_items, expected):
  mk = lambda s: SliceNd(*[Slice(*t) for t in s])
  assert set(partitioned._split_slicend(mk(slicend), max_items)) == {mk(e) for e in expected}


def test_greedy_shard_assignment():
  holders = {SliceNd(Slice(0, 2)): [0, 1], SliceNd(Slice(2, 4)): [1], SliceNd(Slice(4, 6)): [0, 1]}
  bytes_per = [0, 0, 0, 0]
  out = partitioned._create_map_slicend_to_checkpoint_shard(holders, 4, bytes_per, process_count=2)
  assert out[SliceNd(Slice(2, 4))] % 2 == 1
  assert sum(bytes_per) == 24 and max(bytes_per) == 8
  assert partitioned._find_smallest_ckpt_shard([5, 1, 3, 0], (1,), 2) == 3


def test_partitioned_roundtrip_and_resharding(tmp_path):
  full = np.arange(4 * 6, dtype=np.float32).reshape(4, 6)
  bf = torch.arange(8.).bfloat16()
  prefix = str(tmp_path / "ck_5")
  for rank in range(2):
    mesh = Mesh(world_size=2, rank=rank, num_partitions=2)
    tree = {"w": full[rank * 2:(rank + 1) * 2], "r": {"b": bf}, "step": np.asarray(5)}
    partitioned.save_checkpoint(prefix, tree, shardings={"w": ("expert",), "r": {"b": None}, "step": None},
                                mesh=mesh, max_chunk_bytes=16).get()
  files = sorted(os.listdir(tmp_path))
  assert files == ["ck_5.data-00000-of-00002", "ck_5.data-00001-of-00002", "ck_5.index"]
  out = partitioned.restore_checkpoint(prefix, mesh=Mesh())
  np.testing.assert_array_equal(out["w"], full)
  assert out["r"]["b"].dtype.name == "bfloat16" and int(out["step"]) == 5
  out = partitioned.restore_checkpoint(prefix, shardings={"w": ("expert",), "r": {"b": None}, "step": None},
                                       mesh=Mesh(world_size=2, rank=1, num_partitions=2))
  np.testing.assert_array_equal(out["w"], full[2:])
  idx = partitioned.read_index(prefix)
  assert idx["version"] == "20220622" and idx["shard_count"] == 2
  assert idx["index"]["w"].global_shape.shape == (4, 6)
  # A legacy index (no version) needs a target tree.
  legacy = dict(idx); legacy.pop("version")
  base.save_checkpoint(prefix + ".index", legacy)
  with pytest.raises(ValueError, match="must specify the tree"):
    partitioned.restore_checkpoint(prefix, mesh=Mesh())
  out = partitioned.restore_checkpoint(prefix, {"w": None, "r": {"b": None}, "step": None}, mesh=Mesh())
  np.testing.assert_array_equal(out["w"], full)


def test_map_state_dict_rules():
  src = {"a_0": np.zeros(2), "a_1": np.ones(2), "a_2": 2 * np.ones(2), "a_11": 11 * np.ones(2),
         "b": np.arange(6.).reshape(1, 6), "drop": np.zeros(3), "t": np.ones((2,))}
  tgt = {"A": np.zeros((4, 2)), "B": np.zeros(6), "C": np.full(3, 7.), "T": np.zeros((3, 2), np.float32)}
  out = mapping.map_state_dict(
      src, tgt, [(r"a_\d+", "A", "stack", 0), ("^b$", "B", "squeeze", 0), ("drop", None),
                 ("^t$", "T", "expand_tile", 0, 3)], raise_if_target_unmatched=False)
  assert out["A"][:, 0].tolist() == [0, 1, 2, 11] and out["B"].tolist() == list(range(6))
  assert out["C"].tolist() == [7, 7, 7] and out["T"].shape == (3, 2) and out["T"].dtype == np.float32
  with pytest.raises(KeyError, match="does not match any rule"):
    mapping.map_state_dict({"zz": np.zeros(1)}, {"zz": np.zeros(1)}, [("a", "b")])
  with pytest.raises(ValueError, match="is unmatched"):
    mapping.map_state_dict({"a": np.zeros(1)}, {"a": np.zeros(1), "q": np.zeros(1)}, [("a", "a")])
  with pytest.raises(ValueError, match="mismatched shapes"):
    mapping.map_state_dict({"a": np.zeros(2)}, {"a": np.zeros(3)}, [("a", "a")])
  with pytest.raises(ValueError, match="cannot be parsed"):
    rules.Rules.parse([("a", "b", "frobnicate")])


def test_vit_zoom():
  pe = np.random.default_rng(0).normal(size=(1, 1 + 49, 8)).astype(np.float32)
  out = rules.VitZoomTransformation(target=np.zeros((1, 1 + 144, 8), np.float32), source=pe)()
  assert out.shape == (1, 145, 8)
  np.testing.assert_array_equal(out[:, 0], pe[:, 0])
  out = rules.VitZoomTransformation(target=np.zeros((1, 49, 8), np.float32), source=pe)()
  np.testing.assert_allclose(out, pe[:, 1:], atol=1e-6)
  tgt = np.full((1, 1 + 16, 8), 3.0, np.float32)
  out = rules.VitZoomTransformation(target=tgt, source=pe[:, 1:])()
  np.testing.assert_array_equal(out[:, 0], tgt[:, 0])
  with pytest.raises(ValueError, match="neither a perfect square"):
    rules.VitZoomTransformation(target=np.zeros((1, 12, 8)), source=pe)()


def test_flax_layout_names_and_roundtrip():
  from vmoe_b200.models.vit_moe import VisionTransformerMoe
  from vmoe_b200.utils.misc import flatten_dict
  mk = lambda: VisionTransformerMoe(
      num_classes=10, patch_size=(32, 32), hidden_size=64, image_size=64, representation_size=32,
      encoder=dict(num_layers=2, mlp_dim=128, num_heads=4, moe=dict(
          layers=(1,), num_experts=4, group_size=10,
          router=dict(num_selected_experts=2, dispatcher=dict(name="einsum", capacity=8, batch_priority=True)))))
  torch.manual_seed(0)
  m, m2 = mk(), mk()
  params, specs = flax_layout.to_flax(m)
  flat = {k: v.shape for k, v in flatten_dict(params, sep="/").items()}
  assert flat["Encoder/encoderblock_0/SelfAttention/query/kernel"] == (64, 4, 16)
  assert flat["Encoder/encoderblock_0/SelfAttention/query/bias"] == (4, 16)
  assert flat["Encoder/encoderblock_0/SelfAttention/out/kernel"] == (4, 16, 64)
  assert flat["Encoder/encoderblock_0/Mlp/Dense_0/kernel"] == (64, 128)
  assert flat["Encoder/encoderblock_1/Moe/Mlp/Dense_0/kernel"] == (4, 64, 128)
  assert flat["Encoder/encoderblock_1/Moe/Mlp/Dense_1/bias"] == (4, 64)
  assert flat["Encoder/encoderblock_1/Moe/Router/dense/kernel"] == (64, 4)
  assert flat["embedding/kernel"] == (32, 32, 3, 64) and flat["head/kernel"] == (32, 10)
  assert flat["cls"] == (1, 1, 64) and flat["Encoder/posembed_input/pos_embedding"] == (1, 5, 64)
  assert flat["pre_logits/kernel"] == (64, 32)
  assert specs["Encoder"]["encoderblock_1"]["Moe"]["Mlp"]["Dense_0"]["kernel"] == ("expert",)
  assert specs["head"]["kernel"] is None
  flax_layout.from_flax(m2, params)
  x = torch.rand(4, 64, 64, 3)
  m.eval(); m2.eval()
  torch.testing.assert_close(m(x)[0], m2(x)[0])
