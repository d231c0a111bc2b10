"""Dataset builders and the pipeline's configuration surface, with the process index and count
mocked (reference tests: ``vmoe/data/builder_test.py``, ``vmoe/data/input_pipeline_test.py``)."""
from unittest import mock

import numpy as np
import pytest

from vmoe_b200.data import builder
from vmoe_b200.data import input_pipeline
from vmoe_b200.utils.config_dict import ConfigDict


@pytest.mark.parametrize("process_index, expected", [(0, 1), (1, 1), (2, 2)])
def test_fake_examples_even_out_the_batches_of_all_processes(process_index, expected):
  # 20 examples over 3 processes: 7, 7, 6; batches of 4 -> everybody yields 2 full batches.
  counts = [b - a for a, b in (builder.even_split(0, 20, i, 3) for i in range(3))]
  assert counts == [7, 7, 6]
  assert builder.get_num_fake_examples(process_index, 4, counts) == expected
  assert (counts[process_index] + expected) % 4 == 0


@pytest.mark.parametrize("split, expected", [("validation", 20), ("validation[1:6]", 5),
                                             ("validation[:50%]", 10), ("train[90%:]", 10)])
def test_num_examples_of_sub_splits(split, expected):
  b = builder.get_dataset_builder(name="synthetic", split=split, num_train_examples=100,
                                  num_eval_examples=20, image_size=8)
  assert b.num_examples == expected
  config = ConfigDict({"name": "synthetic", "split": split, "num_train_examples": 100,
                       "num_eval_examples": 20, "image_size": 8, "batch_size": 4,
                       "process": "keep('image')"})
  assert input_pipeline.get_data_num_examples(config) == expected


def test_processes_read_disjoint_parts_that_cover_the_split():
  seen = []
  for index in range(3):
    with mock.patch.object(builder, "_process_index_count", return_value=(index, 3)):
      b = builder.get_dataset_builder(name="synthetic", split="validation", num_eval_examples=10,
                                      image_size=4, num_classes=7)
      part = [int(e["image"].sum()) for e in b.as_dataset()]
    seen.append(part)
  assert [len(p) for p in seen] == [4, 3, 3]
  with mock.patch.object(builder, "_process_index_count", return_value=(0, 1)):
    whole = [int(e["image"].sum()) for e in builder.get_dataset_builder(
        name="synthetic", split="validation", num_eval_examples=10, image_size=4,
        num_classes=7).as_dataset()]
  assert sum(seen, []) == whole


def test_examples_are_deterministic_per_index_and_multi_label():
  b = builder.get_dataset_builder(name="synthetic", split="train", num_train_examples=8,
                                  image_size=4, num_classes=11, multi_label=True, max_positives=3)
  a, c = b.example(5), b.example(5)
  np.testing.assert_array_equal(a["image"], c["image"])
  np.testing.assert_array_equal(a["labels"], c["labels"])
  assert 1 <= len(a["labels"]) <= 3 and a["image"].dtype == np.uint8
  assert not np.array_equal(a["image"], b.example(6)["image"])


def test_unknown_builder_and_wrong_variant_config():
  with pytest.raises((ValueError, NotImplementedError, ImportError)):
    builder.get_dataset_builder(name="tfds:does_not_exist", split="train").as_dataset().__next__()
  with pytest.raises(TypeError, match="The config for the 'variant'"):
    input_pipeline.get_datasets(ConfigDict({"variant": 1}, type_safe=False))


def test_get_datasets_builds_one_iterator_per_variant():
  common = {"name": "synthetic", "batch_size": 2, "image_size": 4, "num_classes": 3,
            "num_train_examples": 8, "num_eval_examples": 5,
            "process": "value_range(-1,1)|onehot(3, inkey='label', outkey='labels')|keep('image','labels')"}
  config = ConfigDict({"train": dict(common, split="train", shuffle_buffer=4),
                       "valid": dict(common, split="validation")}, type_safe=False)
  datasets = input_pipeline.get_datasets(config)
  assert set(datasets) == {"train", "valid"}
  batch = next(iter(datasets["train"]))
  assert batch["image"].shape == (2, 4, 4, 3) and batch["labels"].shape == (2, 3)
  valid = list(datasets["valid"])
  assert len(valid) == 3
  flags = np.concatenate([np.asarray(b["__valid__"]) for b in valid])
  assert flags.tolist() == [True] * 5 + [False]


def _write_image_folder(root, splits):
  from PIL import Image
  rng = np.random.default_rng(0)
  for split, per_class in splits.items():
    for cls, n in per_class.items():
      d = root / split / cls
      d.mkdir(parents=True)
      for i in range(n):
        arr = rng.integers(0, 256, (20 + i, 24, 3), dtype=np.uint8)
        Image.fromarray(arr).save(d / f"img_{i}.png")
      (d / "notes.txt").write_text("not an image")


def test_image_folder_builder_labels_splits_and_pipeline(tmp_path):
  """Files under <root>/<split>/<class>/ with classes numbered alphabetically over all splits;
  decoded and batched by the ordinary process string; the last batch is padded with invalid
  examples."""
  from vmoe_b200.data import builder as builder_lib
  from vmoe_b200.data import input_pipeline
  _write_image_folder(tmp_path, {"train": {"cat": 3, "dog": 2, "emu": 1},
                                 "validation": {"cat": 2, "dog": 1}})
  b = builder_lib.get_dataset_builder(name="folder", split="train", data_dir=str(tmp_path))
  assert b.num_examples == 6 and b.num_classes == 3
  ex = list(b.as_dataset())
  assert [int(e["label"]) for e in ex] == [0, 0, 0, 1, 1, 2]
  assert isinstance(ex[0]["image"], bytes) and ex[0]["file_name"].endswith("img_0.png")
  assert builder_lib.get_dataset_builder(name="folder", split="train[50%:]",
                                         data_dir=str(tmp_path)).num_examples == 3
  ds = input_pipeline.get_dataset(
      variant="val", name="folder", split="validation", batch_size=2, data_dir=str(tmp_path),
      process='decode|resize(16)|value_range(-1,1)|onehot(3, inkey="label", outkey="labels")|'
              'keep("image", "labels")')
  batches = list(ds)
  assert len(batches) == 2
  assert batches[0]["image"].shape == (2, 16, 16, 3) and batches[0]["labels"].shape == (2, 3)
  valid = np.concatenate([np.asarray(b_[input_pipeline.VALID_KEY]) for b_ in batches])
  assert valid.tolist() == [True, True, True, False]
  labels = np.concatenate([np.asarray(b_["labels"]) for b_ in batches])[:3].argmax(-1)
  assert labels.tolist() == [0, 0, 1]
  with pytest.raises(FileNotFoundError):
    builder_lib.get_dataset_builder(name="folder", split="test", data_dir=str(tmp_path)).num_examples
