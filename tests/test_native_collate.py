"""Multi-threaded host collate against NumPy. The library holds only host code for these
calls, so the tests run wherever it has been built (they are skipped otherwise)."""
import numpy as np
import pytest

from vmoe_b200.data import input_pipeline
from vmoe_b200.data import native

needs_lib = pytest.mark.skipif(native._library() is None,
                               reason="libvmoe_b200.so has not been built")


@needs_lib
@pytest.mark.parametrize("dtype", [np.uint8, np.float32, np.int64, np.float16])
@pytest.mark.parametrize("n, shape", [(1, (3,)), (7, (5, 4, 3)), (130, (16, 16, 3))])
@pytest.mark.parametrize("threads", [0, 1, 3])
def test_stack_matches_numpy(dtype, n, shape, threads):
  rng = np.random.default_rng(0)
  arrays = [(rng.random(shape) * 100).astype(dtype) for _ in range(n)]
  got = native.stack(arrays, threads=threads, min_bytes=0)
  want = np.stack(arrays)
  assert got.dtype == want.dtype and got.shape == want.shape
  np.testing.assert_array_equal(got, want)


@needs_lib
def test_stack_into_a_given_buffer_and_zero_sized_examples():
  arrays = [np.full((4, 4), i, np.float32) for i in range(9)]
  out = np.empty((9, 4, 4), np.float32)
  assert native.stack(arrays, out=out, min_bytes=0) is out
  np.testing.assert_array_equal(out, np.stack(arrays))
  empty = native.stack([np.zeros((0, 3), np.float32)] * 4, min_bytes=0)
  assert empty.shape == (4, 0, 3)
  with pytest.raises(ValueError):
    native.stack(arrays, out=np.empty((9, 4, 5), np.float32))
  with pytest.raises(ValueError):
    native.stack([])


@needs_lib
@pytest.mark.parametrize("vmin, vmax", [(-1.0, 1.0), (0.0, 1.0)])
def test_u8_to_f32_matches_value_range(vmin, vmax):
  rng = np.random.default_rng(1)
  arrays = [rng.integers(0, 256, size=(8, 8, 3), dtype=np.uint8) for _ in range(33)]
  got = native.stack_u8_to_f32(arrays, vmin, vmax, threads=4, min_bytes=0)
  want = np.stack(arrays).astype(np.float32) / 255.0 * (vmax - vmin) + vmin
  assert got.dtype == np.float32
  np.testing.assert_allclose(got, want, rtol=0, atol=1e-6)
  out = np.empty_like(got)
  assert native.stack_u8_to_f32(arrays, vmin, vmax, out=out, min_bytes=0) is out
  np.testing.assert_array_equal(out, got)
  with pytest.raises(ValueError):
    native.stack_u8_to_f32([a.astype(np.float32) for a in arrays], vmin, vmax)


def test_fallbacks_without_the_native_path():
  # Mixed shapes cannot be stacked by either path; non-contiguous and small inputs go to NumPy.
  base = np.arange(24, dtype=np.float32).reshape(4, 6)
  views = [base[:, ::2], base[:, 1::2]]
  np.testing.assert_array_equal(native.stack(views, min_bytes=0), np.stack(views))
  small = [np.ones(3, np.float32)] * 2
  np.testing.assert_array_equal(native.stack(small), np.stack(small))
  got = native.stack_u8_to_f32([np.full((2, 2), 255, np.uint8)] * 2, -1.0, 1.0)
  np.testing.assert_allclose(got, np.ones((2, 2, 2), np.float32))


def test_pipeline_batches_go_through_the_collate():
  examples = [{"image": np.full((2, 2, 3), i, np.uint8), "label": np.int64(i)} for i in range(5)]
  batch = input_pipeline._stack(examples)
  assert batch["image"].shape == (5, 2, 2, 3) and batch["label"].tolist() == [0, 1, 2, 3, 4]
