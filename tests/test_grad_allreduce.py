"""Range planning of the overlapped gradient all-reduce (host logic, CPU)."""
import torch

from vmoe_b200.parallel import grad_allreduce


def test_plan_ranges_groups_blocks_and_merges_neighbours():
  keys = ["params/embedding/kernel", "params/Encoder/posembed_input/pos_embedding",
          "params/Encoder/encoderblock_0/LayerNorm_0/scale", "params/Encoder/encoderblock_0/Mlp/w",
          "params/Encoder/encoderblock_1/LayerNorm_0/scale", "params/Encoder/encoder_norm/scale",
          "params/head/kernel", "params/Encoder/encoderblock_10/x"]
  sizes = [2048, 1024, 1024, 4096, 1024, 1024, 3072, 1024]
  offsets = [sum(sizes[:i]) for i in range(len(sizes))]
  plan = grad_allreduce.plan_ranges(keys, offsets, sizes, head_tag=11)
  assert plan[0] == [(3072, 5120)]          # both block-0 parameters, merged
  assert plan[1] == [(8192, 1024)]
  assert plan[10] == [(13312, 1024)]        # encoderblock_10 is not mistaken for block 1
  assert plan[11] == [(9216, 4096)]         # encoder_norm + head, merged
  assert plan[grad_allreduce.FINAL_TAG] == [(0, 3072)]
  covered = sorted(r for rs in plan.values() for r in rs)
  assert sum(c for _, c in covered) == sum(sizes)


def test_marker_is_identity_without_reducer():
  x = torch.randn(3, requires_grad=True)
  assert grad_allreduce.grad_marker(x, 0) is x
