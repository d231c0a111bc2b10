"""Headline benchmark: V-MoE B/16 (8 experts on every odd block, K=2, capacity 1.05, Batch
Priority Routing) bf16 training throughput in images/s on N B200 GPUs of one node.

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port 29511 bench.py --gpus 8 --steps 10 --warmup 3

Weak scaling: 512 images per GPU (global batch 4096 on 8 GPUs); the expert axis is
min(8, N) so that at 8 GPUs every GPU holds one expert. Synthetic images uniform[-1, 1],
21843-way multi-hot labels (1-3 positives), sigmoid cross-entropy, Adam (b2 0.999, wd 0.1),
random-init weights. Two numbers are measured over the same K steps each:

* ``value``: device-timed (CUDA events, max over ranks) with the step inputs already on the
  GPU; every step is the full forward + backward + gradient reduction + optimizer update.
* ``e2e``: the same step driven through ``vmoe_b200.train.trainer.train_step`` with, every
  step, the host->device copy of that step's images and labels from pinned host memory and a
  device->host read of the step's loss.

Rank 0 prints one JSON line. ``--impl reference`` times the unmodified reference (JAX / Flax,
``baseline/run_reference.py``) when its dependencies are installed and prints an ``unavailable``
line otherwise.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys

MODEL_DESC = "ViT-B/16, E=8, K=2, Every 2"
NUM_CLASSES = 21843
IMAGE_SIZE = 224
PER_GPU_BATCH = 512


def parse_args():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=8)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="vmoe_b200", choices=["vmoe_b200", "reference"])
  ap.add_argument("--per-gpu-batch", type=int, default=PER_GPU_BATCH)
  ap.add_argument("--global-batch", type=int, default=None,
                  help="total images per step over all GPUs (overrides --per-gpu-batch)")
  ap.add_argument("--model", default=MODEL_DESC)
  ap.add_argument("--library-ops", action="store_true",
                  help="run PyTorch library ops instead of the package's kernels (stand-in baseline)")
  ap.add_argument("--skip-e2e", action="store_true")
  ap.add_argument("--mode", default="train", choices=["train", "eval"],
                  help="eval: forward-only evaluation steps (loss and precision sums) at capacity "
                       "ratio 1.0, no optimizer")
  ap.add_argument("--ensemble-size", type=int, default=1,
                  help=">1: the ensemble-of-experts variant (inputs repeated per member, experts "
                       "split into that many groups)")
  ap.add_argument("--num-partitions", type=int, default=0,
                  help="size of the 'expert' mesh axis (default: all GPUs, at most 8); smaller "
                       "values replicate every expert shard over world / num_partitions ranks")
  return ap.parse_args()


def reference_arm(args) -> int:
  """Runs the unmodified reference tree under ``baseline/_ref`` through its own training step
  (``baseline/run_reference.py``) when its dependencies (jax, flax, optax, ml_collections ...)
  can be imported; otherwise prints the ``unavailable`` line. Rank 0 only: JAX drives all local
  GPUs from one process."""
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return 0
  here = os.path.dirname(os.path.abspath(__file__))
  for p in (os.path.join(here, "baseline", "_ref"), here):
    if p not in sys.path:
      sys.path.insert(0, p)
  try:
    import jax  # noqa: F401
    import flax  # noqa: F401
    import optax  # noqa: F401
    import vmoe  # noqa: F401
    from baseline import run_reference
  except Exception as e:  # pylint: disable=broad-except
    why = (f"the reference's dependencies are not installed: {type(e).__name__}: {e} "
           "(it needs jax, flax, optax, clu, ml_collections; none can be installed offline)")
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")}))
    return 0
  try:
    res = run_reference.run(gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                            per_gpu_batch=args.per_gpu_batch, description=args.model,
                            num_classes=NUM_CLASSES, image_size=IMAGE_SIZE)
  except Exception as e:  # pylint: disable=broad-except
    print(json.dumps({"impl": "reference",
                      "unavailable": f"the reference's step failed: {type(e).__name__}: {e}"
                      .replace("\n", " ")}))
    return 0
  out = {
      "metric": "V-MoE B/16 train images/s", "value": res["value"], "unit": "images/s",
      "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
      "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
      "vs_baseline": None, "dtype": "bf16",
      "data": "synthetic images uniform[-1,1] 224x224x3, 21843-way multi-hot labels; random-init weights",
      "impl": "reference",
      "config": {"model": "V-MoE B/16, 8 experts every odd block, K=2, capacity 1.05, BPR, "
                          "sigmoid xent, Adam wd 0.1",
                 "global_batch": res["global_batch"], "seq_len": 197,
                 "parallelism": f"dp{args.gpus} x ep{res['num_partitions']}",
                 "timing": "host clock around block_until_ready (JAX has no CUDA events)"},
      "e2e": res["e2e"], "final_loss": res["final_loss"],
  }
  print(json.dumps(out))
  return 0


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

  FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
            "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu_index: int):
    self.proc = None
    self.gpu_index = gpu_index

  def start(self):
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
           "-lms", "200", "-i", str(self.gpu_index)],
          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    except OSError:
      self.proc = None

  def stop(self):
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      out, _ = self.proc.communicate(timeout=5)
    except subprocess.TimeoutExpired:
      self.proc.kill()
      out, _ = self.proc.communicate()
    sm, smax, reasons = [], [], set()
    for line in out.splitlines():
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 9:
        continue
      try:
        sm.append(float(parts[1]))
        smax.append(float(parts[2]))
      except ValueError:
        continue
      for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                            "sw_power_cap"), parts[5:9]):
        if val.lower().startswith("active"):
          reasons.add(name)
    return {"sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
            "samples": len(sm)}


def make_labels(torch, batch, num_classes, generator):
  labels = torch.zeros(batch, num_classes, dtype=torch.float32)
  npos = torch.randint(1, 4, (batch,), generator=generator)
  for i in range(batch):
    idx = torch.randint(0, num_classes, (int(npos[i]),), generator=generator)
    labels[i, idx] = 1.0
  return labels


def main() -> int:
  args = parse_args()
  if args.impl == "reference":
    return reference_arm(args)

  import torch
  import torch.distributed as dist
  from vmoe_b200 import ops
  from vmoe_b200.configs.vmoe_paper import common
  from vmoe_b200.data import pjit_utils
  from vmoe_b200.ops import _lib
  from vmoe_b200.parallel import mesh as mesh_lib
  from vmoe_b200.train import trainer

  distributed = mesh_lib.init_distributed()
  rank = dist.get_rank() if distributed else 0
  world = dist.get_world_size() if distributed else 1
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  if world != args.gpus:
    raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N>1")
  if args.global_batch is not None:
    if args.global_batch % world:
      raise SystemExit(f"--global-batch {args.global_batch} is not divisible by {world} GPUs")
    args.per_gpu_batch = args.global_batch // world
  device = torch.device("cuda", local_rank)
  torch.cuda.set_device(device)
  if not args.library_ops:
    _lib.lib()  # the CUDA library must be present on a GPU box

  num_partitions = args.num_partitions or min(8, world)
  if world % num_partitions:
    raise SystemExit(f"--num-partitions {num_partitions} does not divide {world} GPUs")
  mesh = mesh_lib.get_auto_logical_mesh(num_partitions)
  mesh_lib.set_mesh(mesh)

  if args.model.startswith("soft-"):
    # Secondary workload: Soft MoE (e.g. "soft-b16": 128 experts x 1 slot in the last 6 blocks).
    from vmoe_b200.projects.soft_moe.configs import common as soft_common
    from vmoe_b200.projects.soft_moe.configs import pretrain_jft4b
    variant, patch = args.model[5].upper(), int(args.model[6:])
    e, last_n = pretrain_jft4b.get_default_moe_num_experts_and_last_n(variant, patch)
    cfg = soft_common.get_vmoe_soft_router_config(
        variant, patch, NUM_CLASSES, image_size=IMAGE_SIZE, num_experts=e, last_n=last_n,
        capacity_factor=None, num_slots=1)
    cfg.encoder.moe.router.compute_similarity_metrics = False
    cfg.encoder.dtype = "bfloat16"
    num_partitions = min(e, world)
    mesh = mesh_lib.get_auto_logical_mesh(num_partitions)
    mesh_lib.set_mesh(mesh)
  else:
    cfg = common.get_vmoe_config(args.model, IMAGE_SIZE, NUM_CLASSES)
    cfg.encoder.dtype = "bfloat16"
    cfg.encoder.moe.router.dispatcher.batch_priority = True
    if args.mode == "eval":
      cfg.encoder.moe.router.dispatcher.capacity_factor = 1.0
    if args.ensemble_size > 1:
      cfg.name = "VisionTransformerMoeEnsemble"
      cfg.encoder.moe.ensemble_size = args.ensemble_size
      cfg.encoder.moe.group_size = cfg.encoder.moe.group_size * args.ensemble_size
  opt_cfg = dict(name="adam", b1=0.9, b2=0.999, weight_decay=0.1,
                 learning_rate=dict(schedule="warmup_linear_decay", peak_value=8e-4,
                                    end_value=1e-5, warmup_steps=10_000))
  total_steps = 100_000
  batch = args.per_gpu_batch

  import contextlib
  ctx = ops.use_cuda_kernels(False) if args.library_ops else contextlib.nullcontext()
  loss_name, loss_kwargs = "sigmoid_xent", {}
  if args.ensemble_size > 1:
    loss_name, loss_kwargs = "ensemble_sigmoid_xent", {"ensemble_size": args.ensemble_size}
  with ctx:
    if args.mode == "eval":
      from vmoe_b200 import models as models_lib
      from vmoe_b200.evaluate import evaluator
      torch.manual_seed(0)
      model = models_lib.create_model(cfg, deterministic=True, mesh=mesh,
                                      image_size=IMAGE_SIZE).to(device)
      model.eval()
      state = None
      _, loss_fn, pred_fn = trainer.get_loss_fn(loss_name, **loss_kwargs)
    else:
      state = trainer.create_train_state(model_config=cfg, optimizer_config=opt_cfg,
                                         total_steps=total_steps, mesh=mesh, device=device,
                                         seed=0, image_size=IMAGE_SIZE)
      loss_fn, _, _ = trainer.get_loss_fn(loss_name, **loss_kwargs)

    gen = torch.Generator().manual_seed(1234 + rank)
    n_host_batches = 2
    host_batches = []
    for _ in range(n_host_batches):
      images = (torch.rand(batch, IMAGE_SIZE, IMAGE_SIZE, 3, generator=gen) * 2 - 1).pin_memory()
      labels = make_labels(torch, batch, NUM_CLASSES, gen).pin_memory()
      host_batches.append({"image": images, "labels": labels})
    dev_batches = [{k: v.to(device) for k, v in b.items()} for b in host_batches]

    def sync_all():
      if distributed:
        dist.barrier()
      torch.cuda.synchronize()

    ones = torch.ones(batch, device=device)

    def run_step(b):
      if args.mode == "eval":
        st = evaluator.evaluate_step(evaluator.EvalState.zeros(device), model, b["image"],
                                     b["labels"], ones, loss_fn, pred_fn)
        return (st.sum_loss / st.num).float()
      _, metrics = trainer.train_step(state, b["image"], b["labels"], loss_fn)
      return metrics["total_loss"]

    # ---------------------------------------------------------------- device-timed arm
    for i in range(args.warmup):
      run_step(dev_batches[i % n_host_batches])
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
      sampler.start()
    _lib.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
      loss = run_step(dev_batches[i % n_host_batches])
    e1.record()
    sync_all()
    launches = _lib.reset_launch_count()
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if distributed:
      dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps
    final_loss = float(loss)

    # ---------------------------------------------------------------- end-to-end arm
    def run_e2e(input_kind):
      """K steps through the public training step behind the package's prefetcher: every step
      consumes one batch copied from pinned host memory and the loss is read back."""
      e2e_batches = host_batches
      transforms = dtypes = None
      if input_kind == "uint8":
        # The decoder's format: uint8 pixels and 0 / 1 labels cross PCIe, the prefetcher maps the
        # pixels to [-1, 1] and casts the labels on the GPU (same values as the float batches up
        # to the 256 pixel levels).
        e2e_batches = [
            {"image": ((b["image"] + 1.0) * 127.5).round().clamp_(0, 255).to(torch.uint8).pin_memory(),
             "labels": b["labels"].to(torch.uint8).pin_memory()} for b in host_batches]
        transforms = {"image": pjit_utils.value_range_on_device(-1.0, 1.0)}
        dtypes = {"labels": torch.float32}

      def host_iter():
        i = 0
        while True:
          yield e2e_batches[i % n_host_batches]
          i += 1

      # One continuous input pipeline, as in a training run: the prefetcher keeps `depth` copies
      # in flight, so a step's inputs were copied while earlier steps ran. The two priming
      # steps below fill that pipeline; inside the timed region every step consumes one batch
      # and issues the copy of one later batch (K copies of Bi bytes for K steps).
      depth = 2
      feed = pjit_utils.prefetch_to_device(host_iter(), size=depth, device=device,
                                           dtypes=dtypes, transforms=transforms)
      for _ in range(depth):
        run_step(next(feed))
      sync_all()
      loss_host = torch.empty(args.steps, dtype=torch.float32, pin_memory=True)
      e0.record()
      for i in range(args.steps):
        loss = run_step(next(feed))
        loss_host[i:i + 1].copy_(loss.detach().float().reshape(1), non_blocking=True)
      e1.record()
      sync_all()
      feed.close()
      ms2 = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
      if distributed:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
      e2e_ms = float(ms2.item()) / args.steps
      h2d = sum(v.numel() * v.element_size() for v in e2e_batches[0].values())
      return {"value": batch * world / (e2e_ms / 1e3), "unit": "images/s",
              "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
              "input": ("uint8 images and uint8 multi-hot labels in pinned memory; value_range(-1, 1) "
                        "and the label cast run on the GPU behind the copy"
                        if input_kind == "uint8" else "float32 images and labels in pinned memory"),
              "pipeline": f"continuous prefetch, {depth} copies in flight; {args.steps} host->device "
                          f"copies issued and {args.steps} batches consumed inside the timed region",
              "last_loss": float(loss_host[-1])}

    e2e = e2e_uint8 = None
    if not args.skip_e2e:
      e2e = run_e2e("float32")
      # The same with the compact host format the input pipeline offers
      # (``dataset.train.device_value_range``): a quarter of the bytes over PCIe.
      e2e_uint8 = run_e2e("uint8")

  if rank == 0:
    value = batch * world / (ms_per_step / 1e3)
    out = {
        "metric": ("V-MoE B/16 train images/s" if args.model == MODEL_DESC and args.mode == "train"
                   and args.ensemble_size == 1 else
                   f"{args.model}{' x' + str(args.ensemble_size) + ' ensemble' if args.ensemble_size > 1 else ''}"
                   f" {args.mode} images/s"),
        "value": value,
        "unit": "images/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic images uniform[-1,1] 224x224x3, 21843-way multi-hot labels; random-init weights",
        "impl": "library-ops stand-in" if args.library_ops else "vmoe_b200",
        "config": {
            "model": ("V-MoE B/16, 8 experts every odd block, K=2, capacity 1.05, BPR, sigmoid xent, Adam wd 0.1"
                      if args.model == MODEL_DESC and args.mode == "train"
                      and args.ensemble_size == 1 else
                      f"{args.model}, mode={args.mode}, ensemble_size={args.ensemble_size}"),
            "global_batch": batch * world,
            "seq_len": (IMAGE_SIZE // int(cfg.patch_size[0])) ** 2 + 1,
            "parallelism": f"dp{world} x ep{num_partitions}",
            "l2": (f"no flush needed: per-step inputs ({batch * (IMAGE_SIZE * IMAGE_SIZE * 3 + NUM_CLASSES) * 4 / 1e6:.0f} MB per GPU) "
                   "and activations (GBs) exceed the 126 MB L2"),
        },
        "clocks": clocks,
        "e2e": e2e,
        "e2e_uint8_input": e2e_uint8,
        "gpu_launches": launches,
        "final_loss": final_loss,
    }
    print(json.dumps(out))
  if distributed:
    dist.barrier()
    dist.destroy_process_group()
  return 0


if __name__ == "__main__":
  sys.exit(main())
