"""Times the UNMODIFIED reference (google-research/vmoe, JAX / Flax) on the headline benchmark:
V-MoE B/16 training step, synthetic data, bf16 encoder, Adam with weight decay 0.1.

Everything below goes through the reference's own public API and stock code path:
``vmoe.configs.vmoe_paper.common.get_vmoe_config`` for the model,
``vmoe.train.trainer.create_flax_model`` / ``make_create_train_state_fn`` /
``get_loss_fn`` / ``train_step`` for the step (jitted with ``jax.jit`` exactly as
``train_and_evaluate`` does), ``vmoe.partitioning.get_auto_logical_mesh`` for the device mesh.
None of this package's models, kernels or engine is involved. JAX is single-controller: one
process drives all local GPUs, so with several launched ranks only rank 0 runs.

``run`` returns the fields of the benchmark's JSON line (device-timed value and the end-to-end
value whose timed region includes the host->device copy of every step's inputs and the
device->host read of its loss). It needs jax, flax, optax, ml_collections and the reference tree
under ``baseline/_ref``; ``bench.py --impl reference`` reports ``unavailable`` otherwise.
"""
from __future__ import annotations

import time


def run(*, gpus: int, steps: int, warmup: int, per_gpu_batch: int, description: str,
        num_classes: int, image_size: int):
  import jax
  import jax.numpy as jnp
  import numpy as np
  from jax.sharding import NamedSharding, PartitionSpec
  from vmoe import partitioning
  from vmoe.configs.vmoe_paper import common
  from vmoe.train import trainer

  devices = jax.devices()[:gpus]
  if len(devices) < gpus:
    raise RuntimeError(f"{gpus} GPUs requested, JAX sees {len(devices)}")
  batch = per_gpu_batch * gpus
  cfg = common.get_vmoe_config(description + ", 300 Epochs", image_size, num_classes)
  cfg.encoder.dtype = "bfloat16"
  cfg.encoder.moe.router.dispatcher.batch_priority = True
  num_partitions = min(cfg.encoder.moe.num_experts, gpus)
  mesh = partitioning.get_auto_logical_mesh(num_partitions, devices)
  data_sharding = NamedSharding(mesh, PartitionSpec(mesh.axis_names))
  opt_cfg = dict(name="adam", b1=0.9, b2=0.999, mu_dtype="float32", weight_decay=0.1,
                 learning_rate=dict(schedule="warmup_linear_decay", peak_value=8e-4,
                                    end_value=1e-5, warmup_steps=10_000))
  with mesh:
    model = trainer.create_flax_model(config=cfg.to_dict(), deterministic=False)
    image_struct = jax.ShapeDtypeStruct((batch, image_size, image_size, 3), jnp.float32,
                                        sharding=data_sharding)
    init_fn = trainer.make_create_train_state_fn(
        model=model, optimizer_config=opt_cfg, input_shape_dtypes=(image_struct,),
        train_steps=100_000, seed=0, extra_rng_keys=("dropout", "gating"))
    axis_resources = partitioning.tree_axis_resources_from_regexes(
        tree=jax.eval_shape(init_fn), axis_resources_regexes=[("Moe/Mlp/.*", ("expert",))])
    state_sharding = jax.tree_util.tree_map(lambda spec: NamedSharding(mesh, spec), axis_resources)
    state = jax.jit(init_fn, out_shardings=state_sharding)()
    loss_fn, _, _ = trainer.get_loss_fn("sigmoid_xent")
    step_fn = jax.jit(
        lambda s, x, y: trainer.train_step(s, x, y, loss_fn=loss_fn, microsteps=None,
                                           summarizer=None),
        out_shardings=(state_sharding, None), donate_argnums=(0,))

    rng = np.random.default_rng(1234)
    host = []
    for _ in range(2):
      images = rng.uniform(-1, 1, (batch, image_size, image_size, 3)).astype(np.float32)
      labels = np.zeros((batch, num_classes), np.float32)
      for i in range(batch):
        labels[i, rng.integers(0, num_classes, rng.integers(1, 4))] = 1.0
      host.append((images, labels))
    put = lambda b: tuple(jax.device_put(a, data_sharding) for a in b)
    dev = [put(b) for b in host]

    for i in range(warmup):
      state, metrics = step_fn(state, *dev[i % 2])
    jax.block_until_ready(metrics["total_loss"])
    t0 = time.perf_counter()
    for i in range(steps):
      state, metrics = step_fn(state, *dev[i % 2])
    jax.block_until_ready(metrics["total_loss"])
    ms = (time.perf_counter() - t0) * 1e3 / steps
    loss = float(metrics["total_loss"])

    # end to end: every step copies its inputs from host memory and reads its loss back
    for i in range(2):
      state, metrics = step_fn(state, *put(host[i % 2]))
      float(metrics["total_loss"])
    t0 = time.perf_counter()
    for i in range(steps):
      state, metrics = step_fn(state, *put(host[i % 2]))
      last = float(metrics["total_loss"])
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
  h2d = sum(a.nbytes for a in host[0]) // gpus
  return {"ms_per_step": ms, "value": batch / (ms / 1e3), "final_loss": loss,
          "global_batch": batch, "num_partitions": num_partitions,
          "e2e": {"value": batch / (e2e_ms / 1e3), "unit": "images/s", "ms_per_step": e2e_ms,
                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": last}}
