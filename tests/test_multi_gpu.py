"""Multi-GPU tests (run as child processes under torchrun on 2 GPUs of one node)."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  p = s.getsockname()[1]
  s.close()
  return p


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_p2p_moe_matches_nccl_path(tmp_path):
  env = dict(os.environ, NCCL_NVLS_ENABLE="0")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
         os.path.join(HERE, "p2p_worker.py"), str(tmp_path)]
  res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
  for r in range(2):
    out = json.load(open(tmp_path / f"p2p_r{r}.json"))
    assert all(s == 0 for s in out["status"]), out
    for name, errs in out["errs"].items():
      # identical math up to atomics order in the weight-gradient accumulation
      assert max(errs) < 2e-2, (name, errs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_overlapped_grad_allreduce_matches_nccl(tmp_path):
  env = dict(os.environ, NCCL_NVLS_ENABLE="0")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
         os.path.join(HERE, "allreduce_worker.py"), str(tmp_path)]
  res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
  for r in range(2):
    out = json.load(open(tmp_path / f"ar_r{r}.json"))
    assert out["status"] == 0, out
    assert out["ranges"] >= 4, out  # per-block ranges were planned
    assert out["err"] < 2e-2, out
    for a, b in zip(out["norms"], out["ref_norms"]):
      assert abs(a - b) / (abs(b) + 1e-6) < 2e-2, out
