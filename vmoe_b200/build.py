"""Builds ``libvmoe_b200.so`` (all CUDA kernels of the package) for sm_100a with nvcc.

The library has a plain C ABI (``csrc/vmoe_api.h``) and no PyTorch dependency, so it compiles
in seconds and is loaded with ctypes (``vmoe_b200/ops/_lib.py``). The shared object is written
next to the sources, inside the package, and is rebuilt only when a source is newer.

Usage: ``python -m vmoe_b200.build [--force] [--verbose]``

``--define NAME[=VALUE]`` (repeatable) with ``--output PATH`` builds a diagnostic variant into its
own file (e.g. ``--define ATT_TRACE=1`` for the attention kernels' timing probes); the
environment variable ``VMOE_B200_LIB`` makes ``ops/_lib.py`` load it instead of the product.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "csrc", "build")
LIB_PATH = os.path.join(PKG_DIR, "libvmoe_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
  exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  if not os.path.exists(exe):
    raise RuntimeError("nvcc not found; libvmoe_b200.so cannot be built")
  return exe


def sources() -> list[str]:
  return sorted(
      os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
  return sorted(
      os.path.join(CSRC, f) for f in os.listdir(CSRC)
      if f.endswith((".cuh", ".h")))


def needs_build() -> bool:
  if not os.path.exists(LIB_PATH):
    return True
  t = os.path.getmtime(LIB_PATH)
  return any(os.path.getmtime(s) > t for s in sources() + _headers())


def build(force: bool = False, verbose: bool = False, defines=(), output: str | None = None) -> str:
  """Compiles every ``csrc/*.cu`` and links the shared library. Returns its path."""
  if defines or output:
    return _build_variant(list(defines), output, verbose)
  if not force and not needs_build():
    return LIB_PATH
  os.makedirs(OBJ_DIR, exist_ok=True)
  nvcc = _nvcc()
  hdr_time = max([os.path.getmtime(h) for h in _headers()] or [0.0])

  def compile_one(src: str) -> str:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    if (not force and os.path.exists(obj) and
        os.path.getmtime(obj) > max(os.path.getmtime(src), hdr_time)):
      return obj
    cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    if verbose:
      cmd.insert(1, "-Xptxas=-v")
      print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
      raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
      print(res.stderr, flush=True)
    return obj

  with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
    objs = list(pool.map(compile_one, sources()))
  tmp = LIB_PATH + ".tmp"
  cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode",
         "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
  os.replace(tmp, LIB_PATH)
  return LIB_PATH


def _build_variant(defines: list[str], output: str | None, verbose: bool) -> str:
  """A full build with extra ``-D`` flags into ``output`` (objects in a directory beside it)."""
  if not output:
    raise ValueError("--define needs --output: a variant never replaces the product library")
  output = os.path.abspath(output)
  obj_dir = output + ".objs"
  os.makedirs(obj_dir, exist_ok=True)
  nvcc = _nvcc()
  flags = [f"-D{d}" for d in defines]

  def compile_one(src: str) -> str:
    obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
    cmd = [nvcc, *NVCC_FLAGS, *flags, "-I", CSRC, "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
      raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
      print(" ".join(cmd), flush=True)
    return obj

  with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
    objs = list(pool.map(compile_one, sources()))
  cmd = [nvcc, "-shared", "-o", output, *objs, "-gencode",
         "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
  shutil.rmtree(obj_dir, ignore_errors=True)
  return output


def main(argv=None) -> int:
  ap = argparse.ArgumentParser()
  ap.add_argument("--force", action="store_true")
  ap.add_argument("--verbose", action="store_true")
  ap.add_argument("--define", action="append", default=[], metavar="NAME[=VALUE]")
  ap.add_argument("--output", default=None, help="path of a diagnostic variant (with --define)")
  args = ap.parse_args(argv)
  print(build(force=args.force, verbose=args.verbose, defines=args.define, output=args.output))
  return 0


if __name__ == "__main__":
  sys.exit(main())
