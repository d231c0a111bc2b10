"""Every module of the package imports on a machine without a GPU."""
import importlib
import pkgutil

import vmoe_b200


def test_all_modules_import():
  failed = []
  for mod in pkgutil.walk_packages(vmoe_b200.__path__, prefix="vmoe_b200."):
    if mod.name.endswith((".main", ".main_contrastive", ".libvmoe_b200")):
      continue  # scripts, and the CUDA shared library (loaded with ctypes, not a Python module)
    try:
      importlib.import_module(mod.name)
    except Exception as e:  # pylint: disable=broad-except
      failed.append((mod.name, repr(e)))
  assert not failed, failed
