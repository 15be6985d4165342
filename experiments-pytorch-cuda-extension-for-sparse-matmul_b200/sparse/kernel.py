"""Loader of the native binding ``sparse_ops``.

The reference JIT-compiles its sources at import time
(sparse/kernel.py:11-16).  Here the binding is built ahead of time, in tree,
by ``build.py`` next to this package; importing this module only loads it.
There is no Python or CPU fallback: if the binding is missing the import
fails with the build command to run.
"""
import importlib
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))


def _load():
    import torch  # noqa: F401  (libtorch must be loaded before the binding)
    try:
        return importlib.import_module(".sparse_ops", __package__)
    except ImportError as exc:
        raise ImportError(
            "the native binding sparse_ops is not built (or failed to load: %s). "
            "Build it with: python %s" % (exc, os.path.join(os.path.dirname(_PKG_DIR), "build.py"))
        ) from exc


sparse_ops = _load()

# The ops are asynchronous and never read the device status word themselves: a kernel that gives up on a
# bounded wait, or meets a block descriptor that does not belong to its layout, is reported by
# ``sparse_ops.check_device_status(device_index)`` (see there).  With ``debug_checks`` set -- or the environment
# variable BSA_DEBUG_CHECKS=1 at import time -- every autograd op of this package calls it after its forward and
# after its backward pass, which synchronises the device each time: for debugging, not for production.
debug_checks = os.environ.get("BSA_DEBUG_CHECKS", "0") not in ("", "0")


def check(tensor):
    """Opt-in status check after an op (a no-op unless ``debug_checks`` is set); returns ``tensor``."""
    if debug_checks and tensor is not None and tensor.is_cuda:
        sparse_ops.check_device_status(tensor.device.index or 0)
    return tensor
