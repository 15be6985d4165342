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
