"""B200-native token loop behind the reference's C API.

The product is ``libncm_b200.so`` (CUDA, built from ``csrc/`` by ``build.py``) and
its header ``include/ncm_b200.h``.  The Python modules here are thin: ``capi`` binds
the C ABI with ctypes, ``synth`` writes seeded model files in the reference's
formats, ``build`` compiles the library.  The directory name carries a hyphen, so
load the package by path (see ``__graft_entry__.load_package``) or put the
directory itself on ``sys.path`` and import ``capi`` / ``synth`` directly.
"""
import os as _os
import sys as _sys

_HERE = _os.path.dirname(_os.path.abspath(__file__))
if _HERE not in _sys.path:
    _sys.path.insert(0, _HERE)

import build  # noqa: E402,F401
import capi  # noqa: E402,F401
import synth  # noqa: E402,F401

LIB_PATH = _os.path.join(_HERE, "libncm_b200.so")


def load_library():
    """The CUDA library; raises when it is not built (there is no CPU fallback)."""
    if not _os.path.exists(LIB_PATH):
        raise RuntimeError("libncm_b200.so is missing: run `python saphira-cncm_b200/build.py`")
    return capi.NcmLib(LIB_PATH)
