"""Drop-in module name of the reference's extension (`import decdec_ext`, used by
end-to-end/plugin.py, end-to-end/APLinear.py and evaluation/evaltools.py of SNU-ARC/DecDEC).

Re-exports the compiled torch shim that sits on top of the C ABI of libdecdec_b200.so.  There is no
fallback: if the shim or the CUDA library has not been built, the import fails.
"""
import torch  # noqa: F401  (loads the torch shared libraries the shim links against)

try:
    from decdec_b200.decdec_ext import *  # noqa: F401,F403
    from decdec_b200 import decdec_ext as _native
except ImportError as e:  # pragma: no cover
    raise ImportError(
        "decdec_ext: the native module is not built; run `python -m decdec_b200.build` "
        "(needs nvcc and the torch headers).  No CPU fallback exists for this path.") from e

__all__ = [n for n in dir(_native) if not n.startswith("_")]
