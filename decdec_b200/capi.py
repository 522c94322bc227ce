"""ctypes binding of the C ABI declared in include/decdec_b200.h.

This is the thinnest possible host layer: raw pointers in, status codes out.  It is what the parity
tests call, and what a non-torch host would bind.  There is no CPU fallback: if the CUDA library is
missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

FP32, FP16, BF16 = 0, 1, 2

# DECDEC_B200_LIB selects another build of the same library (e.g. one with debug instrumentation)
_LIB_PATH = Path(os.environ.get("DECDEC_B200_LIB") or (Path(__file__).resolve().parent / "libdecdec_b200.so"))


class DecdecError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


class ConfigInfo(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_chunks", "chunk_size", "k_chunk", "channels_per_tb", "n_tb", "block_dim_x", "block_dim_y",
        "shared_memory_size", "reduced_shared_memory")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


def _load():
    if not _LIB_PATH.exists():
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python -m decdec_b200.build` "
            "(there is no CPU fallback for the decode hot path)")
    return C.CDLL(str(_LIB_PATH))


lib = _load()

_vp, _u32, _i, _up, _ll = C.c_void_p, C.c_uint32, C.c_int, C.c_size_t, C.c_longlong

SIGNATURES = {
    "decdec_last_error": (C.c_char_p, []),
    "decdec_compiled_arch": (_i, []),
    "decdec_stream_status": (_i, [_vp, C.POINTER(_u32)]),
    "decdec_stream_reset": (_i, [_vp]),
    "decdec_create_context": (_i, [_u32, _vp, _vp, _u32, _i, C.POINTER(_up)]),
    "decdec_destroy_context": (_i, [_up]),
    "decdec_create_config": (_i, [_up, _u32, _vp, _i, _u32, _u32, _vp, _i, _vp, _i, C.POINTER(_up)]),
    "decdec_update_config": (_i, [_up, _up, _u32]),
    "decdec_destroy_config": (_i, [_up]),
    "decdec_read_config": (_i, [_up, C.POINTER(ConfigInfo)]),
    "decdec_dec": (_i, [_up, _vp, _vp, _u32, _u32, _i, _vp]),
    "decdec_unfused_dec": (_i, [_up, _vp, _vp, _u32, _u32, _i, _vp]),
    "decdec_anyprec_gemv": (_i, [_vp, _vp, _vp, _u32, _vp, _u32, _u32, _i, _i, _vp]),
    "decdec_lutgemm_gemv": (_i, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _i, _vp]),
    "decdec_sqllm_gemv": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _vp]),
    "decdec_lutgemm_gemv_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _i, _vp]),
    "decdec_lutgemm_dequant": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _i, _vp]),
    "decdec_tp_layout": (_i, [_u32, _u32, C.POINTER(_up), C.POINTER(_up), C.POINTER(_up), C.POINTER(_up)]),
    "decdec_tp_create": (_i, [_u32, _u32, _u32, C.POINTER(_up), _vp]),
    "decdec_tp_local_ptr": (_i, [_up, C.POINTER(_vp)]),
    "decdec_tp_connect_ipc": (_i, [_up, _vp]),
    "decdec_tp_connect_ptrs": (_i, [_up, C.POINTER(_up)]),
    "decdec_tp_allreduce": (_i, [_up, _vp, _u32, _i, _vp]),
    "decdec_tp_status": (_i, [_up, C.POINTER(_u32), C.POINTER(_u32)]),
    "decdec_tp_destroy": (_i, [_up]),
    "decdec_anyprec_dequant": (_i, [_vp, _vp, _vp, _u32, _u32, _i, _i, _vp]),
    "decdec_dec_anyprec": (_i, [_up, _vp, _vp, _vp, _u32, _vp, _u32, _u32, _i, _i, _vp]),
    "decdec_dec_lutgemm": (_i, [_up, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _i, _vp]),
    "decdec_dec_sqllm": (_i, [_up, _vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _vp]),
    "decdec_dummy_anyprec": (_i, [_vp, _vp, _vp, _u32, _vp, _u32, _u32, _i, _i, _i, _ll, _vp]),
    "decdec_dummy_lutgemm": (_i, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _i, _i, _ll, _vp]),
    "decdec_dummy_sqllm": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _i, _i, _i, _ll, _vp]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)   # AttributeError here = header and library out of sync
    _fn.restype = _res
    _fn.argtypes = _args


def check(code: int) -> None:
    if code != 0:
        raise DecdecError(code, lib.decdec_last_error().decode("utf-8", "replace"))


def call(name: str, *args) -> None:
    check(getattr(lib, name)(*args))
