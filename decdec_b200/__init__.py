"""decdec_b200 - B200 (sm_100a) implementation of the DecDEC decode hot path.

`decdec_b200.capi`  : ctypes view of the C ABI (include/decdec_b200.h)
`decdec_b200.ops`   : the reference's `decdec_ext` function set over torch tensors, through the C ABI
`decdec_ext`        : (repo root) drop-in module name used by the reference's Python code
"""
__all__ = ["capi", "ops"]
