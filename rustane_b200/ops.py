"""Single operators of the token loop on caller-supplied data."""
import ctypes as C

import numpy as np

from ._ffi import CudaDecodeError, lib

_DT = {"f32": 0, "f16": 1, "bf16": 2}


def to_storage(a, dtype):
    """fp32 array -> the raw storage words of `dtype` (round to nearest even): float32 for
    f32, float16 for f16, uint16 bit patterns for bf16."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == "f32":
        return a
    if dtype == "f16":
        return a.astype(np.float16)
    u = a.view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_storage(s, dtype):
    if dtype == "bf16":
        return (s.astype(np.uint32) << 16).view(np.float32)
    return s.astype(np.float32)


def flash_decode(q, k, v, heads, kv_heads, hd, dtype="bf16", nsplit=0):
    """One query token against attn_len cached positions: q [heads*hd] fp32, k and v
    [attn_len, kv_heads*hd] already in storage form (see to_storage).  Returns [heads*hd] fp32."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
    attn_len = k.shape[0]
    out = np.empty(heads * hd, dtype=np.float32)
    f32p = C.POINTER(C.c_float)
    rc = lib.cd_flash_decode(_DT[dtype], heads, kv_heads, hd, attn_len, nsplit, q.ctypes.data_as(f32p),
                             k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), out.ctypes.data_as(f32p))
    if rc:
        raise CudaDecodeError(rc, lib.cd_last_error(None).decode())
    return out
