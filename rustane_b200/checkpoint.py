"""RSTK checkpoints (crates/engine/src/checkpoint.rs, bin/train.rs:609-647): seeded writer,
header inspection and the deterministic synthetic-tensor generator shared with the GPU."""
import ctypes as C
import os

import numpy as np

from . import _ffi
from ._ffi import CudaDecodeError, lib

_DTYPES = {"f32": 0, "f16": 1, "bf16": 2}


def synth_value(seed, tensor_uid, idx, std=0.02):
    return lib.cd_synth_value(seed, tensor_uid, idx, std)


def synth_prompt(seed, vocab, n):
    """n token ids uniform in [0, vocab), a pure function of (seed, position)."""
    ids = np.empty(n, dtype=np.uint32)
    lib.cd_synth_prompt(seed, vocab, ids.ctypes.data_as(C.POINTER(C.c_uint32)), n)
    return ids


def write_synthetic_checkpoint(path, cfg, dtype="f32", activation=0, untied_head=False, seed=0, std=0.02, version=3):
    c = cfg.to_c()
    rc = lib.cd_write_synthetic_checkpoint(os.fsencode(path), C.byref(c), _DTYPES[dtype], activation,
                                           int(untied_head), seed, std, version)
    if rc:
        raise CudaDecodeError(rc, lib.cd_last_error(None).decode())


def checkpoint_info(path):
    """Parse and validate an RSTK header without touching the GPU; raises ValueError with the
    reference's messages (checkpoint.rs:30-155)."""
    from .decode import Config
    c = _ffi.CdConfig()
    meta = (C.c_int32 * 4)()
    rc = lib.cd_checkpoint_info(os.fsencode(path), C.byref(c), meta)
    if rc:
        raise ValueError(lib.cd_last_error(None).decode())
    return {"cfg": Config.from_c(c), "version": meta[0], "dtype": meta[1], "activation": meta[2], "untied_head": bool(meta[3] & 1),
            "quantised_linears": bool(meta[3] & 2)}


_QUANT = {"fp8": 3, "int4": 4}


def convert_checkpoint(src, dst, dtype, device=-1):
    """Quantise the linears of an RSTK file once (dtype "fp8": E4M3 with a scale per output row; "int4": symmetric
    groups of 32 with fp16 scales) and write an RSTK v3 file that loads without conversion.  Runs on the GPU."""
    rc = lib.cd_convert_checkpoint(os.fsencode(src), os.fsencode(dst), _QUANT[dtype], device)
    if rc:
        raise CudaDecodeError(rc, lib.cd_last_error(None).decode())
