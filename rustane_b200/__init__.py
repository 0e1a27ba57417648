"""rustane_b200 — a B200-native (sm_100a) backend for rustane's autoregressive token loop.

The package is a thin binding over `libcuda_decode.so` (hand-written CUDA kernels behind the
C ABI in include/cuda_decode.h).  There is no CPU fallback: importing fails if the library
has not been built, and every compute call fails without a CUDA device.
"""
from . import _ffi  # noqa: F401  (raises ImportError when the library is missing)
from ._ffi import CudaDecodeError
from .checkpoint import checkpoint_info, convert_checkpoint, synth_prompt, synth_value, write_synthetic_checkpoint
from .decode import MAX_GPU_TOPK, Config, DecodeContext, Model, MoeConfig, merge_topk_candidates
from .inference import (GenerationBatch, GenerationRequest, InferenceSession, SampleResult, auto_prefers_cuda,
                        parse_decode_backend, select_decode_mode)

__all__ = [
    "CudaDecodeError", "Config", "Model", "MoeConfig", "DecodeContext", "MAX_GPU_TOPK", "merge_topk_candidates",
    "GenerationRequest", "GenerationBatch", "SampleResult", "InferenceSession", "select_decode_mode",
    "auto_prefers_cuda", "parse_decode_backend", "write_synthetic_checkpoint", "synth_prompt", "synth_value",
    "checkpoint_info", "convert_checkpoint",
]
