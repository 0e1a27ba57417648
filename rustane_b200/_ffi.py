"""ctypes binding of libcuda_decode.so (include/cuda_decode.h).

The library is the product: there is no Python or CPU fallback.  Importing this module
raises ImportError when the shared library has not been built.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcuda_decode.so")

OK = 0
ERR_INVALID, ERR_SEQ_FULL, ERR_TOKEN, ERR_CAPACITY, ERR_CUDA, ERR_IO, ERR_DEVICE_WAIT, ERR_UNSUPPORTED = range(-1, -9, -1)
DTYPE_F32, DTYPE_F16, DTYPE_BF16, DTYPE_FP8_E4M3, DTYPE_INT4_G32 = 0, 1, 2, 3, 4
KV_AUTO, KV_F32, KV_F16, KV_BF16 = 0, 1, 2, 3
ACT_SWIGLU, ACT_LEAKY_RELU_SQ = 0, 1
BACKEND_AUTO, BACKEND_NAIVE, BACKEND_CUDA = 0, 1, 2
MODE_PREFILL_ONLY, MODE_NAIVE_FULL_CONTEXT, MODE_KV_CACHE_CUDA = 0, 1, 2
MAX_GPU_TOPK = 32
HEAD_BLOCK = 256


class CdConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "dim", "hidden", "heads", "kv_heads", "hd", "seq", "nlayers", "vocab", "q_dim", "kv_dim", "gqa_ratio")]


class CdLayerInit(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in (
        "wq", "wk", "wv", "wo", "w1", "w3", "w2", "gamma1", "gamma2")]


class CdHeadInit(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in ("gamma_final", "embed", "lm_head")]


class CdMoeConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_experts", "top_k", "n_shared", "kv_latent", "rope_dim", "nope_dim", "v_dim")]


class CdOptions(C.Structure):
    _fields_ = [("weight_dtype", C.c_int32), ("activation", C.c_int32), ("device", C.c_int32),
                ("page_tokens", C.c_int32), ("max_samples", C.c_int32), ("use_graph", C.c_int32),
                ("kv_dtype", C.c_int32), ("tp_rank", C.c_int32), ("tp_world", C.c_int32), ("wait_us", C.c_int32),
                ("test_flags", C.c_int32), ("test_ring_kb", C.c_int32)]


class CdRequest(C.Structure):
    _fields_ = [("decode_backend", C.c_int32), ("steps", C.c_int32), ("temperature", C.c_float),
                ("top_k", C.c_int32), ("samples", C.c_int32), ("seed", C.c_uint64)]


class CdSelection(C.Structure):
    _fields_ = [("mode", C.c_int32), ("fallback_reason", C.c_char_p), ("auto_reason", C.c_char_p)]


class CdSampleResult(C.Structure):
    _fields_ = [("seed", C.c_uint64), ("generated_len", C.c_size_t), ("sampled_len", C.c_size_t),
                ("decode_ms", C.c_double)]


class CdBatchInfo(C.Structure):
    _fields_ = [("selection", CdSelection), ("base_prefill_ms", C.c_double), ("request_prefill_ms", C.c_double),
                ("prefill_ms", C.c_double), ("total_decode_ms", C.c_double), ("avg_decode_ms", C.c_double),
                ("total_ms", C.c_double), ("nresults", C.c_int32)]


STREAM_CB = C.CFUNCTYPE(C.c_int, C.c_uint32, C.POINTER(C.c_uint32), C.c_size_t, C.POINTER(C.c_uint32), C.c_size_t,
                        C.c_void_p)

_P = C.POINTER
_f32p, _u32p, _u64p, _szp = _P(C.c_float), _P(C.c_uint32), _P(C.c_uint64), _P(C.c_size_t)
_vp, _vpp = C.c_void_p, _P(C.c_void_p)

# name -> (restype, argtypes); this table is also what the symbol-export test walks.
SIGNATURES = {
    "cd_model_create": (C.c_int, [_P(CdConfig), _P(CdLayerInit), C.c_int, _P(CdHeadInit), _P(CdOptions), _vpp]),
    "cd_model_destroy": (None, [_vp]),
    "cd_last_error": (C.c_char_p, [_vp]),
    "cd_len": (C.c_int, [_vp, _szp]),
    "cd_set_len": (C.c_int, [_vp, C.c_size_t]),
    "cd_seed_layer_cache_cf": (C.c_int, [_vp, C.c_int, C.c_size_t, _f32p, _f32p]),
    "cd_decode_token": (C.c_int, [_vp, _f32p, _f32p]),
    "cd_decode_token_from_id": (C.c_int, [_vp, C.c_uint32, _f32p]),
    "cd_decode_token_argmax": (C.c_int, [_vp, _f32p, _u32p]),
    "cd_decode_token_argmax_from_id": (C.c_int, [_vp, C.c_uint32, _u32p]),
    "cd_decode_token_topk_from_id": (C.c_int, [_vp, C.c_uint32, C.c_size_t, _f32p, _u32p, C.c_size_t, _szp]),
    "cd_decode_token_block_stats_from_id": (C.c_int, [_vp, C.c_uint32, C.c_float, C.c_float, _f32p, _f32p,
                                                       C.c_size_t, _szp]),
    "cd_materialize_current_logits_block": (C.c_int, [_vp, C.c_size_t, C.c_float, _f32p, C.c_size_t, _szp]),
    "cd_model_create_from_checkpoint": (C.c_int, [C.c_char_p, _P(CdOptions), _P(CdConfig), _vpp]),
    "cd_checkpoint_info": (C.c_int, [C.c_char_p, _P(CdConfig), _P(C.c_int32)]),
    "cd_model_create_synthetic": (C.c_int, [_P(CdConfig), _P(CdOptions), C.c_uint64, C.c_float, C.c_int, _vpp]),
    "cd_synth_value": (C.c_float, [C.c_uint64, C.c_uint64, C.c_uint64, C.c_float]),
    "cd_synth_prompt": (None, [C.c_uint64, C.c_int, _u32p, C.c_int]),
    "cd_write_synthetic_checkpoint": (C.c_int, [C.c_char_p, _P(CdConfig), C.c_int, C.c_int, C.c_int, C.c_uint64,
                                                 C.c_float, C.c_int]),
    "cd_model_get_config": (C.c_int, [_vp, _P(CdConfig), _P(CdOptions), _P(C.c_int)]),
    "cd_convert_checkpoint": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int, C.c_int]),
    "cd_model_save_quantised": (C.c_int, [_vp, C.c_char_p]),
    "cd_model_get_linear_rows": (C.c_int, [_vp, C.c_int, C.c_int, _vp, C.c_size_t]),
    "cd_moe_model_create_synthetic": (C.c_int, [_P(CdConfig), _P(CdMoeConfig), _P(CdOptions), C.c_uint64, C.c_float, C.c_int, _vpp]),
    "cd_moe_shard_plan": (C.c_int, [_P(CdConfig), _P(CdMoeConfig), C.c_int, C.c_int, _P(C.c_int32), _P(C.c_int32), _P(C.c_int32), _P(C.c_int32)]),
    "cd_moe_last_experts": (C.c_int, [_vp, C.c_int, _P(C.c_int32), C.c_size_t]),
    "cd_tp_shard_plan": (C.c_int, [_P(CdConfig), C.c_int, C.c_int, _P(CdConfig), _P(C.c_int32), _P(C.c_int32)]),
    "cd_tp_region_handle": (C.c_int, [_vp, _vp, C.c_size_t]),
    "cd_tp_connect": (C.c_int, [_vp, _vp, C.c_int]),
    "cd_tp_region_ptr": (C.c_int, [_vp, _vpp]),
    "cd_tp_connect_ptrs": (C.c_int, [_vp, _vpp, C.c_int]),
    "cd_decode_token_logits_from_id": (C.c_int, [_vp, C.c_uint32, C.c_float, _f32p]),
    "cd_prefill": (C.c_int, [_vp, _u32p, C.c_size_t, C.c_float, _f32p]),
    "cd_decode_steps_greedy": (C.c_int, [_vp, C.c_uint32, C.c_size_t, _u32p]),
    "cd_decode_steps_topk": (C.c_int, [_vp, C.c_uint32, C.c_size_t, C.c_size_t, C.c_float, C.c_float, _u64p, _u32p]),
    "cd_decode_steps_fullvocab": (C.c_int, [_vp, C.c_uint32, C.c_size_t, C.c_float, C.c_float, _u64p, _u32p]),
    "cd_decode_steps_samples": (C.c_int, [_vp, _u32p, C.c_size_t, C.c_size_t, C.c_int, C.c_size_t, C.c_float, C.c_float, _u64p, _u32p]),
    "cd_profile_decode_step": (C.c_int, [_vp, C.c_uint32, _f32p, _u32p, C.c_size_t]),
    "cd_debug_phase_trace": (C.c_int, [_vp, _u64p, C.c_size_t, _szp]),
    "cd_last_device_ms": (C.c_int, [_vp, _f32p]),
    "cd_kernel_launches": (C.c_int, [_vp, _u64p]),
    "cd_flash_decode": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_int, _f32p, _vp, _vp, _f32p]),
    "cd_flash_decode_static": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_int, C.c_int, _f32p, _vp,
                                         _P(C.c_int32), _f32p, _vp]),
    "cd_param_count": (C.c_size_t, [_P(CdConfig)]),
    "cd_select_decode_mode": (C.c_int, [_P(CdConfig), C.c_int, C.c_size_t, C.c_size_t, _P(CdSelection)]),
    "cd_backend_name": (C.c_char_p, [C.c_int]),
    "cd_backend_parse": (C.c_int, [C.c_char_p]),
    "cd_mode_name": (C.c_char_p, [C.c_int]),
    "cd_lcg_next_u64": (C.c_uint64, [_u64p]),
    "cd_lcg_next_f32": (C.c_float, [_u64p]),
    "cd_sample_next": (C.c_uint32, [_f32p, C.c_size_t, C.c_float, C.c_size_t, _u64p]),
    "cd_sample_topk_candidates": (C.c_uint32, [_u32p, _f32p, C.c_size_t, C.c_float, _u64p]),
    "cd_sample_block_from_stats": (C.c_size_t, [_f32p, _f32p, C.c_size_t, _u64p]),
    "cd_sample_softmax_index": (C.c_size_t, [_f32p, C.c_size_t, C.c_float, _u64p]),
    "cd_merge_topk_candidates": (C.c_size_t, [_f32p, _u32p, C.c_size_t, C.c_size_t, _f32p, _u32p]),
    "cd_session_create": (C.c_int, [_vp, _u32p, C.c_size_t, C.c_float, _vpp]),
    "cd_session_destroy": (None, [_vp]),
    "cd_session_last_error": (C.c_char_p, [_vp]),
    "cd_session_prompt_len": (C.c_size_t, [_vp]),
    "cd_session_prefill_ms": (C.c_double, [_vp]),
    "cd_session_prompt_logits": (C.c_int, [_vp, _f32p, C.c_size_t]),
    "cd_session_generate": (C.c_int, [_vp, _P(CdRequest), _u32p, C.c_size_t, _P(CdBatchInfo)]),
    "cd_session_generate_stream": (C.c_int, [_vp, _P(CdRequest), _u32p, C.c_size_t, STREAM_CB, _vp, _P(CdBatchInfo)]),
    "cd_session_result": (C.c_int, [_vp, C.c_int, _P(CdSampleResult)]),
    "cd_session_result_tokens": (C.c_int, [_vp, C.c_int, _u32p, C.c_size_t, _u32p, C.c_size_t]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "rustane_b200: %s is missing — build it with `make -C rustane_b200/csrc` "
            "(or __graft_entry__.build()); there is no fallback path" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the .so is stale
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


class CudaDecodeError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("cuda_decode error %d: %s" % (code, message))
        self.code = code
        self.message = message
