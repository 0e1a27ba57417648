"""Python mirror of `engine::inference` (crates/engine/src/inference.rs): GenerationRequest,
select_decode_mode, the samplers and InferenceSession, all executed by the C++ host layer
of libcuda_decode.so.
"""
import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import _ffi
from ._ffi import CudaDecodeError, lib

AUTO_PARAM_THRESHOLD = 20_000_000  # AUTO_METAL_PARAM_THRESHOLD, inference.rs:9
_BACKENDS = {"auto": _ffi.BACKEND_AUTO, "naive": _ffi.BACKEND_NAIVE, "cuda": _ffi.BACKEND_CUDA}
_MODES = {_ffi.MODE_PREFILL_ONLY: "prefill_only", _ffi.MODE_NAIVE_FULL_CONTEXT: "naive_full_context",
          _ffi.MODE_KV_CACHE_CUDA: "kv_cache_cuda"}


def _u32(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint32))


def _f32(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def parse_decode_backend(raw):
    """DecodeBackendRequest::parse (inference.rs:19-26); None when unknown."""
    return raw if raw in _BACKENDS else None


@dataclass
class GenerationRequest:
    """inference.rs:61-82 (same defaults)."""
    decode_backend: str = "auto"
    steps: int = 32
    temperature: float = 0.0
    top_k: int = 0
    samples: int = 1
    seed: int = 1

    def to_c(self):
        return _ffi.CdRequest(_BACKENDS[self.decode_backend], self.steps, self.temperature, self.top_k,
                              self.samples, self.seed & 0xFFFFFFFFFFFFFFFF)


@dataclass
class DecodeSelection:
    mode: str
    fallback_reason: Optional[str]
    auto_reason: Optional[str]


@dataclass
class SampleResult:
    seed: int
    generated: List[int]
    sampled: List[int]
    decode_elapsed_ms: float


@dataclass
class GenerationBatch:
    decode_selection: DecodeSelection
    base_prefill_ms: float
    request_prefill_ms: float
    prefill_ms: float
    total_decode_ms: float
    avg_decode_ms: float
    total_ms: float
    results: List[SampleResult] = field(default_factory=list)


def _selection(sel):
    return DecodeSelection(_MODES[sel.mode], sel.fallback_reason.decode() if sel.fallback_reason else None,
                           sel.auto_reason.decode() if sel.auto_reason else None)


def select_decode_mode(cfg, requested, effective_context_len, steps):
    """inference.rs:458-528."""
    c, sel = cfg.to_c(), _ffi.CdSelection()
    lib.cd_select_decode_mode(C.byref(c), _BACKENDS[requested], effective_context_len, steps, C.byref(sel))
    return _selection(sel)


def auto_prefers_cuda(cfg):
    return cfg.param_count() >= AUTO_PARAM_THRESHOLD


# ---- samplers (inference.rs:759-921); rng is a one-element uint64 numpy array updated in place
def _rng(state):
    return state.ctypes.data_as(C.POINTER(C.c_uint64))


def next_f32(state):
    return lib.cd_lcg_next_f32(_rng(state))


def sample_next(logits, temperature, top_k, state):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    return lib.cd_sample_next(_f32(lg), len(lg), temperature, top_k, _rng(state))


def sample_topk_candidates(idxs, logits, temperature, state):
    ix = np.ascontiguousarray(idxs, dtype=np.uint32)
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    return lib.cd_sample_topk_candidates(_u32(ix), _f32(lg), len(lg), temperature, _rng(state))


def sample_block_from_stats(maxes, sums, state):
    mx = np.ascontiguousarray(maxes, dtype=np.float32)
    sm = np.ascontiguousarray(sums, dtype=np.float32)
    return lib.cd_sample_block_from_stats(_f32(mx), _f32(sm), len(mx), _rng(state))


def sample_block_logits(base, logits, temperature, state):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    return base + lib.cd_sample_softmax_index(_f32(lg), len(lg), temperature, _rng(state))


class InferenceSession:
    """inference.rs:105-451.  Construction runs the prefill on the GPU; `generate` and
    `generate_with_suffix` reuse it for every sample and every later request."""

    def __init__(self, model, prompt_ids, softcap=0.0):
        self.model = model
        ids = np.ascontiguousarray(prompt_ids, dtype=np.uint32)
        h = C.c_void_p()
        rc = lib.cd_session_create(model._h, _u32(ids), len(ids), softcap, C.byref(h))
        if rc:
            raise ValueError(lib.cd_session_last_error(None).decode())
        self._h = h
        self._prompt_ids = [int(t) for t in ids]
        self._softcap = softcap

    def close(self):
        if getattr(self, "_h", None):
            lib.cd_session_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def prompt_ids(self):
        return list(self._prompt_ids)

    def prompt_len(self):
        return lib.cd_session_prompt_len(self._h)

    def prefill_elapsed_ms(self):
        return lib.cd_session_prefill_ms(self._h)

    def softcap(self):
        return self._softcap

    def prompt_logits(self):
        out = np.empty(self.model.cfg.vocab, dtype=np.float32)
        lib.cd_session_prompt_logits(self._h, _f32(out), len(out))
        return out

    def _collect(self, info):
        results = []
        for i in range(info.nresults):
            r = _ffi.CdSampleResult()
            lib.cd_session_result(self._h, i, C.byref(r))
            gen = np.empty(r.generated_len, dtype=np.uint32)
            smp = np.empty(r.sampled_len, dtype=np.uint32)
            lib.cd_session_result_tokens(self._h, i, _u32(gen), len(gen), _u32(smp), len(smp))
            results.append(SampleResult(r.seed, [int(t) for t in gen], [int(t) for t in smp], r.decode_ms))
        return GenerationBatch(_selection(info.selection), info.base_prefill_ms, info.request_prefill_ms,
                               info.prefill_ms, info.total_decode_ms, info.avg_decode_ms, info.total_ms, results)

    def generate(self, req):
        return self.generate_with_suffix(req, [])

    def generate_with_suffix(self, req, prompt_suffix):
        sfx = np.ascontiguousarray(prompt_suffix, dtype=np.uint32)
        c, info = req.to_c(), _ffi.CdBatchInfo()
        rc = lib.cd_session_generate(self._h, C.byref(c), _u32(sfx), len(sfx), C.byref(info))
        if rc:
            raise ValueError(lib.cd_session_last_error(self._h).decode())
        return self._collect(info)

    def generate_stream_with_suffix(self, req, prompt_suffix, on_token):
        """on_token(token, sampled, generated) may raise to abort, as the reference's Err."""
        sfx = np.ascontiguousarray(prompt_suffix, dtype=np.uint32)
        c, info = req.to_c(), _ffi.CdBatchInfo()
        failure = []

        def trampoline(tok, sampled, ns, generated, ng, _user):
            try:
                on_token(int(tok), [sampled[i] for i in range(ns)], [generated[i] for i in range(ng)])
                return 0
            except Exception as exc:  # noqa: BLE001 - forwarded to the caller below
                failure.append(exc)
                return 1

        cb = _ffi.STREAM_CB(trampoline)
        rc = lib.cd_session_generate_stream(self._h, C.byref(c), _u32(sfx), len(sfx), cb, None, C.byref(info))
        if failure:
            raise failure[0]
        if rc:
            raise ValueError(lib.cd_session_last_error(self._h).decode())
        return self._collect(info)
