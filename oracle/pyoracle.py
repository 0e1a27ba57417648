"""ctypes binding of the CPU oracle (oracle/oracle.h) — TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may
import this module; the shipped package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

F32, F16, BF16 = 0, 1, 2
QUANT_FP8, QUANT_INT4 = 3, 4
ACT_SWIGLU, ACT_LEAKY_RELU_SQ = 0, 1
BACKEND_AUTO, BACKEND_NAIVE, BACKEND_KV = 0, 1, 2
MODE_PREFILL_ONLY, MODE_NAIVE, MODE_KV = 0, 1, 2
BLOCK = 256

# tensor selectors of orc_model_tensor
T_EMBED, T_GAMMA_FINAL, T_LM_HEAD = 0, 1, 2
T_WQ, T_WK, T_WV, T_WO, T_W1, T_W3, T_W2, T_GAMMA1, T_GAMMA2 = range(10, 19)


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "dim", "hidden", "heads", "kv_heads", "hd", "seq", "nlayers", "vocab",
        "q_dim", "kv_dim", "gqa_ratio", "activation", "dtype", "untied")]


class Request(C.Structure):
    _fields_ = [("backend", C.c_int32), ("steps", C.c_int32), ("temperature", C.c_float),
                ("top_k", C.c_int32), ("samples", C.c_int32), ("seed", C.c_uint64)]


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "dim", "hidden", "heads", "seq", "nlayers", "vocab", "n_experts", "top_k", "n_shared",
        "kv_latent", "rope_dim", "nope_dim", "v_dim", "dtype", "untied")]


def make_config(dim, hidden, heads, hd, seq, nlayers, vocab, kv_heads=None, activation=ACT_SWIGLU,
                dtype=F32, untied=0):
    kv_heads = heads if kv_heads is None else kv_heads
    return Config(dim, hidden, heads, kv_heads, hd, seq, nlayers, vocab, heads * hd, kv_heads * hd,
                  heads // kv_heads, activation, dtype, untied)


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])


def _load():
    if not os.path.exists(_SO):
        build()
    lib = C.CDLL(_SO)
    P = C.POINTER
    f32p, u32p, i32p, u64p = P(C.c_float), P(C.c_uint32), P(C.c_int32), P(C.c_uint64)
    vp, cfgp = C.c_void_p, P(Config)
    sig = {
        "orc_rmsnorm": (C.c_float, [f32p, f32p, f32p, C.c_int]),
        "orc_embedding": (None, [f32p, C.c_int, u32p, C.c_int, f32p]),
        "orc_next_u64": (C.c_uint64, [u64p]),
        "orc_next_f32": (C.c_float, [u64p]),
        "orc_reference_random_vec": (None, [f32p, C.c_size_t, C.c_float]),
        "orc_round_to": (C.c_float, [C.c_float, C.c_int]),
        "orc_synth_value": (C.c_float, [C.c_uint64, C.c_uint64, C.c_uint64, C.c_float]),
        "orc_synth_prompt": (None, [C.c_uint64, C.c_int, u32p, C.c_int]),
        "orc_model_synth": (vp, [cfgp, C.c_uint64, C.c_float]),
        "orc_model_reference_random": (vp, [cfgp]),
        "orc_quant_dequant": (None, [f32p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "orc_model_synth_quant": (vp, [cfgp, C.c_uint64, C.c_float, C.c_int]),
        "orc_model_load": (vp, [C.c_char_p, C.c_char_p, C.c_int]),
        "orc_model_save": (C.c_int, [vp, C.c_char_p, C.c_int]),
        "orc_model_free": (None, [vp]),
        "orc_model_get_config": (None, [vp, cfgp]),
        "orc_model_set_kv_dtype": (None, [vp, C.c_int]),
        "orc_param_count": (C.c_size_t, [cfgp]),
        "orc_model_tensor": (C.c_size_t, [vp, C.c_int, C.c_int, f32p, C.c_size_t]),
        "orc_forward_logits": (C.c_int, [vp, u32p, C.c_int, C.c_float, C.c_int, i32p, C.c_int, f32p,
                                         f32p, f32p, f32p]),
        "orc_cache_new": (vp, [vp, C.c_int]),
        "orc_cache_free": (None, [vp]),
        "orc_cache_len": (C.c_size_t, [vp]),
        "orc_cache_set_len": (None, [vp, C.c_size_t]),
        "orc_cache_seed_cf": (None, [vp, C.c_int, C.c_size_t, f32p, f32p]),
        "orc_decode_token": (C.c_int, [vp, f32p, f32p]),
        "orc_decode_token_from_id": (C.c_int, [vp, C.c_uint32, f32p]),
        "orc_decode_logits": (C.c_int, [vp, C.c_uint32, C.c_float, f32p]),
        "orc_decode_argmax_from_id": (C.c_int, [vp, C.c_uint32, u32p]),
        "orc_decode_topk_from_id": (C.c_int, [vp, C.c_uint32, C.c_int, f32p, u32p]),
        "orc_decode_block_stats_from_id": (C.c_int, [vp, C.c_uint32, C.c_float, C.c_float, f32p, f32p]),
        "orc_materialize_block": (C.c_int, [vp, C.c_int, C.c_float, f32p]),
        "orc_sample_next": (C.c_uint32, [f32p, C.c_int, C.c_float, C.c_int, u64p]),
        "orc_sample_topk_candidates": (C.c_uint32, [u32p, f32p, C.c_int, C.c_float, u64p]),
        "orc_sample_block_from_stats": (C.c_int, [f32p, f32p, C.c_int, u64p]),
        "orc_sample_softmax_index": (C.c_int, [f32p, C.c_int, C.c_float, u64p]),
        "orc_merge_topk": (C.c_int, [f32p, u32p, C.c_int, C.c_int, f32p, u32p]),
        "orc_select_decode_mode": (C.c_int, [cfgp, C.c_int, C.c_int, C.c_int, P(C.c_char_p), P(C.c_char_p)]),
        "orc_moe_synth": (vp, [P(MoeConfig), C.c_uint64, C.c_float]),
        "orc_moe_free": (None, [vp]),
        "orc_moe_len": (C.c_size_t, [vp]),
        "orc_moe_set_len": (None, [vp, C.c_size_t]),
        "orc_moe_set_kv_dtype": (None, [vp, C.c_int]),
        "orc_moe_decode_logits": (C.c_int, [vp, C.c_uint32, f32p]),
        "orc_moe_last_experts": (C.c_int, [vp, C.c_int, i32p]),
        "orc_generate": (C.c_int, [vp, u32p, C.c_int, u32p, C.c_int, P(Request), C.c_float, C.c_int,
                                   u32p, f32p, i32p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def _f32(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _u32(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint32))


def _i32(a):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


def f32arr(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def u32arr(x):
    return np.ascontiguousarray(x, dtype=np.uint32)


def synth_prompt(seed, vocab, n):
    ids = np.zeros(n, dtype=np.uint32)
    lib.orc_synth_prompt(seed, vocab, _u32(ids), n)
    return ids


class Model:
    """An oracle model: synthetic, reference-random or loaded from an RSTK file."""

    def __init__(self, handle):
        if not handle:
            raise RuntimeError("oracle model construction failed")
        self.h = C.c_void_p(handle)
        self.cfg = Config()
        lib.orc_model_get_config(self.h, C.byref(self.cfg))

    @classmethod
    def synth(cls, cfg, seed, std=0.02):
        return cls(lib.orc_model_synth(C.byref(cfg), seed, std))

    @classmethod
    def synth_quant(cls, cfg, seed, mode, std=0.02):
        """Synthetic model with quantised linears (mode QUANT_FP8 / QUANT_INT4); cfg.dtype must be F32."""
        return cls(lib.orc_model_synth_quant(C.byref(cfg), seed, std, mode))

    @classmethod
    def reference_random(cls, cfg):
        return cls(lib.orc_model_reference_random(C.byref(cfg)))

    @classmethod
    def load(cls, path):
        err = C.create_string_buffer(256)
        h = lib.orc_model_load(os.fsencode(path), err, 256)
        if not h:
            raise ValueError(err.value.decode())
        return cls(h)

    def save(self, path, version=3):
        rc = lib.orc_model_save(self.h, os.fsencode(path), version)
        if rc:
            raise ValueError("orc_model_save failed: %d" % rc)

    def __del__(self):
        if getattr(self, "h", None):
            lib.orc_model_free(self.h)
            self.h = None

    def set_kv_dtype(self, dtype):
        """What a rounding cache (kv_round=1) rounds keys and values to: F32, F16 or BF16."""
        lib.orc_model_set_kv_dtype(self.h, dtype)
        return self

    def tensor(self, which, layer=0):
        n = lib.orc_model_tensor(self.h, layer, which, None, 0)
        out = np.zeros(n, dtype=np.float32)
        if n:
            lib.orc_model_tensor(self.h, layer, which, _f32(out), n)
        return out

    def forward_logits(self, tokens, rows=None, softcap=0.0, kv_round=0, want_kv=False, want_x=False):
        """naive_full_context forward over len(tokens) positions; returns logits rows."""
        c = self.cfg
        tokens = u32arr(tokens)
        npos = len(tokens)
        rows = np.ascontiguousarray([npos - 1] if rows is None else rows, dtype=np.int32)
        logits = np.zeros((len(rows), c.vocab), dtype=np.float32)
        kcf = vcf = None
        if want_kv:
            kcf = np.zeros((c.nlayers, c.kv_dim, c.seq), dtype=np.float32)
            vcf = np.zeros_like(kcf)
        x = np.zeros(c.dim, dtype=np.float32) if want_x else None
        rc = lib.orc_forward_logits(self.h, _u32(tokens), npos, softcap, kv_round, _i32(rows), len(rows),
                                    _f32(logits), _f32(kcf) if want_kv else None,
                                    _f32(vcf) if want_kv else None, _f32(x) if want_x else None)
        if rc:
            raise ValueError("orc_forward_logits failed: %d" % rc)
        out = [logits]
        if want_kv:
            out += [kcf, vcf]
        if want_x:
            out.append(x)
        return out[0] if len(out) == 1 else tuple(out)

    def generate(self, prompt, steps, backend=BACKEND_NAIVE, temperature=0.0, top_k=0, samples=1, seed=1,
                 suffix=(), softcap=0.0, kv_round=0, trace=False):
        prompt, suffix = u32arr(prompt), u32arr(suffix)
        req = Request(backend, steps, temperature, top_k, samples, seed)
        toks = np.zeros((samples, steps), dtype=np.uint32)
        tr = np.zeros((steps, self.cfg.vocab), dtype=np.float32) if trace else None
        mode = C.c_int32(-1)
        rc = lib.orc_generate(self.h, _u32(prompt), len(prompt), _u32(suffix), len(suffix), C.byref(req),
                              softcap, kv_round, _u32(toks), _f32(tr) if trace else None,
                              C.cast(C.byref(mode), C.POINTER(C.c_int32)))
        if rc:
            raise ValueError("orc_generate failed: %d" % rc)
        return (toks, tr, mode.value) if trace else (toks, mode.value)


class Cache:
    """The KV-cached decode model (restates metal_decode::Model's public methods)."""

    def __init__(self, model, kv_round=0):
        self.model = model
        self.h = C.c_void_p(lib.orc_cache_new(model.h, kv_round))
        self.nblocks = (model.cfg.vocab + BLOCK - 1) // BLOCK

    def __del__(self):
        if getattr(self, "h", None):
            lib.orc_cache_free(self.h)
            self.h = None

    def len(self):
        return lib.orc_cache_len(self.h)

    def set_len(self, n):
        lib.orc_cache_set_len(self.h, n)

    def seed_layer_cache_from_channel_first(self, layer, live_len, k_cf, v_cf):
        k_cf, v_cf = f32arr(k_cf), f32arr(v_cf)
        lib.orc_cache_seed_cf(self.h, layer, live_len, _f32(k_cf), _f32(v_cf))

    def _chk(self, rc):
        if rc < 0:
            raise ValueError("oracle decode failed: %d" % rc)
        return rc

    def decode_token(self, x_in):
        x_in = f32arr(x_in)
        out = np.zeros(self.model.cfg.dim, dtype=np.float32)
        self._chk(lib.orc_decode_token(self.h, _f32(x_in), _f32(out)))
        return out

    def decode_token_from_id(self, tok):
        out = np.zeros(self.model.cfg.dim, dtype=np.float32)
        self._chk(lib.orc_decode_token_from_id(self.h, tok, _f32(out)))
        return out

    def decode_logits(self, tok, softcap=0.0):
        out = np.zeros(self.model.cfg.vocab, dtype=np.float32)
        self._chk(lib.orc_decode_logits(self.h, tok, softcap, _f32(out)))
        return out

    def decode_token_argmax_from_id(self, tok):
        out = C.c_uint32(0)
        self._chk(lib.orc_decode_argmax_from_id(self.h, tok, C.byref(out)))
        return out.value

    def decode_token_topk_from_id(self, tok, k):
        vals = np.zeros(self.nblocks * k, dtype=np.float32)
        idxs = np.zeros(self.nblocks * k, dtype=np.uint32)
        n = self._chk(lib.orc_decode_topk_from_id(self.h, tok, k, _f32(vals), _u32(idxs)))
        return vals[:n], idxs[:n]

    def decode_token_block_stats_from_id(self, tok, inv_t, softcap=0.0):
        mx = np.zeros(self.nblocks, dtype=np.float32)
        sm = np.zeros(self.nblocks, dtype=np.float32)
        self._chk(lib.orc_decode_block_stats_from_id(self.h, tok, inv_t, softcap, _f32(mx), _f32(sm)))
        return mx, sm

    def materialize_current_logits_block(self, block, softcap=0.0):
        out = np.zeros(BLOCK, dtype=np.float32)
        n = self._chk(lib.orc_materialize_block(self.h, block, softcap, _f32(out)))
        return out[:n]


class MoeModel:
    """The MoE + MLA decoder of oracle_moe.cpp: one cached sequence, logits per fed token."""

    def __init__(self, cfg, seed, std=0.02):
        self.cfg = cfg
        self.h = C.c_void_p(lib.orc_moe_synth(C.byref(cfg), seed, std))
        if not self.h:
            raise RuntimeError("oracle MoE model construction failed")

    def __del__(self):
        if getattr(self, "h", None):
            lib.orc_moe_free(self.h)
            self.h = None

    def len(self):
        return lib.orc_moe_len(self.h)

    def set_len(self, n):
        lib.orc_moe_set_len(self.h, n)

    def set_kv_dtype(self, dtype):
        lib.orc_moe_set_kv_dtype(self.h, dtype)
        return self

    def decode_logits(self, tok):
        out = np.zeros(self.cfg.vocab, dtype=np.float32)
        if lib.orc_moe_decode_logits(self.h, tok, _f32(out)):
            raise ValueError("oracle MoE decode failed")
        return out

    def last_experts(self, layer):
        out = np.zeros(self.cfg.top_k, dtype=np.int32)
        lib.orc_moe_last_experts(self.h, layer, _i32(out))
        return out


def merge_topk(vals, idxs, top_k):
    vals, idxs = f32arr(vals), u32arr(idxs)
    ov = np.zeros(top_k, dtype=np.float32)
    oi = np.zeros(top_k, dtype=np.uint32)
    n = lib.orc_merge_topk(_f32(vals), _u32(idxs), len(vals), top_k, _f32(ov), _u32(oi))
    return ov[:n], oi[:n]


def select_decode_mode(cfg, backend, ctx_len, steps):
    fb, ar = C.c_char_p(), C.c_char_p()
    mode = lib.orc_select_decode_mode(C.byref(cfg), backend, ctx_len, steps, C.byref(fb), C.byref(ar))
    return mode, (fb.value.decode() if fb.value else None), (ar.value.decode() if ar.value else None)
