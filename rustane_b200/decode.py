"""Python mirror of `metal_decode::Model` (crates/metal-decode/src/lib.rs:129-511) and of
`engine::decode::DecodeContext` (crates/engine/src/decode.rs:14-197) over the CUDA library.

Method names, argument meaning and error behaviour follow the reference; where the
reference panics (assert!/expect) these raise CudaDecodeError carrying the same message.
"""
import ctypes as C
import os

import numpy as np

from . import _ffi
from ._ffi import CudaDecodeError, lib

MAX_GPU_TOPK = _ffi.MAX_GPU_TOPK
HEAD_BLOCK = _ffi.HEAD_BLOCK
_DTYPES = {"f32": 0, "fp32": 0, "f16": 1, "fp16": 1, "bf16": 2, "fp8": 3, "int4": 4}


def _f32(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _u32(a):
    return a.ctypes.data_as(C.POINTER(C.c_uint32))


def _cf32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


class Config:
    """metal_decode::Config (lib.rs:22-35)."""

    def __init__(self, dim, hidden, heads, hd, seq, nlayers, vocab, kv_heads=None):
        kv_heads = heads if kv_heads is None else kv_heads
        self.dim, self.hidden, self.heads, self.kv_heads, self.hd = dim, hidden, heads, kv_heads, hd
        self.seq, self.nlayers, self.vocab = seq, nlayers, vocab
        self.q_dim, self.kv_dim, self.gqa_ratio = heads * hd, kv_heads * hd, heads // kv_heads

    def to_c(self):
        return _ffi.CdConfig(self.dim, self.hidden, self.heads, self.kv_heads, self.hd, self.seq, self.nlayers,
                             self.vocab, self.q_dim, self.kv_dim, self.gqa_ratio)

    @classmethod
    def from_c(cls, c):
        return cls(c.dim, c.hidden, c.heads, c.hd, c.seq, c.nlayers, c.vocab, kv_heads=c.kv_heads)

    def param_count(self):
        """ModelConfig::param_count (model.rs:182-187)."""
        c = self.to_c()
        return lib.cd_param_count(C.byref(c))

    def __repr__(self):
        return "Config(dim=%d, hidden=%d, heads=%d, kv_heads=%d, hd=%d, seq=%d, nlayers=%d, vocab=%d)" % (
            self.dim, self.hidden, self.heads, self.kv_heads, self.hd, self.seq, self.nlayers, self.vocab)


_KV_DTYPES = {None: 0, "auto": 0, "f32": 1, "fp32": 1, "f16": 2, "fp16": 2, "bf16": 3}


def _options(dtype="f32", activation=0, device=-1, page_tokens=0, max_samples=1, use_graph=False, kv_dtype=None,
             tp_rank=0, tp_world=1, wait_us=0, pdl=True, ring_kb=0, mega=True, trace=False, drop_stage=False):
    """cd_options.  kv_dtype: storage of the KV cache (None: fp32 with fp32 weights, else fp16);
    tp_rank / tp_world: this process holds shard tp_rank of a tensor-parallel model over tp_world GPUs;
    wait_us: bound of every device-side wait on a peer GPU.  Test-only: pdl (programmatic dependent
    launch between the kernels of a token), ring_kb (shared memory per GEMV CTA), mega (False: one kernel
    per operator even where the one-kernel-per-token path applies), trace (phase stamps of that path),
    drop_stage (a weight stage of every streamed GEMV never arrives: the bounded wait for it runs out)."""
    o = _ffi.CdOptions()
    o.weight_dtype = _DTYPES[dtype] if isinstance(dtype, str) else int(dtype)
    o.activation, o.device, o.page_tokens = activation, device, page_tokens
    o.max_samples, o.use_graph = max_samples, int(bool(use_graph))
    o.kv_dtype = _KV_DTYPES[kv_dtype]
    o.tp_rank, o.tp_world, o.wait_us = tp_rank, tp_world, wait_us
    o.test_flags = (0 if pdl else 1) | (0 if mega else 2) | (4 if trace else 0) | (8 if drop_stage else 0)
    o.test_ring_kb = ring_kb
    return o


class MoeConfig:
    """cd_moe_config + the matching cd_config of a MoE + MLA decoder (no reference counterpart)."""

    def __init__(self, dim, hidden, heads, seq, nlayers, vocab, n_experts, top_k, n_shared, kv_latent, rope_dim, nope_dim, v_dim):
        self.n_experts, self.top_k, self.n_shared = n_experts, top_k, n_shared
        self.kv_latent, self.rope_dim, self.nope_dim, self.v_dim = kv_latent, rope_dim, nope_dim, v_dim
        self.base = Config(dim, hidden, heads, nope_dim + rope_dim, seq, nlayers, vocab, kv_heads=1)
        self.base.kv_dim = kv_latent + rope_dim

    def to_c(self):
        return _ffi.CdMoeConfig(self.n_experts, self.top_k, self.n_shared, self.kv_latent, self.rope_dim, self.nope_dim, self.v_dim)


class Model:
    """A KV-cached single-token decoder resident on one B200."""

    def __init__(self, handle, cfg):
        self._h = C.c_void_p(handle)
        self.cfg = cfg
        self.argmax_blocks = (cfg.vocab + HEAD_BLOCK - 1) // HEAD_BLOCK

    # ---- construction -------------------------------------------------------------
    @classmethod
    def new(cls, cfg, layers, final_head, **opts):
        """Model::new (lib.rs:147): `layers` is a sequence of dicts with wq, wk, wv, wo, w1, w3,
        w2, gamma1, gamma2 (fp32, reference layouts); `final_head` has gamma_final, embed and
        optionally lm_head.  Returns None when the layer count is wrong, as the reference."""
        layers = list(layers)
        if len(layers) != cfg.nlayers:
            return None
        keep = []
        arr = (_ffi.CdLayerInit * len(layers))()
        for i, L in enumerate(layers):
            for name in ("wq", "wk", "wv", "wo", "w1", "w3", "w2", "gamma1", "gamma2"):
                a = _cf32(L[name])
                keep.append(a)
                setattr(arr[i], name, _f32(a))
        head = _ffi.CdHeadInit()
        for name in ("gamma_final", "embed", "lm_head"):
            v = final_head.get(name)
            if v is not None:
                a = _cf32(v)
                keep.append(a)
                setattr(head, name, _f32(a))
        c, o, h = cfg.to_c(), _options(**opts), C.c_void_p()
        rc = lib.cd_model_create(C.byref(c), arr, len(layers), C.byref(head), C.byref(o), C.byref(h))
        if rc:
            raise CudaDecodeError(rc, lib.cd_last_error(None).decode())
        return cls(h.value, cfg)

    @classmethod
    def synthetic(cls, cfg, seed, std=0.02, untied_head=False, **opts):
        c, o, h = cfg.to_c(), _options(**opts), C.c_void_p()
        rc = lib.cd_model_create_synthetic(C.byref(c), C.byref(o), seed, std, int(untied_head), C.byref(h))
        if rc:
            raise CudaDecodeError(rc, lib.cd_last_error(None).decode())
        return cls(h.value, cfg)

    @classmethod
    def moe_synthetic(cls, mcfg, seed, std=0.02, untied_head=False, **opts):
        """A MoE + MLA decoder with seeded synthetic weights; every Model method that takes token ids works on it."""
        c, mc, o, h = mcfg.base.to_c(), mcfg.to_c(), _options(**opts), C.c_void_p()
        rc = lib.cd_moe_model_create_synthetic(C.byref(c), C.byref(mc), C.byref(o), seed, std, int(untied_head), C.byref(h))
        if rc:
            raise CudaDecodeError(rc, lib.cd_last_error(None).decode())
        m = cls(h.value, mcfg.base)
        m.moe = mcfg
        return m

    def moe_last_experts(self, layer):
        out = np.zeros(self.moe.top_k, dtype=np.int32)
        self._check(lib.cd_moe_last_experts(self._h, layer, out.ctypes.data_as(C.POINTER(C.c_int32)), len(out)))
        return out

    @classmethod
    def from_checkpoint(cls, path, dtype=None, **opts):
        o = _options(**opts)
        o.weight_dtype = -1 if dtype is None else _DTYPES[dtype]
        c, h = _ffi.CdConfig(), C.c_void_p()
        rc = lib.cd_model_create_from_checkpoint(os.fsencode(path), C.byref(o), C.byref(c), C.byref(h))
        if rc:
            raise CudaDecodeError(rc, lib.cd_last_error(None).decode())
        return cls(h.value, Config.from_c(c))

    def save_quantised(self, path):
        """Write this (single-GPU, dense, FP8 or INT4) model as a quantised RSTK v3 file."""
        self._check(lib.cd_model_save_quantised(self._h, os.fsencode(path)))

    def linear_rows(self, layer, which, nbytes):
        """This rank's rows of linear `which` (0 wq, 1 wk, 2 wv, 3 wo, 4 w1, 5 w3, 6 w2) of a quantised model, as stored on the device."""
        out = np.empty(nbytes, dtype=np.uint8)
        self._check(lib.cd_model_get_linear_rows(self._h, layer, which, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def close(self):
        if self._h:
            lib.cd_model_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def _check(self, rc):
        if rc:
            raise CudaDecodeError(rc, lib.cd_last_error(self._h).decode())

    # ---- state ------------------------------------------------------------------
    def len(self):
        n = C.c_size_t()
        self._check(lib.cd_len(self._h, C.byref(n)))
        return n.value

    def set_len(self, n):
        self._check(lib.cd_set_len(self._h, n))

    def seed_layer_cache_from_channel_first(self, layer_idx, live_len, k_rope_cf, v_cf):
        k, v = _cf32(k_rope_cf), _cf32(v_cf)
        need = self.cfg.kv_dim * self.cfg.seq
        if k.size < need or v.size < need:
            raise ValueError("k_rope_cf / v_cf must hold kv_dim * seq values")
        self._check(lib.cd_seed_layer_cache_cf(self._h, layer_idx, live_len, _f32(k), _f32(v)))

    # ---- the six decode entry points --------------------------------------------------
    def decode_token(self, x_in):
        x = _cf32(x_in)
        if x.size != self.cfg.dim:
            raise ValueError("x_in must have dim elements")
        out = np.empty(self.cfg.dim, dtype=np.float32)
        self._check(lib.cd_decode_token(self._h, _f32(x), _f32(out)))
        return out

    def decode_token_from_id(self, token):
        out = np.empty(self.cfg.dim, dtype=np.float32)
        self._check(lib.cd_decode_token_from_id(self._h, token, _f32(out)))
        return out

    def decode_token_argmax(self, x_in):
        x = _cf32(x_in)
        if x.size != self.cfg.dim:
            raise ValueError("x_in must have dim elements")
        tok = C.c_uint32()
        self._check(lib.cd_decode_token_argmax(self._h, _f32(x), C.byref(tok)))
        return tok.value

    def decode_token_argmax_from_id(self, token):
        tok = C.c_uint32()
        self._check(lib.cd_decode_token_argmax_from_id(self._h, token, C.byref(tok)))
        return tok.value

    def decode_token_topk_from_id(self, token, top_k):
        cap = self.argmax_blocks * max(int(top_k), 1)
        vals = np.empty(cap, dtype=np.float32)
        idxs = np.empty(cap, dtype=np.uint32)
        n = C.c_size_t()
        self._check(lib.cd_decode_token_topk_from_id(self._h, token, top_k, _f32(vals), _u32(idxs), cap, C.byref(n)))
        return vals[:n.value], idxs[:n.value]

    def decode_token_block_stats_from_id(self, token, inv_temperature, softcap=0.0):
        mx = np.empty(self.argmax_blocks, dtype=np.float32)
        sm = np.empty(self.argmax_blocks, dtype=np.float32)
        n = C.c_size_t()
        self._check(lib.cd_decode_token_block_stats_from_id(self._h, token, inv_temperature, softcap, _f32(mx),
                                                            _f32(sm), self.argmax_blocks, C.byref(n)))
        return mx[:n.value], sm[:n.value]

    def materialize_current_logits_block(self, block_idx, softcap=0.0):
        out = np.empty(HEAD_BLOCK, dtype=np.float32)
        n = C.c_size_t()
        self._check(lib.cd_materialize_current_logits_block(self._h, block_idx, softcap, _f32(out), HEAD_BLOCK,
                                                            C.byref(n)))
        return out[:n.value]

    # ---- additive: device-resident loops ------------------------------------------------
    def decode_token_logits_from_id(self, token, softcap=0.0):
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        self._check(lib.cd_decode_token_logits_from_id(self._h, token, softcap, _f32(out)))
        return out

    def prefill(self, ids, softcap=0.0, want_logits=True):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        out = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        self._check(lib.cd_prefill(self._h, _u32(ids), len(ids), softcap, _f32(out) if want_logits else None))
        return out

    def decode_steps_greedy(self, first_token, nsteps):
        out = np.empty(nsteps, dtype=np.uint32)
        self._check(lib.cd_decode_steps_greedy(self._h, first_token, nsteps, _u32(out)))
        return out

    def decode_steps_topk(self, first_token, nsteps, top_k, temperature, rng_state, softcap=0.0):
        out = np.empty(nsteps, dtype=np.uint32)
        rng = C.c_uint64(rng_state)
        self._check(lib.cd_decode_steps_topk(self._h, first_token, nsteps, top_k, temperature, softcap,
                                             C.byref(rng), _u32(out)))
        return out, rng.value

    def decode_steps_fullvocab(self, first_token, nsteps, temperature, rng_state, softcap=0.0):
        out = np.empty(nsteps, dtype=np.uint32)
        rng = C.c_uint64(rng_state)
        self._check(lib.cd_decode_steps_fullvocab(self._h, first_token, nsteps, temperature, softcap,
                                                  C.byref(rng), _u32(out)))
        return out, rng.value

    def decode_steps_samples(self, first_tokens, nsteps, mode="greedy", top_k=0, temperature=0.0, rng_states=None, softcap=0.0):
        """`--samples N` sharing the cached prompt: sample s feeds first_tokens[s] and draws nsteps tokens
        with LCG state rng_states[s], all samples advancing together.  Returns (ids [N, nsteps], rng states)."""
        first = np.ascontiguousarray(first_tokens, dtype=np.uint32)
        ns = len(first)
        out = np.empty((ns, nsteps), dtype=np.uint32)
        rng = np.array(rng_states if rng_states is not None else np.zeros(ns), dtype=np.uint64)  # a copy: the call advances it
        self._check(lib.cd_decode_steps_samples(self._h, _u32(first), ns, nsteps, {"greedy": 0, "topk": 1, "fullvocab": 2}[mode], top_k,
                                                temperature, softcap, rng.ctypes.data_as(C.POINTER(C.c_uint64)), _u32(out)))
        return out, rng

    # ---- tensor parallelism (one process per GPU) -------------------------------------------
    def tp_region_handle(self):
        """The 64-byte CUDA IPC handle of this rank's link region."""
        buf = C.create_string_buffer(64)
        self._check(lib.cd_tp_region_handle(self._h, buf, 64))
        return buf.raw

    def tp_connect(self, handles):
        """handles: the regions' handles of all ranks, in rank order (bytes each)."""
        blob = b"".join(handles)
        self._check(lib.cd_tp_connect(self._h, blob, len(handles)))

    def tp_region_ptr(self):
        """This rank's link region as a device pointer (ranks living in one process)."""
        p = C.c_void_p()
        self._check(lib.cd_tp_region_ptr(self._h, C.byref(p)))
        return p.value

    def tp_connect_ptrs(self, regions):
        arr = (C.c_void_p * len(regions))(*regions)
        self._check(lib.cd_tp_connect_ptrs(self._h, arr, len(regions)))

    def tp_connect_group(self, group=None):
        """Exchange the handles over torch.distributed (any backend) and connect."""
        import torch
        import torch.distributed as dist
        world = dist.get_world_size(group)
        dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
        mine = torch.tensor(list(self.tp_region_handle()), dtype=torch.uint8, device=dev)
        allh = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine, group=group)
        self.tp_connect([bytes(t.cpu().tolist()) for t in allh])
        dist.barrier(group)

    KERNEL_CLASSES = ("misc", "qkv_gemv", "attention", "wo_gemv", "w13_gemv", "w2_gemv", "head_gemv", "head_reduce")

    def profile_decode_step(self, token):
        """One greedy step with an event behind every kernel: {class: (ms, launches)}."""
        ms = np.zeros(8, dtype=np.float32)
        n = np.zeros(8, dtype=np.uint32)
        self._check(lib.cd_profile_decode_step(self._h, token, _f32(ms), _u32(n), 8))
        return {k: (float(ms[i]), int(n[i])) for i, k in enumerate(self.KERNEL_CLASSES)}

    def last_device_ms(self):
        ms = C.c_float()
        self._check(lib.cd_last_device_ms(self._h, C.byref(ms)))
        return ms.value

    def kernel_launches(self):
        n = C.c_uint64()
        self._check(lib.cd_kernel_launches(self._h, C.byref(n)))
        return n.value


def merge_topk_candidates(vals, idxs, top_k):
    """decode.rs:218-253."""
    vals, idxs = _cf32(vals), np.ascontiguousarray(idxs, dtype=np.uint32)
    ov = np.empty(top_k, dtype=np.float32)
    oi = np.empty(top_k, dtype=np.uint32)
    n = lib.cd_merge_topk_candidates(_f32(vals), _u32(idxs), len(vals), top_k, _f32(ov), _u32(oi))
    return ov[:n], oi[:n]


class DecodeContext:
    """engine::decode::DecodeContext (decode.rs:14-197): the five per-token calls the session makes."""

    def __init__(self, model):
        self.model = model

    def seed_from_forward_caches(self, k_cf_layers, v_cf_layers, live_len):
        live_len = min(live_len, self.model.cfg.seq)
        self.model.set_len(live_len)
        for l, (k, v) in enumerate(zip(k_cf_layers, v_cf_layers)):
            self.model.seed_layer_cache_from_channel_first(l, live_len, k, v)

    def decode_next_logits(self, token, softcap=0.0):
        return self.model.decode_token_logits_from_id(token, softcap)

    def decode_next_greedy_token(self, token):
        return self.model.decode_token_argmax_from_id(token)

    def decode_next_topk_candidates(self, token, top_k, softcap=0.0):
        top_k = min(top_k, MAX_GPU_TOPK, self.model.cfg.vocab)
        vals, idxs = self.model.decode_token_topk_from_id(token, top_k)
        mv, mi = merge_topk_candidates(vals, idxs, top_k)
        if softcap > 0.0:
            mv = (softcap * np.tanh(mv / np.float32(softcap))).astype(np.float32)
        return mi, mv

    def decode_next_fullvocab_block_stats(self, token, temperature, softcap=0.0):
        inv_t = np.float32(1.0) / max(np.float32(temperature), np.finfo(np.float32).tiny)
        return self.model.decode_token_block_stats_from_id(token, float(inv_t), softcap)

    def materialize_current_logits_block(self, block_idx, softcap=0.0):
        return self.model.materialize_current_logits_block(block_idx, softcap)
