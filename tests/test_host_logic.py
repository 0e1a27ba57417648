"""CPU-only checks of the shipped library's host side: the C ABI loads and exports every
symbol the header declares, and the host policy / samplers / checkpoint code agree with
the oracle bit for bit.  No compute call is made here (there is no GPU)."""
import ctypes as C
import os
import re
import struct

import numpy as np
import pytest

from helpers import gpu_cfg, oracle_cfg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(R):
    from rustane_b200 import _ffi
    header = open(os.path.join(ROOT, "include", "cuda_decode.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(cd_[a-z0-9_]+)\s*\(", header))
    declared -= {"cd_stream_cb"}
    assert len(declared) >= 45
    raw = C.CDLL(_ffi.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), "libcuda_decode.so does not export %s" % name
    assert declared == set(_ffi.SIGNATURES), "binding table and header disagree: %s" % (
        declared ^ set(_ffi.SIGNATURES))


def test_construction_fails_loudly_without_a_gpu(R):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(R.CudaDecodeError):
        R.Model.synthetic(R.Config(256, 640, 2, 128, 64, 2, 64), seed=0)


def test_policy_matches_oracle(R, oracle):
    O = oracle
    names = {O.MODE_PREFILL_ONLY: "prefill_only", O.MODE_NAIVE: "naive_full_context", O.MODE_KV: "kv_cache_cuda"}
    back = {"auto": O.BACKEND_AUTO, "naive": O.BACKEND_NAIVE, "cuda": O.BACKEND_KV}
    for dims in [(256, 640, 2, 128, 64, 2, 8192), (1024, 2816, 8, 128, 512, 8, 8192)]:
        oc = oracle_cfg(O, *dims)
        gc = gpu_cfg(R, oc)
        assert gc.param_count() == O.lib.orc_param_count(C.byref(oc))
        for b in back:
            for ctx in (1, 4, 60, 500, 512):
                for steps in (0, 1, 2, 8, 20, 600):
                    mode, fb, ar = O.select_decode_mode(oc, back[b], ctx, steps)
                    sel = R.select_decode_mode(gc, b, ctx, steps)
                    assert (sel.mode, sel.fallback_reason, sel.auto_reason) == (names[mode], fb, ar)
    assert R.parse_decode_backend("cuda") == "cuda" and R.parse_decode_backend("metal") is None


def test_samplers_match_oracle(R, oracle):
    from rustane_b200 import inference as I
    O = oracle
    rng = np.random.default_rng(1)
    for trial in range(40):
        n = int(rng.integers(2, 700))
        logits = (rng.standard_normal(n) * 3).astype(np.float32)
        if trial % 5 == 0:
            logits[rng.integers(0, n, 3)] = logits.max()  # exact ties
        for (t, k) in [(0.0, 0), (0.8, 1), (0.8, 8), (1.0, 0), (0.7, 40), (1.3, 5000)]:
            s1 = np.array([trial * 977 + 11], dtype=np.uint64)
            s2 = C.c_uint64(int(s1[0]))
            a = I.sample_next(logits, t, k, s1)
            b = O.lib.orc_sample_next(O._f32(logits), n, t, k, C.byref(s2))
            assert a == b and int(s1[0]) == s2.value
        idxs = rng.permutation(n)[: min(n, 8)].astype(np.uint32)
        cl = np.sort(logits[idxs])[::-1].copy()
        s1 = np.array([trial + 5], dtype=np.uint64)
        s2 = C.c_uint64(trial + 5)
        assert I.sample_topk_candidates(idxs, cl, 0.9, s1) == O.lib.orc_sample_topk_candidates(
            O._u32(idxs), O._f32(cl), len(idxs), 0.9, C.byref(s2))
        mx = (rng.standard_normal(9) * 2).astype(np.float32)
        sm = (rng.random(9) * 100 + 1).astype(np.float32)
        if trial % 7 == 0:
            mx[2] = -np.inf
            sm[4] = 0
        s1 = np.array([trial + 99], dtype=np.uint64)
        s2 = C.c_uint64(trial + 99)
        assert I.sample_block_from_stats(mx, sm, s1) == O.lib.orc_sample_block_from_stats(
            O._f32(mx), O._f32(sm), 9, C.byref(s2))
        assert I.sample_block_logits(256, logits[:200], 0.8, s1) == 256 + O.lib.orc_sample_softmax_index(
            O._f32(np.ascontiguousarray(logits[:200])), min(n, 200), 0.8, C.byref(s2))
        assert int(s1[0]) == s2.value


def test_merge_matches_oracle(R, oracle):
    rng = np.random.default_rng(2)
    for _ in range(30):
        n = int(rng.integers(1, 300))
        vals = rng.integers(-5, 5, n).astype(np.float32)  # many ties
        idxs = rng.permutation(5000)[:n].astype(np.uint32)
        vals[rng.integers(0, n)] = -np.inf
        idxs[rng.integers(0, n)] = 0xFFFFFFFF
        for k in (1, 4, 32):
            v1, i1 = R.merge_topk_candidates(vals, idxs, k)
            v2, i2 = oracle.merge_topk(vals, idxs, k)
            np.testing.assert_array_equal(v1, v2)
            np.testing.assert_array_equal(i1, i2)


def test_synthetic_generator_matches_oracle_and_is_plausibly_normal(R, oracle):
    vals = np.array([R.synth_value(3, 16 + 5, i, 0.02) for i in range(20000)], dtype=np.float32)
    ref = np.array([oracle.lib.orc_synth_value(3, 16 + 5, i, 0.02) for i in range(20000)], dtype=np.float32)
    np.testing.assert_array_equal(vals, ref)
    assert abs(vals.mean()) < 1e-3 and abs(vals.std() - 0.02) < 5e-4
    np.testing.assert_array_equal(R.synth_prompt(1, 32000, 512), oracle.synth_prompt(1, 32000, 512))
    assert R.synth_prompt(1, 32000, 512).max() < 32000


@pytest.mark.parametrize("dtype,untied", [("f32", False), ("bf16", True), ("f16", False)])
def test_written_checkpoint_equals_oracle_synth(R, oracle, tmp_path, dtype, untied):
    O = oracle
    oc = oracle_cfg(O, 128, 256, 2, 64, 32, 2, 96, dtype=dtype, untied=int(untied), activation=1)
    path = str(tmp_path / "m.rstk")
    R.write_synthetic_checkpoint(path, gpu_cfg(R, oc), dtype=dtype, activation=1, untied_head=untied, seed=4)
    info = R.checkpoint_info(path)
    assert (info["version"], info["dtype"], info["activation"], info["untied_head"]) == (3, oc.dtype, 1, untied)
    assert repr(info["cfg"]) == repr(gpu_cfg(R, oc))
    loaded, synth = O.Model.load(path), O.Model.synth(oc, 4)
    for which, layer in [(O.T_EMBED, 0), (O.T_WQ, 1), (O.T_WO, 0), (O.T_W2, 1), (O.T_W3, 0), (O.T_GAMMA2, 1)] + (
            [(O.T_LM_HEAD, 0)] if untied else []):
        np.testing.assert_array_equal(loaded.tensor(which, layer), synth.tensor(which, layer))


def test_checkpoint_errors_carry_reference_messages(R, tmp_path):
    p = tmp_path / "bad.bin"
    cases = [
        (b"RST", "checkpoint too small for header"),
        (b"XXXX" + b"\0" * 28, "invalid checkpoint magic"),
        (b"RSTK" + struct.pack("<6I", 7, 0, 128, 1, 1, 1), "unsupported checkpoint version 7"),
        (b"RSTK" + struct.pack("<7I", 2, 0, 128, 1, 1, 1, 5), "unsupported checkpoint activation code 5"),
        (b"RSTK" + struct.pack("<7I", 2, 0, 0, 1, 1, 1, 0), "zero dimension"),
        (b"RSTK" + struct.pack("<7I", 2, 0, 100, 1, 1, 1, 0) + b"\0" * 8, "not divisible by 128"),
        (b"RSTK" + struct.pack("<7I", 2, 0, 128, 1, 1, 1, 0) + b"\0" * 7, "not aligned to f32"),
        (b"RSTK" + struct.pack("<7I", 2, 0, 128, 1, 1, 1, 0) + b"\0" * 64, "too small for fixed-size tensors"),
        (b"RSTK" + struct.pack("<13I", 3, 0, 128, 1, 8, 8, 0, 64, 2, 2, 64, 0, 0) + b"\0" * 64, "unexpected EOF"),
    ]
    for blob, msg in cases:
        p.write_bytes(blob)
        with pytest.raises(ValueError, match=msg):
            R.checkpoint_info(str(p))
    with pytest.raises(ValueError, match="cannot open"):
        R.checkpoint_info(str(tmp_path / "absent.bin"))


def test_v2_writer_reader_roundtrip_and_shape_rule(R, oracle, tmp_path):
    cfg = R.Config(256, 640, 2, 128, 64, 2, 64)
    path = str(tmp_path / "v2.rstk")
    R.write_synthetic_checkpoint(path, cfg, dtype="f32", version=2, seed=8)
    info = R.checkpoint_info(path)
    assert info["version"] == 2 and info["cfg"].hidden == 640 and info["cfg"].heads == 2
    om = oracle.Model.load(path)  # the reference's v2 rules: hd 128, heads = dim/128, hidden inferred
    assert (om.cfg.hidden, om.cfg.heads, om.cfg.hd) == (640, 2, 128)
    with pytest.raises(R.CudaDecodeError):  # hd 64 cannot be expressed before v3
        R.write_synthetic_checkpoint(path, R.Config(128, 256, 2, 64, 32, 2, 96), version=2)


def test_quantised_checkpoint_header(R, tmp_path):
    """RSTK v3 with flags bit1: dtype code 3 (FP8 rows of K + 16 bytes) or 4 (INT4 rows of K/2 + K/16 bytes, padded to
    16); the payload length is checked against those row sizes, embedding as bf16."""
    import struct
    D, H, HEADS, HD, V, L = 128, 256, 2, 64, 96, 2
    def body(dtype_code, flags, trim=0):
        rb = (lambda k: k + 16) if dtype_code == 3 else (lambda k: (k // 2 + k // 16 + 15) // 16 * 16)
        q = kv = HEADS * HD
        per_layer = (q + 2 * kv + 2 * H) * rb(D) + D * rb(q) + D * rb(H) + 2 * D * 4
        n = V * D * 2 + D * 4 + L * per_layer - trim
        return b"RSTK" + struct.pack("<13I", 3, 0, D, L, V, 32, 0, H, HEADS, HEADS, HD, dtype_code, flags) + b"\0" * n
    for code in (3, 4):
        p = tmp_path / ("q%d.rstk" % code)
        p.write_bytes(body(code, 2))
        info = R.checkpoint_info(str(p))
        assert info["quantised_linears"] and not info["untied_head"] and info["dtype"] == code
        assert (info["cfg"].dim, info["cfg"].hidden, info["cfg"].heads, info["cfg"].hd) == (D, H, HEADS, HD)
        p.write_bytes(body(code, 2, trim=16))
        with pytest.raises(ValueError, match="unexpected EOF reading tensor"):
            R.checkpoint_info(str(p))
    bad = tmp_path / "bad.rstk"
    bad.write_bytes(body(3, 0))  # a quantised dtype code without the flag
    with pytest.raises(ValueError, match="invalid v3 header fields"):
        R.checkpoint_info(str(bad))
    bad.write_bytes(body(2, 2))  # the flag without a quantised dtype code
    with pytest.raises(ValueError, match="invalid v3 header fields"):
        R.checkpoint_info(str(bad))


def test_prompt_pass_exchange_protocol_never_reads_a_rewritten_buffer():
    """The tensor-parallel prompt pass exchanges partial sums through two alternating buffers per rank and one
    sequence number per (buffer, rank) that a rank posts to every peer (prefill.cuh: tp_pf_publish_kernel,
    tp_pf_reduce_kernel).  A model of that protocol under random interleavings of the ranks: a rank writes buffer
    (seq & 1) for all-reduce seq, posts seq, waits until every rank's number for that buffer is >= seq, then reads
    every rank's buffer - and must always find all-reduce seq's data there, never a later one's."""
    import random
    for trial in range(200):
        rng = random.Random(trial)
        world, nred = rng.choice([2, 3, 4, 8]), 7
        buf = [[None, None] for _ in range(world)]                          # buf[rank][b] = seq whose partial it holds
        flags = [[[0] * world for _ in range(2)] for _ in range(world)]      # flags[at_rank][b][from_rank]
        pc = [("write", 1)] * world                                         # per rank: next action and its all-reduce
        pending = [dict() for _ in range(world)]                            # reads still to do in the current reduce
        done = [0] * world
        while min(done) < nred:
            r = rng.randrange(world)
            if done[r] >= nred:
                continue
            act, seq = pc[r]
            b = seq & 1
            if act == "write":      # the GEMM's epilogue stores this rank's partial product
                buf[r][b] = seq
                pc[r] = ("post", seq)
            elif act == "post":     # one peer at a time, in any order relative to the other ranks
                todo = pending[r].setdefault("post", list(range(world)))
                p = todo.pop(rng.randrange(len(todo)))
                flags[p][b][r] = seq
                if not todo:
                    del pending[r]["post"]
                    pc[r] = ("wait", seq)
            elif act == "wait":     # proceeds only when every rank has posted seq (or later) for this buffer
                if all(f >= seq for f in flags[r][b]):
                    pending[r]["read"] = list(range(world))
                    pc[r] = ("read", seq)
            else:                   # reads the ranks' buffers one at a time
                todo = pending[r]["read"]
                p = todo.pop(rng.randrange(len(todo)))
                assert buf[p][b] == seq, (trial, world, r, p, seq, buf[p][b])
                if not todo:
                    del pending[r]["read"]
                    done[r] = seq
                    pc[r] = ("write", seq + 1)
