"""Pins of the CPU oracle against everything the reference's own tests hold for this path.

The reference has no golden-vector files; what it pins are small known answers
(cpu/rmsnorm.rs:245-277, cpu/embedding.rs:51-62), the backend policy table
(inference.rs:946-974), the checkpoint round trip (checkpoint.rs:254-313) and the
self-consistency contracts of tests/auto_kv_decode.rs:67-215 (cached == naive on
ModelWeights::random).  Each is replayed here on the oracle.
"""
import ctypes as C
import struct

import numpy as np
import pytest

from helpers import oracle_cfg


def test_rmsnorm_unit_gamma(oracle):  # cpu/rmsnorm.rs:245-256
    x = np.array([3.0, 4.0], dtype=np.float32)
    g = np.ones(2, dtype=np.float32)
    out = np.zeros(2, dtype=np.float32)
    inv = oracle.lib.orc_rmsnorm(oracle._f32(x), oracle._f32(g), oracle._f32(out), 2)
    rms = np.sqrt(np.float32(12.5) + np.float32(1e-5))
    assert abs(inv - 1.0 / rms) < 1e-5
    assert abs(out[0] - 3.0 / rms) < 1e-5 and abs(out[1] - 4.0 / rms) < 1e-5


def test_rmsnorm_with_gamma(oracle):  # cpu/rmsnorm.rs:258-277
    x = np.array([1, 2, 3, 4], dtype=np.float32)
    g = np.full(4, 0.5, dtype=np.float32)
    out = np.zeros(4, dtype=np.float32)
    inv = oracle.lib.orc_rmsnorm(oracle._f32(x), oracle._f32(g), oracle._f32(out), 4)
    expect = 1.0 / np.sqrt(7.5 + 1e-5)
    assert abs(inv - expect) < 1e-5
    np.testing.assert_allclose(out, x * expect * 0.5, atol=1e-5)


def test_embedding_lookup(oracle):  # cpu/embedding.rs:51-62
    table = np.array([1, 2, 3, 4, 5, 6], dtype=np.float32)
    ids = np.array([2, 0, 1], dtype=np.uint32)
    out = np.zeros(6, dtype=np.float32)
    oracle.lib.orc_embedding(oracle._f32(table), 2, oracle._u32(ids), 3, oracle._f32(out))
    assert out.tolist() == [5, 6, 1, 2, 3, 4]


def test_lcg_matches_closed_form(oracle):  # inference.rs:759-768
    s = C.c_uint64(7)
    py = 7
    for _ in range(5):
        py = (py * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        f = oracle.lib.orc_next_f32(C.byref(s))
        assert s.value == py
        assert f == np.float32(py >> 40) / np.float32(1 << 24)


def test_reference_random_vec(oracle):  # layer.rs:806-817
    n = 5
    out = np.zeros(n, dtype=np.float32)
    oracle.lib.orc_reference_random_vec(oracle._f32(out), n, 0.5)
    seed = 42 + n
    for i in range(n):
        seed = (seed * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        r = np.float32(np.float32(seed >> 32) / np.float32(0xFFFFFFFF)) * np.float32(2.0) - np.float32(1.0)
        assert out[i] == np.float32(r * np.float32(0.5))


def _tiny(oracle, vocab=8192):  # inference.rs:929-944
    return oracle_cfg(oracle, 256, 640, 2, 128, 64, 2, vocab)


def test_policy_table(oracle):  # inference.rs:946-974
    O = oracle
    assert O.select_decode_mode(_tiny(O), O.BACKEND_AUTO, 4, 8) == (O.MODE_NAIVE, None, "model_param_count_lt_threshold")
    gpt1024 = oracle_cfg(O, 1024, 2816, 8, 128, 512, 8, 8192)  # >= 20M parameters, as ModelConfig::gpt_1024
    assert O.lib.orc_param_count(C.byref(gpt1024)) >= 20_000_000
    assert O.select_decode_mode(gpt1024, O.BACKEND_AUTO, 4, 32) == (O.MODE_KV, None, "model_param_count_ge_threshold")
    assert O.select_decode_mode(gpt1024, O.BACKEND_KV, 500, 20) == (O.MODE_NAIVE, "requested_length_exceeds_cfg_seq", None)
    assert O.select_decode_mode(gpt1024, O.BACKEND_KV, 4, 1) == (O.MODE_NAIVE, "single_step_prefers_naive", None)
    assert O.select_decode_mode(gpt1024, O.BACKEND_AUTO, 4, 0)[0] == O.MODE_PREFILL_ONLY
    assert O.select_decode_mode(gpt1024, O.BACKEND_AUTO, 500, 20) == (
        O.MODE_NAIVE, "requested_length_exceeds_cfg_seq", "window_not_metal_eligible")
    assert O.select_decode_mode(gpt1024, O.BACKEND_NAIVE, 4, 32) == (O.MODE_NAIVE, None, None)


def test_merge_topk_rules(oracle):  # decode.rs:218-253
    vals = np.array([1.0, 3.0, 3.0, -np.inf, 2.0, np.nan], dtype=np.float32)
    idxs = np.array([5, 9, 4, 1, 0xFFFFFFFF, 2], dtype=np.uint32)
    v, i = oracle.merge_topk(vals, idxs, 4)
    assert i.tolist() == [4, 9, 5]  # tie to the lower index; sentinel / non-finite dropped
    assert v.tolist() == [3.0, 3.0, 1.0]


def test_checkpoint_v2_roundtrip(oracle, tmp_path):  # checkpoint.rs:254-313
    dim, hidden, nlayers, vocab, seq = 128, 256, 2, 16, 8
    rng = np.random.default_rng(0)
    body = b""
    tensors = []

    def put(n):
        nonlocal body
        a = rng.standard_normal(n).astype(np.float32)
        tensors.append(a)
        body += a.tobytes()

    put(vocab * dim)
    put(dim)
    for _ in range(nlayers):
        for n in (dim * dim, dim * dim, dim * dim, dim * dim, dim * hidden, dim * hidden, dim * hidden, dim, dim):
            put(n)
    p = tmp_path / "ck.bin"
    p.write_bytes(b"RSTK" + struct.pack("<7I", 2, 7, dim, nlayers, vocab, seq, 1) + body)
    m = oracle.Model.load(str(p))
    assert (m.cfg.dim, m.cfg.hidden, m.cfg.heads, m.cfg.hd, m.cfg.seq, m.cfg.nlayers, m.cfg.vocab) == (
        dim, hidden, 1, 128, seq, nlayers, vocab)
    assert m.cfg.activation == oracle.ACT_LEAKY_RELU_SQ
    np.testing.assert_array_equal(m.tensor(oracle.T_EMBED), tensors[0])
    np.testing.assert_array_equal(m.tensor(oracle.T_W2, 1), tensors[2 + 9 + 6])
    # error messages of checkpoint.rs:30-155
    for blob, msg in [(b"XXXX" + b"\0" * 28, "invalid checkpoint magic"),
                      (b"RSTK" + struct.pack("<6I", 9, 0, dim, 1, 1, 1), "unsupported checkpoint version 9"),
                      (b"RSTK" + struct.pack("<7I", 2, 0, 100, 1, 1, 1, 0) + b"\0" * 4, "not divisible by 128"),
                      (b"RSTK" + struct.pack("<7I", 2, 0, dim, nlayers, vocab, seq, 0) + body + b"\0" * 4,
                       "integer hidden size")]:
        q = tmp_path / "bad.bin"
        q.write_bytes(blob)
        with pytest.raises(ValueError, match=msg):
            oracle.Model.load(str(q))


def _argmax_last(x):
    return len(x) - 1 - int(np.argmax(x[::-1]))


def test_kv_decode_matches_naive_on_reference_random(oracle):  # auto_kv_decode.rs:67-134
    O = oracle
    cfg = oracle_cfg(O, 256, 640, 2, 128, 64, 2, 64)
    m = O.Model.reference_random(cfg)
    generated = [1, 2, 3]
    logits, kcf, vcf = m.forward_logits(generated, want_kv=True)
    cache = O.Cache(m)
    cache.set_len(len(generated))
    for l in range(cfg.nlayers):
        cache.seed_layer_cache_from_channel_first(l, len(generated), kcf[l], vcf[l])
    nxt = _argmax_last(logits[0])
    generated.append(nxt)
    cache2 = O.Cache(m)
    cache2.set_len(3)
    for l in range(cfg.nlayers):
        cache2.seed_layer_cache_from_channel_first(l, 3, kcf[l], vcf[l])
    for _ in range(3):
        cached = _argmax_last(cache.decode_logits(nxt))
        gpu_style = cache2.decode_token_argmax_from_id(nxt)
        naive = _argmax_last(m.forward_logits(generated)[0])
        assert cached == naive == gpu_style
        nxt = cached
        generated.append(nxt)


def test_topk_and_block_stats_match_naive(oracle):  # auto_kv_decode.rs:136-215
    O = oracle
    cfg = oracle_cfg(O, 256, 640, 2, 128, 64, 2, 320)
    for m in (O.Model.reference_random(cfg), O.Model.synth(cfg, 5)):
        generated = [1, 2, 3, 4]
        logits, kcf, vcf = m.forward_logits(generated, want_kv=True)
        nxt = _argmax_last(logits[0])
        naive = m.forward_logits(generated + [nxt])[0]

        def seeded():
            c = O.Cache(m)
            c.set_len(4)
            for l in range(cfg.nlayers):
                c.seed_layer_cache_from_channel_first(l, 4, kcf[l], vcf[l])
            return c

        vals, idxs = seeded().decode_token_topk_from_id(nxt, 4)
        mv, mi = O.merge_topk(vals, idxs, 4)
        order = sorted(range(cfg.vocab), key=lambda i: (-naive[i], i))[:4]
        assert mi.tolist() == order
        np.testing.assert_allclose(mv, naive[order], atol=1e-4)

        c = seeded()
        t = 0.8
        mx, sm = c.decode_token_block_stats_from_id(nxt, 1.0 / t)
        for b in range(len(mx)):
            z = naive[b * 256:(b + 1) * 256] / np.float32(t)
            assert abs(mx[b] - z.max()) < 1e-4
            assert abs(sm[b] - np.exp(z - z.max()).sum()) < 1e-3
        np.testing.assert_allclose(c.materialize_current_logits_block(1), naive[256:320], atol=1e-4)


def test_truncated_forward_equals_padded_forward(oracle):
    """Causality: the first npos rows do not depend on the reference's zero padding to cfg.seq."""
    O = oracle
    cfg = oracle_cfg(O, 128, 256, 2, 64, 16, 2, 96, untied=1)
    m = O.Model.synth(cfg, 3)
    ids = [5, 9, 2, 7]
    short = m.forward_logits(ids, rows=[3])
    padded = m.forward_logits(ids + [0] * 12, rows=[3])
    np.testing.assert_array_equal(short, padded)


def test_session_contracts_on_oracle(oracle):  # inference.rs:976-1033
    O = oracle
    cfg = oracle_cfg(O, 256, 640, 2, 128, 64, 2, 8192)
    m = O.Model.synth(cfg, 9)
    a, _ = m.generate([1, 2, 3, 4], 8, backend=O.BACKEND_KV, temperature=0.8, top_k=4, samples=2, seed=7)
    b, _ = m.generate([1, 2, 3, 4], 8, backend=O.BACKEND_KV, temperature=0.8, top_k=4, samples=2, seed=7)
    np.testing.assert_array_equal(a, b)
    ext, _ = m.generate([1, 2, 3], 6, backend=O.BACKEND_KV, temperature=0.8, top_k=4, samples=2, seed=17, suffix=[4, 5])
    fresh, _ = m.generate([1, 2, 3, 4, 5], 6, backend=O.BACKEND_KV, temperature=0.8, top_k=4, samples=2, seed=17)
    np.testing.assert_array_equal(ext, fresh)


@pytest.mark.parametrize("in_major", [0, 1])
def test_quantisers_against_independent_restatement(oracle, in_major):
    """FP8-E4M3 per-row and INT4 group-32 have no reference definition; the oracle's quantiser is
    checked against torch's float8_e4m3fn cast and a vectorised restatement of the INT4 rule."""
    import torch
    rs = np.random.RandomState(3)
    w = (rs.randn(48, 320) * 0.02).astype(np.float32)
    w[5] = 0.0                      # all-zero row / groups
    w[7, :32] *= 1e-6               # a group far below the row maximum (FP8 denormals)
    t = torch.from_numpy(w)

    def run(mode):
        a = np.ascontiguousarray(w.T if in_major else w).copy()
        oracle.lib.orc_quant_dequant(oracle._f32(a), 320, 48, in_major, mode)
        return a.T if in_major else a

    amax = t.abs().amax(dim=1, keepdim=True)
    sc = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    ref8 = ((t / sc).to(torch.float8_e4m3fn).float() * sc).numpy()
    assert np.array_equal(run(oracle.QUANT_FP8), ref8)

    g = t.view(48, 10, 32)
    s = (g.abs().amax(dim=2, keepdim=True) / 7.0).half().float()
    q = torch.where(s > 0, torch.clamp(torch.round(g / torch.where(s > 0, s, torch.ones_like(s))), -8, 7), torch.zeros_like(g))
    ref4 = (q * s).view(48, 320).numpy()
    assert np.array_equal(run(oracle.QUANT_INT4), ref4)
