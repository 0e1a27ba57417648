"""Quantised linears (FP8-E4M3 per output channel, INT4 group-32) against the oracle.

The reference has no quantised path, so the rule itself is builder-defined; what is pinned is
that the CUDA library and the oracle quantise identically and that decoding with the
quantised rows equals the oracle run on the dequantised values.  Both sides then hold
the same numbers, so the stated bound is the one of the 16-bit formats: logits within 1e-3
max-abs (summation order plus one-ulp flips of bf16 KV values), greedy ids identical.
"""
import numpy as np
import pytest

from helpers import gpu_cfg, oracle_cfg, top2_gap

pytestmark = pytest.mark.gpu

QUANT_TOL = 1e-3
MODES = {"fp8": 3, "int4": 4}

SHAPES = [
    ((256, 640, 2, 128, 64, 2, 320), {}),                      # the reference's small decode shape
    ((512, 1536, 8, 64, 96, 3, 8192), dict(untied=1)),         # configuration-1 widths, untied head
    ((384, 992, 3, 128, 80, 2, 1000), dict(page_tokens=16)),   # K = 992 = 31 groups: partial chunk rows
    ((256, 512, 4, 64, 80, 2, 512), dict(kv_heads=2, activation=1)),
]


def _pair(R, O, dims, dtype, seed=9, **kw):
    opts = {k: kw.pop(k) for k in ("use_graph", "page_tokens") if k in kw}
    oc = oracle_cfg(O, *dims, dtype="f32", **kw)
    om = O.Model.synth_quant(oc, seed, MODES[dtype])
    gm = R.Model.synthetic(gpu_cfg(R, oc), seed, untied_head=bool(oc.untied), dtype=dtype, activation=oc.activation, **opts)
    return oc, om, gm


@pytest.mark.parametrize("dims,kw", SHAPES)
@pytest.mark.parametrize("dtype", ["fp8", "int4"])
def test_quantised_decode_matches_oracle_on_dequantised_weights(R, oracle, dims, kw, dtype):
    oc, om, gm = _pair(R, oracle, dims, dtype, **dict(kw))
    cache = oracle.Cache(om, kv_round=1)
    tok, worst = 3, 0.0
    for _ in range(16):
        a, b = gm.decode_token_logits_from_id(tok), cache.decode_logits(tok)
        worst = max(worst, float(np.abs(a - b).max()))
        tok = int(np.argmax(b))
    assert worst < QUANT_TOL, worst


@pytest.mark.parametrize("dtype", ["fp8", "int4"])
def test_quantised_greedy_loop_and_host_weights(R, oracle, dtype):
    """Greedy ids of the on-device loop equal the oracle's; a model built from host fp32
    tensors (relayout + quantise at construction) equals the self-generated one bit for bit."""
    dims = (512, 1536, 8, 64, 128, 4, 8192)
    oc, om, gm = _pair(R, oracle, dims, dtype, use_graph=True)
    prompt = oracle.synth_prompt(1, oc.vocab, 8)
    cache = oracle.Cache(om, kv_round=1)
    for t in prompt[:-1]:
        cache.decode_token_from_id(int(t))
    ref = cache.decode_logits(int(prompt[-1]))
    got = gm.prefill(prompt)
    assert np.abs(got - ref).max() < QUANT_TOL
    assert top2_gap(ref) > QUANT_TOL
    tok = int(np.argmax(ref))
    gpu_ids = gm.decode_steps_greedy(tok, 24).tolist()
    ref_ids, cur = [], tok
    for _ in range(24):
        cur = cache.decode_token_argmax_from_id(cur)
        ref_ids.append(cur)
    assert gpu_ids == ref_ids
    # host-tensor construction: unquantised fp32 tensors in, quantised at construction
    plain = oracle.Model.synth(oracle_cfg(oracle, *dims, dtype="f32"), 9)
    layers = [{n: plain.tensor(getattr(oracle, "T_" + n.upper()), l) for n in
               ("wq", "wk", "wv", "wo", "w1", "w3", "w2", "gamma1", "gamma2")} for l in range(oc.nlayers)]
    head = {"gamma_final": plain.tensor(oracle.T_GAMMA_FINAL), "embed": plain.tensor(oracle.T_EMBED)}
    gm2 = R.Model.new(gpu_cfg(R, oc), layers, head, dtype=dtype)
    gm3 = R.Model.synthetic(gpu_cfg(R, oc), 9, dtype=dtype)
    for t in (1, 7, 300):
        assert np.array_equal(gm2.decode_token_logits_from_id(t), gm3.decode_token_logits_from_id(t))


def test_quantised_rejections(R):
    cfg = R.Config(264, 640, 2, 128, 64, 2, 320)  # dim not a multiple of 16 / 32
    for dtype in ("fp8", "int4"):
        with pytest.raises(Exception):
            R.Model.synthetic(cfg, 1, dtype=dtype)


@pytest.mark.parametrize("dims,n", [((512, 1536, 8, 64, 256, 3, 8192), 150), ((256, 640, 2, 128, 128, 2, 320), 40)])
def test_fp8_prompt_pass_on_the_tensor_cores(R, oracle, dims, n, monkeypatch):
    """FP8 models run prompts of 8+ tokens through the tensor-core pass (e4m3 values widened exactly to
    bf16 per layer, row scales on the GEMM's output columns); INT4 models keep the per-token path.
    Same bound as the bf16 prompt pass: 2e-3 against the oracle on the dequantised weights."""
    oc, om, gm = _pair(R, oracle, dims, "fp8")
    prompt = oracle.synth_prompt(2, oc.vocab, n)
    cache = oracle.Cache(om, kv_round=1)
    for t in prompt[:-1]:
        cache.decode_token_from_id(int(t))
    ref = cache.decode_logits(int(prompt[-1]))
    launches = gm.kernel_launches()
    got = gm.prefill(prompt)
    assert gm.kernel_launches() - launches < 20 * oc.nlayers + 8      # the batched pass, not n single-token steps
    assert float(np.abs(got - ref).max()) < 2e-3
    tok = int(np.argmax(ref))
    for _ in range(4):  # the K / V it wrote, through ordinary decode steps
        a, b = gm.decode_token_logits_from_id(tok), cache.decode_logits(tok)
        assert float(np.abs(a - b).max()) < 2e-3
        tok = int(np.argmax(b))
    monkeypatch.setenv("CD_PREFILL", "token")
    gm.set_len(0)
    assert float(np.abs(gm.prefill(prompt) - ref).max()) < QUANT_TOL


def _row_bytes(dtype, k):
    return k + 16 if dtype == "fp8" else (k // 2 + k // 16 + 15) // 16 * 16


@pytest.mark.parametrize("dtype", ["fp8", "int4"])
def test_stored_quantised_checkpoint_loads_bit_identically(R, tmp_path, dtype):
    """A plain RSTK file converted once (cd_convert_checkpoint) loads, without conversion, to the very rows and logits
    that quantising the plain file at load produces; a tensor-parallel rank takes its shard of the stored rows (whole-row
    FP8 scales, its own INT4 groups) exactly as the load-time quantiser cuts it."""
    cfg = R.Config(256, 640, 4, 64, 64, 2, 320, kv_heads=2)
    plain, quant = str(tmp_path / "plain.rstk"), str(tmp_path / ("q_%s.rstk" % dtype))
    R.write_synthetic_checkpoint(plain, cfg, dtype="bf16", untied_head=True, seed=6)
    R.convert_checkpoint(plain, quant, dtype)
    info = R.checkpoint_info(quant)
    assert info["quantised_linears"] and info["untied_head"] and info["dtype"] == MODES[dtype] and info["version"] == 3
    a = R.Model.from_checkpoint(plain, dtype=dtype)   # quantised at load
    b = R.Model.from_checkpoint(quant)                # stored rows
    widths = [(cfg.q_dim, cfg.dim), (cfg.kv_dim, cfg.dim), (cfg.kv_dim, cfg.dim), (cfg.dim, cfg.q_dim),
              (cfg.hidden, cfg.dim), (cfg.hidden, cfg.dim), (cfg.dim, cfg.hidden)]
    for layer in range(cfg.nlayers):
        for which, (rows, k) in enumerate(widths):
            n = rows * _row_bytes(dtype, k)
            assert np.array_equal(a.linear_rows(layer, which, n), b.linear_rows(layer, which, n)), (layer, which)
    tok = 5
    for _ in range(6):
        la, lb = a.decode_token_logits_from_id(tok), b.decode_token_logits_from_id(tok)
        assert np.array_equal(la, lb)
        tok = int(np.argmax(la))
    with pytest.raises(R.CudaDecodeError, match="loads in its own format only"):
        R.Model.from_checkpoint(quant, dtype="bf16")
    # a live quantised model writes the same file
    again = str(tmp_path / "again.rstk")
    a.save_quantised(again)
    assert open(again, "rb").read() == open(quant, "rb").read()
    a.close(); b.close()
    # rank 1 of 2: shards of the stored rows against shards quantised at load (construction only; nothing is decoded)
    sa = R.Model.from_checkpoint(plain, dtype=dtype, tp_rank=1, tp_world=2)
    sb = R.Model.from_checkpoint(quant, tp_rank=1, tp_world=2)
    half = [(cfg.q_dim // 2, cfg.dim), (cfg.kv_dim // 2, cfg.dim), (cfg.kv_dim // 2, cfg.dim), (cfg.dim, cfg.q_dim // 2),
            (cfg.hidden // 2, cfg.dim), (cfg.hidden // 2, cfg.dim), (cfg.dim, cfg.hidden // 2)]
    for which, (rows, k) in enumerate(half):
        n = rows * _row_bytes(dtype, k)
        assert np.array_equal(sa.linear_rows(1, which, n), sb.linear_rows(1, which, n)), which
    sa.close(); sb.close()
