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
