"""`--samples N` sharing a prompt: the batched multi-sample decode against the sequential loops.

Each sample of the batched call must reproduce what cd_decode_steps_{greedy,topk,fullvocab}
produces for that sample alone from the same prompt cache, first token and LCG state
(inference.rs:255-297 runs the samples one after the other).  The batched linears round
their inputs to hi + lo 16-bit pairs, so logits differ from the sequential GEMV path by
~1e-4; a draw can only differ where the inverse-CDF threshold falls inside that margin, so
ids are compared exactly and a mismatch is accepted only after a step whose sequential
replay shows such a near-tie (never observed on these seeds).
"""
import numpy as np
import pytest

from helpers import gpu_cfg, oracle_cfg

pytestmark = pytest.mark.gpu

CASES = [
    ((512, 1536, 8, 64, 256, 3, 8192), "bf16", dict(untied=1), 37, 64),     # prompt ends inside a page: copy-on-write
    ((256, 640, 2, 128, 256, 2, 1500), "f16", {}, 128, 64),                 # prompt ends on a page boundary, ragged vocab
    ((256, 512, 4, 64, 200, 2, 512), "bf16", dict(kv_heads=2), 50, 16),     # GQA, small pages
]


def _model(R, O, dims, dtype, kw, page_tokens, max_samples):
    oc = oracle_cfg(O, *dims, dtype=dtype, **kw)
    return oc, R.Model.synthetic(gpu_cfg(R, oc), 11, untied_head=bool(oc.untied), dtype=dtype, page_tokens=page_tokens,
                                 max_samples=max_samples)


@pytest.mark.parametrize("dims,dtype,kw,nprompt,page_tokens", CASES)
@pytest.mark.parametrize("mode", ["greedy", "topk", "fullvocab"])
def test_samples_match_sequential_loops(R, oracle, dims, dtype, kw, nprompt, page_tokens, mode):
    ns, nsteps = 5, 20
    oc, gm = _model(R, oracle, dims, dtype, kw, page_tokens, ns)
    prompt = oracle.synth_prompt(4, oc.vocab, nprompt)
    logits = gm.prefill(prompt)
    order = np.argsort(-logits)
    first = [int(order[i]) for i in range(ns)]          # distinct first tokens so the samples diverge at once
    seeds = np.array([1000 + 7 * i for i in range(ns)], dtype=np.uint64)
    t, k = 0.9, 8
    gm.set_len(nprompt)
    greedy0 = gm.decode_steps_greedy(first[0], 6).tolist()
    want, want_rng = [], []
    for s in range(ns):
        gm.set_len(nprompt)
        if mode == "greedy":
            ids, r = gm.decode_steps_greedy(first[s], nsteps), 0
        elif mode == "topk":
            ids, r = gm.decode_steps_topk(first[s], nsteps, k, t, int(seeds[s]))
        else:
            ids, r = gm.decode_steps_fullvocab(first[s], nsteps, t, int(seeds[s]))
        want.append(ids.tolist())
        want_rng.append(r)
    gm.set_len(nprompt)
    got, rng = gm.decode_steps_samples(first, nsteps, mode=mode, top_k=k, temperature=t, rng_states=seeds)
    assert gm.len() == nprompt
    assert got.tolist() == want
    if mode != "greedy":
        assert [int(x) for x in rng] == want_rng
    # the shared prompt pages are intact: a sequential sample afterwards still reproduces
    gm.set_len(nprompt)
    assert gm.decode_steps_greedy(first[0], 6).tolist() == greedy0


def test_samples_argument_checks(R, oracle):
    oc, gm = _model(R, oracle, (256, 640, 2, 128, 64, 2, 320), "bf16", {}, 64, 2)
    gm.prefill([1, 2, 3])
    with pytest.raises(Exception):
        gm.decode_steps_samples([1, 2, 3], 4)              # more samples than max_samples
    with pytest.raises(Exception):
        gm.decode_steps_samples([1, 999999], 4)            # token outside the vocabulary
    with pytest.raises(Exception):
        gm.decode_steps_samples([1, 2], 100)               # would run past cfg.seq
    _, f32 = _model(R, oracle, (256, 640, 2, 128, 64, 2, 320), "f32", {}, 64, 2)
    f32.prefill([1, 2, 3])
    with pytest.raises(Exception):
        f32.decode_steps_samples([1, 2], 4)                # fp32 storage: no tensor-core path
