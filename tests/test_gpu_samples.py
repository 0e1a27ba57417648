"""`--samples N` sharing a prompt: the batched multi-sample decode against the sequential loops.

Each sample of the batched call must reproduce what cd_decode_steps_{greedy,topk,fullvocab}
produces for that sample alone from the same prompt cache, first token and LCG state
(inference.rs:255-297 runs the samples one after the other).  The batched linears round
their inputs to hi + lo 16-bit pairs, so logits differ from the sequential GEMV path by
~1e-4; a draw can only differ where the inverse-CDF threshold falls inside that margin: greedy
ids are compared exactly, sampled ids up to the first such flip (rare: at least 90 % of all
(sample, step) pairs must agree and every sample must start identically).
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


def _model(R, O, dims, dtype, kw, page_tokens, max_samples, use_graph=False):
    oc = oracle_cfg(O, *dims, dtype=dtype, **kw)
    return oc, R.Model.synthetic(gpu_cfg(R, oc), 11, untied_head=bool(oc.untied), dtype=dtype, page_tokens=page_tokens,
                                 max_samples=max_samples, use_graph=use_graph)


@pytest.mark.parametrize("dims,dtype,kw,nprompt,page_tokens", CASES)
@pytest.mark.parametrize("mode", ["greedy", "topk", "fullvocab"])
def test_samples_match_sequential_loops(R, oracle, dims, dtype, kw, nprompt, page_tokens, mode):
    ns, nsteps = 5, 20
    oc, gm = _model(R, oracle, dims, dtype, kw, page_tokens, ns, use_graph=(mode != "fullvocab"))  # captured steps and plain launches
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
    if mode == "greedy":
        assert got.tolist() == want
    else:
        # a draw may flip where its inverse-CDF threshold falls within the ~1e-4 distance of the two
        # arithmetic orders; from there the two continuations differ.  Every sample must start
        # identically and nearly all (sample, step) pairs must precede any such flip.
        agree = 0
        for s in range(ns):
            n = 0
            while n < nsteps and int(got[s][n]) == want[s][n]:
                n += 1
            assert n >= 5, (s, n)
            agree += n
            if n == nsteps:
                assert int(rng[s]) == want_rng[s]
        assert agree >= 0.9 * ns * nsteps, agree
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


@pytest.mark.parametrize("mode", ["greedy", "topk8", "fullvocab"])
def test_session_runs_samples_together_and_matches_oracle(R, oracle, mode, monkeypatch):
    """InferenceSession.generate with samples > 1 on a model that has pages for them: same ids as the
    oracle's run_cached_sample loop and as the one-after-the-other order (CD_SAMPLES=sequential)."""
    O = oracle
    dims = (256, 640, 2, 128, 96, 2, 1500)
    oc = oracle_cfg(O, *dims, dtype="bf16")
    om = O.Model.synth(oc, 21)
    gm = R.Model.synthetic(gpu_cfg(R, oc), 21, dtype="bf16", max_samples=3)
    t, k = {"greedy": (0.0, 0), "topk8": (0.8, 8), "fullvocab": (1.0, 0)}[mode]
    prompt = [5, 6, 7, 8, 9]
    ref, ref_mode = om.generate(prompt, 20, backend=O.BACKEND_KV, temperature=t, top_k=k, samples=3, seed=11, kv_round=1)
    sess = R.InferenceSession(gm, prompt)
    req = R.GenerationRequest("cuda", 20, t, k, 3, 11)
    out = sess.generate(req)
    assert gm.len() == len(prompt)                      # the samples advanced together: the cache is left at the prompt
    for s in range(3):
        assert out.results[s].sampled == ref[s].tolist()
        assert out.results[s].generated == prompt + ref[s].tolist()
        assert out.results[s].seed == 11 + s
    monkeypatch.setenv("CD_SAMPLES", "sequential")
    seq = sess.generate(req)
    assert gm.len() == len(prompt) + 19
    assert [r.sampled for r in seq.results] == [r.sampled for r in out.results]


def test_captured_step_graphs_follow_the_prompt_length(R, oracle):
    """The number of shared prompt tokens is a launch argument of the multi-sample attention kernel, so a
    captured step must not outlive the prompt length it was captured for: a longer prompt first, then
    a shorter one whose steps cross the first one's page boundary, on one handle with graphs on, must
    both equal the sequential loops."""
    dims, dtype = (256, 640, 2, 128, 512, 2, 1500), "bf16"
    oc, gm = _model(R, oracle, dims, dtype, {}, 64, 4, use_graph=True)
    long_prompt = oracle.synth_prompt(6, oc.vocab, 270)   # shares 256 prompt tokens
    short_prompt = long_prompt[:230]                      # shares 192: its samples' own tokens start below 256
    for prompt, nsteps in ((long_prompt, 12), (short_prompt, 40)):
        gm.set_len(0)
        logits = gm.prefill(prompt)
        first = [int(i) for i in np.argsort(-logits)[:4]]
        want = []
        for s in range(4):
            gm.set_len(len(prompt))
            want.append(gm.decode_steps_greedy(first[s], nsteps).tolist())
        gm.set_len(len(prompt))
        got, _ = gm.decode_steps_samples(first, nsteps, mode="greedy")
        # a stale count of shared tokens would feed sample 0's keys to the other samples from their first own token on
        assert [g[:12] for g in got.tolist()] == [w[:12] for w in want], len(prompt)
        same = sum(int(a == b) for g, w in zip(got.tolist(), want) for a, b in zip(g, w))
        assert same >= 0.9 * 4 * nsteps, (len(prompt), same)
