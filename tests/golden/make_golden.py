"""Regenerates the golden vectors under tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py

config1_greedy.npz — the tiny rustane LM (fp32, N(0, 0.02) synthetic weights from seed 0,
vocab 8192, dim 512, 8 layers, 8 heads x 64, SwiGLU hidden 1536, seq 512, untied head),
prompt [1, 2, 3, 4], 32 greedy steps through the oracle's naive_full_context path:
`tokens` [32] and `logits` [32, 8192] (the row each token was taken from), float32.
small_kv.npz — a 2-layer bf16 model with the fp16 KV cache the library gives it: per-step hidden states, block top-k and block stats
from the oracle's KV-cached path, so the CUDA head kernels have fixed expectations.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import pyoracle as O  # noqa: E402


def config1():
    cfg = O.make_config(dim=512, hidden=1536, heads=8, hd=64, seq=512, nlayers=8, vocab=8192, untied=1)
    m = O.Model.synth(cfg, 0)
    toks, trace, mode = m.generate([1, 2, 3, 4], 32, backend=O.BACKEND_NAIVE, trace=True)
    assert mode == O.MODE_NAIVE
    np.savez_compressed(os.path.join(HERE, "config1_greedy.npz"), tokens=toks[0], logits=trace,
                        prompt=np.array([1, 2, 3, 4], dtype=np.uint32))


def small_kv():
    cfg = O.make_config(dim=256, hidden=640, heads=2, hd=128, seq=64, nlayers=2, vocab=1500, dtype=O.BF16)
    m = O.Model.synth(cfg, 5)
    c = O.Cache(m, kv_round=1)
    hidden = np.stack([c.decode_token_from_id(t) for t in (1, 2, 3)])
    tv, ti = c.decode_token_topk_from_id(9, 4)
    mx, sm = c.decode_token_block_stats_from_id(11, 1.25)
    blk = c.materialize_current_logits_block(5)
    nxt = c.decode_token_argmax_from_id(7)
    np.savez_compressed(os.path.join(HERE, "small_kv.npz"), hidden=hidden, topk_vals=tv, topk_idxs=ti, maxes=mx,
                        sums=sm, block5=blk, argmax=np.uint32(nxt))


if __name__ == "__main__":
    config1()
    small_kv()
    print("golden vectors written to", HERE)
