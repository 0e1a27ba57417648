"""Shared builders for the parity tests: the same model on the oracle and on the GPU."""
import numpy as np

DT = {"f32": 0, "f16": 1, "bf16": 2}


def oracle_cfg(O, dim, hidden, heads, hd, seq, nlayers, vocab, kv_heads=None, activation=0, dtype="f32", untied=0):
    return O.make_config(dim=dim, hidden=hidden, heads=heads, hd=hd, seq=seq, nlayers=nlayers, vocab=vocab,
                         kv_heads=kv_heads, activation=activation, dtype=DT[dtype], untied=untied)


def gpu_cfg(R, oc):
    return R.Config(oc.dim, oc.hidden, oc.heads, oc.hd, oc.seq, oc.nlayers, oc.vocab, kv_heads=oc.kv_heads)


def gpu_model_from_oracle(R, O, om, dtype, **opts):
    """Build the CUDA model through Model::new from the oracle's (already rounded) tensors."""
    oc = om.cfg
    layers = []
    for l in range(oc.nlayers):
        layers.append({name: om.tensor(getattr(O, "T_" + name.upper()), l)
                       for name in ("wq", "wk", "wv", "wo", "w1", "w3", "w2", "gamma1", "gamma2")})
    head = {"gamma_final": om.tensor(O.T_GAMMA_FINAL), "embed": om.tensor(O.T_EMBED)}
    if oc.untied:
        head["lm_head"] = om.tensor(O.T_LM_HEAD)
    return R.Model.new(gpu_cfg(R, oc), layers, head, dtype=dtype, activation=oc.activation, **opts)


def top2_gap(logits):
    s = np.sort(np.asarray(logits))
    return float(s[-1] - s[-2])
