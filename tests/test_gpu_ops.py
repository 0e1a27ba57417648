"""Kernel-level numerics: the split-K flash-decode attention kernel against a plain fp32
softmax-attention reference (the math of sdpa_causal, metal-decode/src/lib.rs:1426-1489)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def reference_attention(q, k, v, heads, kv_heads, hd):
    out = np.zeros(heads * hd, dtype=np.float32)
    for h in range(heads):
        kvh = h // (heads // kv_heads)
        ks, vs = k[:, kvh * hd:(kvh + 1) * hd], v[:, kvh * hd:(kvh + 1) * hd]
        s = (ks @ q[h * hd:(h + 1) * hd]) * np.float32(1.0 / np.sqrt(hd))
        p = np.exp(s - s.max())
        out[h * hd:(h + 1) * hd] = (p / p.sum()) @ vs
    return out


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("heads,kv_heads,hd,attn_len,nsplit", [
    (2, 2, 128, 1, 0), (4, 4, 64, 63, 0), (4, 2, 128, 64, 0), (8, 8, 128, 65, 0), (32, 32, 128, 1280, 0),
    (8, 8, 64, 2048, 32), (3, 1, 128, 700, 5), (6, 6, 128, 4096, 32),
])
def test_flash_decode_matches_fp32_reference(dtype, heads, kv_heads, hd, attn_len, nsplit):
    from rustane_b200 import ops
    rng = np.random.default_rng(attn_len + heads)
    q = rng.standard_normal(heads * hd).astype(np.float32)
    k = ops.to_storage(rng.standard_normal((attn_len, kv_heads * hd)).astype(np.float32), dtype)
    v = ops.to_storage(rng.standard_normal((attn_len, kv_heads * hd)).astype(np.float32), dtype)
    got = ops.flash_decode(q, k, v, heads, kv_heads, hd, dtype=dtype, nsplit=nsplit)
    ref = reference_attention(q, ops.from_storage(k, dtype), ops.from_storage(v, dtype), heads, kv_heads, hd)
    np.testing.assert_allclose(got, ref, atol=2e-5, rtol=1e-4)  # fp32 math on identical rounded inputs
