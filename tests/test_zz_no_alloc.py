"""cd_flash_decode_static — the attention kernel for callers that cannot allocate device
memory (an engine that owns all of HBM through its own arena, a latency-critical thread that
may not take cudaMalloc's device-wide synchronisation, a plug-in host that forbids driver
allocations after start-up).  Its scratch is a fixed array inside the library, so this test
hands it device buffers it allocated itself (through torch, as such a caller would through its
arena) and checks the result against the allocating entry point cd_flash_decode and against a
plain fp32 numpy attention, twice in a row: the second call finds the previous call's
leftovers in the shared scratch.

Collected last on purpose (file name), so that a run that stops at the first failure has
already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _pack_pages(k, v, kv_heads, hd, page_tokens=64):
    """[attn_len, kv_heads*hd] rows -> [pages][2][kv_heads][page_tokens][hd] (zero padded)."""
    attn_len = k.shape[0]
    npages = (attn_len + page_tokens - 1) // page_tokens
    pool = np.zeros((npages, 2, kv_heads, page_tokens, hd), dtype=k.dtype)
    for t in range(attn_len):
        pool[t // page_tokens, 0, :, t % page_tokens, :] = k[t].reshape(kv_heads, hd)
        pool[t // page_tokens, 1, :, t % page_tokens, :] = v[t].reshape(kv_heads, hd)
    return pool, npages


@pytest.mark.parametrize("dtype,heads,kv_heads,hd,attn_len", [("bf16", 32, 32, 128, 1280), ("f32", 4, 2, 64, 100)])
def test_static_scratch_variant_matches_allocating_entry_point(dtype, heads, kv_heads, hd, attn_len):
    import torch

    from rustane_b200 import _ffi, ops
    rng = np.random.default_rng(7)
    dt = {"f32": 0, "f16": 1, "bf16": 2}[dtype]
    for call in range(2):  # two calls in a row share the scratch array
        q = rng.standard_normal(heads * hd).astype(np.float32)
        k = ops.to_storage(rng.standard_normal((attn_len, kv_heads * hd)).astype(np.float32), dtype)
        v = ops.to_storage(rng.standard_normal((attn_len, kv_heads * hd)).astype(np.float32), dtype)
        want = ops.flash_decode(q, k, v, heads, kv_heads, hd, dtype=dtype)

        pool, npages = _pack_pages(k, v, kv_heads, hd)
        raw = pool.view(np.int16) if pool.dtype == np.uint16 else pool
        d_pool = torch.from_numpy(raw.copy()).cuda()
        d_q = torch.from_numpy(q).cuda()
        d_pt = torch.arange(npages, dtype=torch.int32, device="cuda")
        d_out = torch.full((heads * hd,), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream().cuda_stream
        rc = _ffi.lib.cd_flash_decode_static(dt, heads, kv_heads, hd, attn_len, 0, 64,
                                             C.cast(d_q.data_ptr(), C.POINTER(C.c_float)), C.c_void_p(d_pool.data_ptr()),
                                             C.cast(d_pt.data_ptr(), C.POINTER(C.c_int32)),
                                             C.cast(d_out.data_ptr(), C.POINTER(C.c_float)), C.c_void_p(stream))
        assert rc == 0, _ffi.lib.cd_last_error(None).decode()
        torch.cuda.synchronize()
        got = d_out.cpu().numpy()
        np.testing.assert_allclose(got, want, atol=2e-5, rtol=1e-4)
        from test_gpu_ops import reference_attention
        ref = reference_attention(q, ops.from_storage(k, dtype), ops.from_storage(v, dtype), heads, kv_heads, hd)
        np.testing.assert_allclose(got, ref, atol=2e-5, rtol=1e-4)


def test_static_scratch_variant_rejects_shapes_beyond_its_fixed_array():
    import torch

    from rustane_b200 import _ffi
    buf = torch.zeros(1 << 16, dtype=torch.float32, device="cuda")
    pt = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = C.cast(buf.data_ptr(), C.POINTER(C.c_float))
    rc = _ffi.lib.cd_flash_decode_static(0, 128, 128, 64, 10, 1, 64, p, C.c_void_p(buf.data_ptr()),
                                         C.cast(pt.data_ptr(), C.POINTER(C.c_int32)), p, None)
    assert rc == _ffi.ERR_UNSUPPORTED
    assert b"at most 64 heads" in _ffi.lib.cd_last_error(None)
