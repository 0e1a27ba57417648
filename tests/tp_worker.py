"""Worker of the tensor-parallel tests: launched once per rank by torch.distributed.run.

GPU mode (default): every rank builds its shard of a synthetic model, connects the link
regions, and checks greedy decoding against a single-GPU model of the same weights.
CPU mode (--cpu, gloo): checks the shard plan, the partial-sum algebra and the two sampler exchanges
(per-block candidates; per-block (max, sum) with the block's owner drawing) the GPU path relies on.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import rustane_b200 as R  # noqa: E402
from rustane_b200 import _ffi  # noqa: E402


def shard_plan(cfg, world, rank):
    c, loc = cfg.to_c(), _ffi.CdConfig()
    v0, vn = C.c_int32(), C.c_int32()
    rc = _ffi.lib.cd_tp_shard_plan(C.byref(c), world, rank, C.byref(loc), C.byref(v0), C.byref(vn))
    assert rc == 0, rc
    return loc, v0.value, vn.value


def cpu_main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = R.Config(4096, 11008, 32, 128, 4096, 26, 32000)
    loc, v0, vn = shard_plan(cfg, world, rank)
    mine = torch.tensor([loc.heads, loc.kv_heads, loc.hidden, loc.q_dim, loc.kv_dim, v0, vn])
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    tot = torch.stack(everyone)
    assert tot[:, 0].sum() == cfg.heads and tot[:, 2].sum() == cfg.hidden and tot[:, 3].sum() == cfg.q_dim
    assert int(tot[0, 5]) == 0 and int(tot[-1, 5] + tot[-1, 6]) == cfg.vocab
    for r in range(1, world):
        assert int(tot[r, 5]) == int(tot[r - 1, 5] + tot[r - 1, 6]) and int(tot[r, 5]) % 256 == 0
    # the algebra: a product split along its input is a sum of per-rank partial vectors, a product
    # split along its output is a concatenation; every rank adds the partials in rank order
    rng = np.random.default_rng(0)
    D, H = 64, 96
    x = rng.standard_normal(D).astype(np.float32)
    w1 = rng.standard_normal((D, H)).astype(np.float32)   # [in, out]: split along out
    w2 = rng.standard_normal((D, H)).astype(np.float32)   # [out, in]: split along in
    hs = H // world
    h_local = x @ w1[:, rank * hs:(rank + 1) * hs]
    partial = torch.from_numpy(w2[:, rank * hs:(rank + 1) * hs] @ h_local)
    parts = [torch.zeros_like(partial) for _ in range(world)]
    dist.all_gather(parts, partial)
    y = np.zeros(D, dtype=np.float32)
    for p in parts:  # fixed rank order on every rank
        y += p.numpy()
    np.testing.assert_allclose(y, w2 @ (x @ w1), rtol=2e-5, atol=2e-5)
    ys = [torch.zeros(D) for _ in range(world)]
    dist.all_gather(ys, torch.from_numpy(y))
    for other in ys:
        assert torch.equal(other, ys[0])  # bit-identical on all ranks
    sampler_exchange_cpu(rank, world)
    expert_parallel_cpu(rank, world)
    dist.destroy_process_group()
    if rank == 0:
        print("tp cpu ok")


def expert_parallel_cpu(rank, world):
    """Expert placement and the combine step of expert parallelism on CPU ranks: the plan tiles the routed
    experts and the shared FFN's columns; every rank evaluates only the chosen experts it holds (and its slice
    of the shared FFN); the partial sums gathered from all ranks and added in rank order give, on every rank
    alike, the single-process FFN output."""
    mcfg = R.MoeConfig(dim=64, hidden=48, heads=4, seq=32, nlayers=1, vocab=256, n_experts=8, top_k=3, n_shared=2,
                       kv_latent=32, rope_dim=16, nope_dim=16, v_dim=16)
    c, mc = mcfg.base.to_c(), mcfg.to_c()
    plan = [C.c_int32() for _ in range(4)]
    assert _ffi.lib.cd_moe_shard_plan(C.byref(c), C.byref(mc), world, rank, *[C.byref(p) for p in plan]) == 0
    e0, ne, s0, sc = (p.value for p in plan)
    mine = torch.tensor([e0, ne, s0, sc])
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    tot = torch.stack(everyone)
    assert int(tot[:, 1].sum()) == mcfg.n_experts and int(tot[:, 3].sum()) == mcfg.n_shared * 48
    for r in range(1, world):
        assert int(tot[r, 0]) == int(tot[r - 1, 0] + tot[r - 1, 1]) and int(tot[r, 2]) == int(tot[r - 1, 2] + tot[r - 1, 3])
    rng = np.random.default_rng(3)  # the same tensors on every rank
    D, Hd, SH = 64, 48, 96
    x = rng.standard_normal(D).astype(np.float32)
    w1 = rng.standard_normal((8, D, Hd)).astype(np.float32) * 0.1
    w3 = rng.standard_normal((8, D, Hd)).astype(np.float32) * 0.1
    w2 = rng.standard_normal((8, D, Hd)).astype(np.float32) * 0.1           # [out, in]
    s1, s3 = (rng.standard_normal((D, SH)).astype(np.float32) * 0.1 for _ in range(2))
    s2 = rng.standard_normal((D, SH)).astype(np.float32) * 0.1
    wr = rng.standard_normal((D, 8)).astype(np.float32)
    logits = x @ wr
    p = np.exp(logits - logits.max()); p /= p.sum()
    chosen = sorted(range(8), key=lambda e: (-p[e], e))[:3]                 # every rank picks the same experts

    def ffn(a1, a3, a2):
        h = x @ a1
        return a2 @ ((h / (1.0 + np.exp(-h))) * (x @ a3))
    whole = sum(p[e] * ffn(w1[e], w3[e], w2[e]) for e in chosen) + ffn(s1, s3, s2)
    part = np.zeros(D, dtype=np.float32)
    for e in chosen:
        if e0 <= e < e0 + ne:
            part += (p[e] * ffn(w1[e], w3[e], w2[e])).astype(np.float32)
    part += ffn(s1[:, s0:s0 + sc], s3[:, s0:s0 + sc], s2[:, s0:s0 + sc]).astype(np.float32)
    parts = [torch.zeros(D) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(part))
    y = np.zeros(D, dtype=np.float32)
    for q in parts:  # fixed rank order on every rank
        y += q.numpy()
    np.testing.assert_allclose(y, whole, rtol=2e-4, atol=2e-5)
    ys = [torch.zeros(D) for _ in range(world)]
    dist.all_gather(ys, torch.from_numpy(y))
    assert all(torch.equal(o, ys[0]) for o in ys)


def sampler_exchange_cpu(rank, world):
    """The two head exchanges of sampled decoding, with the oracle's samplers as the arithmetic:
    (a) full-vocabulary block sampler: per-block (max, sum) of every shard to every rank, all pick the
    same block, the rank that owns it draws the token and hands (token, LCG state) on;
    (b) top-k: per-block candidates of every shard to every rank, the same merge and draw everywhere.
    Both must equal the single-process result on the whole logits vector."""
    from oracle import pyoracle as O
    V, T, K = 2000, 0.8, 8  # 8 blocks of 256 (the last ragged); the last rank owns fewer rows
    nblk = (V + 255) // 256
    per = (nblk + world - 1) // world
    v0 = min(V, rank * per * 256)
    vn = min(V - v0, per * 256)
    logits = (np.random.default_rng(5).standard_normal(V) * 3).astype(np.float32)

    def stats(lg, nb):  # logits_block_stats: max of z = logit / T and sum exp(z - max) per 256-row block; padding blocks carry no weight
        mx = np.full(nb, -np.inf, dtype=np.float32)
        sm = np.full(nb, np.nan, dtype=np.float32)
        for b in range((len(lg) + 255) // 256):
            z = lg[b * 256:(b + 1) * 256] * np.float32(1.0 / T)
            mx[b] = z.max()
            sm[b] = np.exp(z - mx[b], dtype=np.float32).sum(dtype=np.float32)
        return mx, sm

    for seed in range(40):
        # single process
        rng = C.c_uint64(1000 + seed)
        mx, sm = stats(logits, nblk)
        blk = O.lib.orc_sample_block_from_stats(O._f32(mx), O._f32(sm), nblk, C.byref(rng))
        row = np.ascontiguousarray(logits[blk * 256:min(V, blk * 256 + 256)])
        want = blk * 256 + O.lib.orc_sample_softmax_index(O._f32(row), len(row), T, C.byref(rng))
        want_rng = rng.value
        # tensor parallel
        mine = torch.from_numpy(np.stack(stats(logits[v0:v0 + vn], per)))
        rows = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(rows, mine)
        gmx = np.ascontiguousarray(np.concatenate([r[0].numpy() for r in rows]))
        gsm = np.ascontiguousarray(np.concatenate([r[1].numpy() for r in rows]))
        rng = C.c_uint64(1000 + seed)
        gblk = O.lib.orc_sample_block_from_stats(O._f32(gmx), O._f32(gsm), world * per, C.byref(rng))
        owner = gblk // per
        msg = torch.zeros(3, dtype=torch.int64)
        if owner == rank:
            lo = gblk * 256 - v0
            row = np.ascontiguousarray(logits[v0 + lo:v0 + min(vn, lo + 256)])
            tok = gblk * 256 + O.lib.orc_sample_softmax_index(O._f32(row), len(row), T, C.byref(rng))
            msg = torch.tensor([tok, rng.value >> 32, rng.value & 0xFFFFFFFF], dtype=torch.int64)
        dist.broadcast(msg, src=owner)
        got_rng = (int(msg[1]) << 32) | int(msg[2])
        assert int(msg[0]) == want and got_rng == want_rng, (rank, seed, int(msg[0]), want)

        # top-k candidates: k rounds of arg-max-and-remove per block, lower index wins ties
        def block_topk(lg, first_row, nb):
            vals = np.full(nb * K, -np.inf, dtype=np.float32)
            idxs = np.full(nb * K, 0xFFFFFFFF, dtype=np.uint32)
            for b in range((len(lg) + 255) // 256):
                seg = lg[b * 256:(b + 1) * 256]
                order = sorted(range(len(seg)), key=lambda i: (-seg[i], i))[:K]
                for j, i in enumerate(order):
                    vals[b * K + j], idxs[b * K + j] = seg[i], first_row + b * 256 + i
            return vals, idxs
        wv, wi = block_topk(logits, 0, nblk)
        mv, mi = O.merge_topk(wv, wi, K)
        rng = C.c_uint64(77 + seed)
        want = O.lib.orc_sample_topk_candidates(O._u32(mi), O._f32(mv), len(mv), T, C.byref(rng))
        lv, li = block_topk(logits[v0:v0 + vn], v0, per)
        tv, ti = torch.from_numpy(lv), torch.from_numpy(li.astype(np.int64))
        gv = [torch.zeros_like(tv) for _ in range(world)]
        gi = [torch.zeros_like(ti) for _ in range(world)]
        dist.all_gather(gv, tv)
        dist.all_gather(gi, ti)
        av = np.ascontiguousarray(torch.cat(gv).numpy())
        ai = np.ascontiguousarray(torch.cat(gi).numpy().astype(np.uint32))
        mv2, mi2 = O.merge_topk(av, ai, K)
        rng2 = C.c_uint64(77 + seed)
        got = O.lib.orc_sample_topk_candidates(O._u32(mi2), O._f32(mv2), len(mv2), T, C.byref(rng2))
        assert got == want and rng2.value == rng.value, (rank, seed, got, want)


def gpu_main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cases = [((512, 1536, 8, 64, 512, 3, 8192), "f32", True, False), ((1024, 2816, 8, 128, 512, 4, 32000), "bf16", False, True),
             ((2048, 5632, 16, 128, 1024, 2, 32000), "f16", True, True),
             # quantised linears: every rank quantises its shard with the scales of the unsharded matrix
             ((1024, 2816, 8, 128, 512, 3, 32000), "fp8", False, True), ((1024, 2816, 8, 128, 512, 3, 32000), "int4", False, False)]
    for dims, dtype, untied, graph in cases:
        cfg = R.Config(*dims)
        tp = R.Model.synthetic(cfg, 17, dtype=dtype, untied_head=untied, device=local, tp_rank=rank, tp_world=world, use_graph=graph)
        tp.tp_connect_group()
        one = R.Model.synthetic(cfg, 17, dtype=dtype, untied_head=untied, device=local)
        prompt = R.synth_prompt(5, cfg.vocab, 33)
        logits = one.prefill(prompt)
        first = int(np.argmax(logits))
        tp.prefill(prompt, want_logits=False)
        want = one.decode_steps_greedy(first, 40).tolist()
        got = tp.decode_steps_greedy(first, 40).tolist()
        n = 0  # the all-reduce adds the ranks' partial sums in another order than one GPU's GEMV: a near tie may flip late
        while n < 40 and got[n] == want[n]:
            n += 1
        assert n >= 20, (rank, dims, dtype, got, want)
        if dtype in ("bf16", "f16"):
            # the batched prompt pass under tensor parallelism (Wo / W2 partial products all-reduced through the link
            # region), a 200-token prompt in two chunks: the continuation is the single GPU's
            long_prompt = R.synth_prompt(9, cfg.vocab, 200)
            one.set_len(0); tp.set_len(0)
            f2 = int(np.argmax(one.prefill(long_prompt)))
            before = tp.kernel_launches()
            tp.prefill(long_prompt[:120], want_logits=False)
            tp.prefill(long_prompt[120:], want_logits=False)
            assert tp.kernel_launches() - before < 200 * cfg.nlayers, "the prompt went one token at a time"
            w2, g2 = one.decode_steps_greedy(f2, 24).tolist(), tp.decode_steps_greedy(f2, 24).tolist()
            n = 0
            while n < 24 and g2[n] == w2[n]:
                n += 1
            assert n >= 12, (rank, dims, dtype, g2, w2)
            one.set_len(0); tp.set_len(0)
            one.prefill(prompt); tp.prefill(prompt, want_logits=False)
        tp.set_len(len(prompt)); one.set_len(len(prompt))
        cur_a = cur_b = first
        for _ in range(6):  # the reference-shaped per-token call
            cur_a, cur_b = tp.decode_token_argmax_from_id(cur_a), one.decode_token_argmax_from_id(cur_b)
            assert cur_a == cur_b
        # sampled decoding: every rank's per-block candidates go to every rank, all draw the same token
        tp.set_len(len(prompt)); one.set_len(len(prompt))
        want_s, want_rng = one.decode_steps_topk(first, 24, 8, 0.9, 77)
        got_s, got_rng = tp.decode_steps_topk(first, 24, 8, 0.9, 77)
        n = 0
        while n < 24 and int(got_s[n]) == int(want_s[n]):
            n += 1
        assert n >= 12, (rank, dims, got_s.tolist(), want_s.tolist())  # partial sums add in another order: a draw may flip late
        assert n < 24 or got_rng == want_rng
        got = got + got_s.tolist()
        # full-vocabulary block sampler: per-block (max, sum) to every rank, the block's owner draws the token
        tp.set_len(len(prompt)); one.set_len(len(prompt))
        want_f, want_rng = one.decode_steps_fullvocab(first, 24, 0.8, 91)
        got_f, got_rng = tp.decode_steps_fullvocab(first, 24, 0.8, 91)
        n = 0
        while n < 24 and int(got_f[n]) == int(want_f[n]):
            n += 1
        assert n >= 12, (rank, dims, got_f.tolist(), want_f.tolist())
        assert n < 24 or got_rng == want_rng
        got = got + got_f.tolist() + [got_rng]
        # the reference-shaped per-token top-k call: every rank returns all ranks' per-block candidates, in block order
        tp.set_len(len(prompt)); one.set_len(len(prompt))
        wv, wi = one.decode_token_topk_from_id(first, 8)
        gv, gi = tp.decode_token_topk_from_id(first, 8)
        assert gv.shape == wv.shape and np.mean(gi == wi) > 0.99, (rank, dims, float(np.mean(gi == wi)))
        np.testing.assert_allclose(gv, wv, atol=2e-3, rtol=0)
        assert tp.len() == len(prompt) + 1
        got = got + gi.tolist()
        everyone = [None] * world
        dist.all_gather_object(everyone, got)
        assert all(e == got for e in everyone)
        try:
            tp.decode_token_logits_from_id(1)
            raise AssertionError("logits call should be refused on a tensor-parallel model")
        except R.CudaDecodeError as exc:
            assert exc.code == _ffi.ERR_UNSUPPORTED
        dist.barrier()
        tp.close(); one.close()
    # expert parallelism: the MoE + MLA decoder with its routed experts and the shared FFN's columns spread over the ranks
    mcfg = R.MoeConfig(dim=1024, hidden=704, heads=16, seq=256, nlayers=3, vocab=8192, n_experts=16, top_k=6, n_shared=2,
                       kv_latent=512, rope_dim=64, nope_dim=128, v_dim=128)
    for graph in (False, True):
        ep = R.Model.moe_synthetic(mcfg, 23, dtype="bf16", device=local, tp_rank=rank, tp_world=world, use_graph=graph)
        ep.tp_connect_group()
        one = R.Model.moe_synthetic(mcfg, 23, dtype="bf16", device=local)
        prompt = R.synth_prompt(6, mcfg.base.vocab, 30)
        first = int(np.argmax(one.prefill(prompt)))
        ep.prefill(prompt, want_logits=False)
        want = one.decode_steps_greedy(first, 24).tolist()
        got = ep.decode_steps_greedy(first, 24).tolist()
        n = 0
        while n < 24 and got[n] == want[n]:
            n += 1
        assert n >= 12, (rank, "moe", got, want)
        for layer in range(3):
            assert ep.moe_last_experts(layer).tolist() == one.moe_last_experts(layer).tolist() or n < 24
        ep.set_len(len(prompt)); one.set_len(len(prompt))
        want_s, _ = one.decode_steps_topk(first, 16, 8, 0.9, 5)
        got_s, _ = ep.decode_steps_topk(first, 16, 8, 0.9, 5)
        assert got_s.tolist()[:8] == want_s.tolist()[:8], (rank, got_s.tolist(), want_s.tolist())
        everyone = [None] * world
        dist.all_gather_object(everyone, got + got_s.tolist())
        assert all(e == everyone[0] for e in everyone)
        dist.barrier()
        ep.close(); one.close()
    dist.destroy_process_group()
    if rank == 0:
        print("tp gpu ok")


if __name__ == "__main__":
    cpu_main() if "--cpu" in sys.argv else gpu_main()
