#!/usr/bin/env python
"""Decode-throughput benchmark of the rustane token loop on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE config 3): the ~5B rustane LM in bf16 — vocab 32000, dim 4096, 26
layers, 32 heads x 128, SwiGLU hidden 11008, seq 4096 — with seeded synthetic weights
~N(0, 0.02) (seed 2), a 1024-token uniform-random prompt, batch-1 greedy decode.
One *step* is one sample's decode loop: 512 tokens generated from the shared prompt
prefill (positions 1024..1535).  `value` is decoded tokens per second with everything
resident in HBM (device loop, CUDA-event time); `e2e` is the same metric through the
reference-shaped per-token call `decode_token_argmax_from_id` (token id up from pinned
host memory, next id back, one host synchronisation per token).

`--impl reference` times the CPU restatement of the reference's KV-cached decode (the
oracle; the reference itself is an Apple ANE/Metal program and cannot run here) on the
host cores, on a bounded sample of the same model.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(dim=4096, hidden=11008, heads=32, hd=128, seq=4096, nlayers=26, vocab=32000)
SEED, PROMPT_LEN, DECODE_TOKENS = 2, 1024, 512
METRIC, UNIT = "decode_tokens_per_s", "tokens/s"
# DRAM bytes moved per algorithmic byte by one launch of the persistent token kernel, from the ncu capture on the
# 3-layer profile case (profiles/decode_mega_5b_profile_case.md): 1.5367 GB of DRAM traffic for 1.5271 GB algorithmic
MEGA_TRAFFIC_RATIO = 1.006
WORKLOAD = ("config 3: 5B rustane LM bf16 (V32000 D4096 L26 32x128 H11008 seq4096), synthetic N(0,0.02) seed 2, "
            "1024-token random prompt, batch-1 greedy, 512 decode tokens per step")


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


def bytes_per_token(ctx):
    """Algorithmic HBM bytes to decode one token at context length ctx (bf16 storage):
    every linear and the LM head once, one embedding row, the gammas (fp32), K and V of
    ctx cached positions read and one position written."""
    m = MODEL
    D, H, V, L = m["dim"], m["hidden"], m["vocab"], m["nlayers"]
    Q = KV = m["heads"] * m["hd"]
    linears = L * (D * Q + 2 * D * KV + Q * D + 3 * D * H) * 2
    head = V * D * 2
    small = D * 2 + (2 * L + 1) * D * 4
    kv = 2 * L * ctx * KV * 2 + 2 * L * KV * 2
    return linears + head + small + kv, linears + head


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, reasons = [], None, set()
        for line in self.tmp.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[0].isdigit() or int(f[0]) != self.gpu:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.tmp.name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def host_available_gb():
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:  # noqa: BLE001
        avail = 0
    for path in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            raw = open(path).read().strip()
            if raw.isdigit():
                used = 0
                try:
                    used = int(open(path.replace("memory.max", "memory.current")
                                    .replace("memory.limit_in_bytes", "memory.usage_in_bytes")).read())
                except Exception:  # noqa: BLE001
                    pass
                avail = min(avail, int(raw) - used) if avail else int(raw) - used
        except OSError:
            pass
    return avail / 2 ** 30


class CpuDecoder:
    """The oracle's KV-cached decode (fp32 math on the bf16-rounded weights, fp16-rounded cache) on the
    host cores, positioned where the GPU arm decodes: context PROMPT_LEN.  The cache rows of the prompt
    are left at zero instead of running the prompt through the CPU (that alone would take minutes):
    the time of a decode step does not depend on the cached values, only on how many there are.  Full
    depth when host memory allows (11 GB of weights), else 4 of 26 layers with the rate scaled by
    per-token bytes; either way the sample is described."""

    def __init__(self):
        from oracle import pyoracle as O
        self.cores = host_threads()
        os.environ.setdefault("OMP_NUM_THREADS", str(self.cores))
        self.layers = MODEL["nlayers"] if host_available_gb() > 24 else 4
        cfg = O.make_config(dtype=O.BF16, **dict(MODEL, nlayers=self.layers))
        self.model = O.Model.synth(cfg, SEED)
        self.cache = O.Cache(self.model, kv_round=1)
        self.cur = 1
        self.rewind()
        self.cur = self.cache.decode_token_argmax_from_id(self.cur)  # warm-up token (page-in of the weights)

    def rewind(self):
        self.cache.set_len(PROMPT_LEN)

    def decode(self, tokens, budget_s=1e9):
        """Greedy tokens from context PROMPT_LEN on; returns (tokens done, seconds)."""
        self.rewind()
        done, t0 = 0, time.perf_counter()
        while done < tokens and (done == 0 or time.perf_counter() - t0 < budget_s):
            self.cur = self.cache.decode_token_argmax_from_id(self.cur)
            done += 1
        return done, time.perf_counter() - t0

    def describe(self, done):
        text = "%d greedy tokens from context %d (cached rows of the prompt left at zero: step time does not depend on " \
               "their values), KV-cached CPU restatement, %d of %d layers" % (done, PROMPT_LEN, self.layers, MODEL["nlayers"])
        if self.layers != MODEL["nlayers"]:
            text += " (host memory too small for full depth: rate scaled by per-token bytes)"
        return text

    def scale(self, rate):
        if self.layers == MODEL["nlayers"]:
            return rate
        full, _ = bytes_per_token(PROMPT_LEN)
        part = full - (MODEL["nlayers"] - self.layers) * (full - MODEL["vocab"] * MODEL["dim"] * 2) / MODEL["nlayers"]
        return rate * part / full


def run_reference(args, rank, world):
    """The reference arm: a step is a bounded sample of the GPU arm's step (the first `per_step` of its
    512 tokens, decoded from the same context 1024); exactly `steps` steps are timed after `warmup`
    untimed ones, and ms_per_step is the measured time of such a sample, not an extrapolation."""
    if rank != 0:
        return
    per_step = max(8, min(64, 640 // max(1, args.steps + args.warmup)))
    cpu = CpuDecoder()
    for _ in range(args.warmup):
        cpu.decode(min(per_step, 4))
    done, secs = 0, 0.0
    for _ in range(args.steps):
        n, dt = cpu.decode(per_step)
        done += n
        secs += dt
    rate = cpu.scale(done / secs)
    sample = cpu.describe(done) + "; %d steps of %d tokens" % (args.steps, per_step)
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": secs / max(1, args.steps) * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 math on bf16-stored weights", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_step": per_step,
                   "arm": "CPU restatement of the reference's KV-cached decode (metal-decode shader math) on the host cores; "
                          "the reference itself needs Apple ANE/Metal — unavailable on this box"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cpu.cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


MOE = dict(dim=2048, hidden=1408, heads=16, seq=8192, nlayers=24, vocab=32000, n_experts=64, top_k=6, n_shared=2,
           kv_latent=512, rope_dim=64, nope_dim=128, v_dim=128)
MOE_PROMPT, MOE_STEPS = 2048, 256


def moe_bytes_per_token(ctx):
    """Algorithmic HBM bytes per decoded token of configuration 5 (bf16 weights, fp16 latent cache): attention
    and router matrices, top_k routed experts and the shared FFN of every layer, the LM head, the cached
    [latent | rope key] rows of ctx positions."""
    m = MOE
    D, H, L = m["dim"], m["heads"], m["nlayers"]
    qh, w = m["nope_dim"] + m["rope_dim"], m["kv_latent"] + m["rope_dim"]
    attn = D * (H * qh + w) + m["kv_latent"] * H * (m["nope_dim"] + m["v_dim"]) + H * m["v_dim"] * D
    ffn = 3 * D * m["hidden"] * (m["top_k"] + m["n_shared"]) + D * m["n_experts"]
    return (L * (attn + ffn) + m["vocab"] * D) * 2 + L * ctx * w * 2


def bench_moe(R, np, local_rank, rank, world, use_graph):
    """Configuration 5 beside the headline: the MoE + MLA decoder, 2048-token prompt (fed one token at a time: the
    batched prompt pass does not cover this architecture), 256 greedy steps at batch 1, then 8 samples with the
    full-vocabulary sampler at T 1.0, one after the other from the shared prompt.  world > 1: expert parallel."""
    mcfg = R.MoeConfig(**MOE)
    model = R.Model.moe_synthetic(mcfg, 4, dtype="bf16", device=local_rank, use_graph=use_graph, tp_rank=rank, tp_world=world)
    if world > 1:
        model.tp_connect_group()
    prompt = R.synth_prompt(4, MOE["vocab"], MOE_PROMPT)
    if world > 1:
        model.prefill(prompt[:-1], want_logits=False)
        first = model.decode_token_argmax_from_id(int(prompt[-1]))
    else:
        first = int(np.argmax(model.prefill(prompt)))
    prefill_ms = model.last_device_ms()
    model.set_len(MOE_PROMPT)
    model.decode_steps_greedy(first, 16)
    model.set_len(MOE_PROMPT)
    model.decode_steps_greedy(first, MOE_STEPS)
    ms1 = model.last_device_ms()
    ms8 = 0.0
    for s in range(8):
        model.set_len(MOE_PROMPT)
        model.decode_steps_fullvocab(first, MOE_STEPS, 1.0, 4 + s)
        ms8 += model.last_device_ms()
    model.close()
    rate1 = MOE_STEPS / (ms1 / 1e3)
    peak, _ = measured_peak_gbs()
    return {"workload": "config 5: MoE + MLA bf16 (V32000 D2048 L24, 16 heads over a 512 + 64 latent cache, 64 routed experts x 1408 + 2 shared, top-6), "
                        "2048-token prompt, 256 decode steps", "parallelism": "single GPU" if world == 1 else "ep%d" % world,
            "batch1_greedy_tokens_per_s": rate1, "samples8_fullvocab_tokens_per_s": 8 * MOE_STEPS / (ms8 / 1e3),
            "samples8_mode": "one after the other from the shared prompt",
            "prompt_tokens_per_s_token_at_a_time": MOE_PROMPT / (prefill_ms / 1e3),
            "hbm_bytes_per_token": moe_bytes_per_token(MOE_PROMPT + MOE_STEPS / 2),
            "token_roofline_frac_of_measured_peak": moe_bytes_per_token(MOE_PROMPT + MOE_STEPS / 2) / world * rate1 / 1e9 / peak}


def profile_case(dtype="bf16", per_operator=False):
    """Small case for `ncu`: identical kernels and shapes per layer, 3 of 26 layers (about
    1.5 GB resident, weights still far larger than L2), context 1024 (cache contents are
    zeros: timing and traffic do not depend on the values), 8 greedy tokens, no graph.
    per_operator selects one kernel per operator instead of the persistent per-token kernel."""
    import rustane_b200 as R
    model = R.Model.synthetic(R.Config(**dict(MODEL, nlayers=3)), SEED, dtype=dtype, use_graph=False, mega=not per_operator)
    model.set_len(PROMPT_LEN)
    ids = model.decode_steps_greedy(1, 8)
    print("profile case done: %d launches, last ids %s, %.3f ms/token" % (
        model.kernel_launches(), ids[-2:].tolist(), model.last_device_ms() / 8))


def profile_moe():
    """Small case for `ncu` on the MoE + MLA decoder: configuration 5's architecture cut to 3 of 24 layers
    (3.4 GB resident), context 2048 (zero-filled latent cache), 8 greedy tokens, no graph."""
    import rustane_b200 as R
    mcfg = dict(MOE)
    mcfg["nlayers"] = 3
    model = R.Model.moe_synthetic(R.MoeConfig(**mcfg), 4, dtype="bf16", use_graph=False)
    model.set_len(MOE_PROMPT)
    ids = model.decode_steps_greedy(1, 8)
    print("MoE profile case done: %d launches, last ids %s, %.3f ms/token" % (
        model.kernel_launches(), ids[-2:].tolist(), model.last_device_ms() / 8))


def profile_prefill():
    """Small case for `ncu` on the prompt pass: 3 of 26 layers, one 512-token prompt run twice
    (the first pass allocates the workspace); six GEMM launches per layer."""
    import rustane_b200 as R
    model = R.Model.synthetic(R.Config(**dict(MODEL, nlayers=3)), SEED, dtype="bf16", use_graph=False)
    prompt = R.synth_prompt(SEED, MODEL["vocab"], 512)
    for _ in range(2):
        model.set_len(0)
        model.prefill(prompt)
    print("prefill profile case done: 512 tokens in %.3f ms" % model.last_device_ms())


def profile_samples():
    """Small case for `ncu` on the multi-sample decode step: 3 of 26 layers, eight samples at
    position 1024 (cache contents are zeros), six steps with the full-vocabulary sampler."""
    import numpy as np

    import rustane_b200 as R
    model = R.Model.synthetic(R.Config(**dict(MODEL, nlayers=3)), SEED, dtype="bf16", use_graph=False, max_samples=8)
    model.set_len(PROMPT_LEN)
    model.decode_steps_samples(list(range(1, 9)), 6, mode="fullvocab", temperature=1.0, rng_states=np.arange(8, dtype=np.uint64))
    print("samples profile case done: %.3f ms per step of 8 samples" % (model.last_device_ms() / 6))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the quantised (configuration 4) side measurement")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for ncu captures: the same architecture cut to 3 layers, 1024-token context "
                         "seeded without a prefill pass, 8 decode tokens, no graph; prints no bench line")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8", "int4"],
                    help="storage of the linears in --profile-case (fp8 / int4: configuration 4's quantised rows)")
    ap.add_argument("--per-operator", action="store_true",
                    help="--profile-case with one kernel per operator (the path quantised and tensor-parallel models take)")
    ap.add_argument("--profile-moe", action="store_true",
                    help="small case for ncu captures of the MoE + MLA decoder (3 layers, context 2048, 8 tokens); prints no bench line")
    ap.add_argument("--profile-prefill", action="store_true",
                    help="small case for ncu captures of the batched prompt pass (3 layers, 512 tokens); prints no bench line")
    ap.add_argument("--profile-samples", action="store_true",
                    help="small case for ncu captures of the multi-sample decode step (3 layers, 8 samples); prints no bench line")
    args = ap.parse_args()
    if args.profile_case:
        return profile_case(args.dtype, args.per_operator)
    if args.profile_moe:
        return profile_moe()
    if args.profile_prefill:
        return profile_prefill()
    if args.profile_samples:
        return profile_samples()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import numpy as np
    import torch
    import torch.distributed as dist

    import rustane_b200 as R

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg = R.Config(**MODEL)
    prompt = R.synth_prompt(SEED, MODEL["vocab"], PROMPT_LEN)
    if world == 1:
        model = R.Model.synthetic(cfg, SEED, dtype="bf16", device=local_rank, use_graph=not args.no_graph,
                                  max_samples=1 if args.no_extras else 8)  # pages for the --samples 8 side measurement
        model.prefill(prompt)      # first pass allocates the prompt-pass workspace
        model.set_len(0)
        logits = model.prefill(prompt)
        prefill_ms = model.last_device_ms()
        first = int(np.argmax(logits))
    else:
        # tensor parallel: heads, FFN columns and LM-head rows split over the ranks, two [dim]
        # all-reduces per layer pushed over NVLink from inside the GEMV kernels
        model = R.Model.synthetic(cfg, SEED, dtype="bf16", device=local_rank, use_graph=not args.no_graph,
                                  tp_rank=rank, tp_world=world)
        model.tp_connect_group()
        model.prefill(prompt[:-1], want_logits=False)      # first pass allocates the prompt-pass workspace
        model.set_len(0)
        barrier()                                          # the ranks start the timed pass together; its time is the slowest rank's
        model.prefill(prompt[:-1], want_logits=False)
        pf = torch.tensor([model.last_device_ms()], dtype=torch.float64, device="cuda")
        dist.all_reduce(pf, op=dist.ReduceOp.MAX)
        prefill_ms = float(pf.item()) * PROMPT_LEN / (PROMPT_LEN - 1)
        first = model.decode_token_argmax_from_id(int(prompt[-1]))

    def one_step():
        model.set_len(PROMPT_LEN)
        ids = model.decode_steps_greedy(first, DECODE_TOKENS)
        return ids, model.last_device_ms()

    ref_ids = None
    for _ in range(args.warmup):
        ref_ids, _ = one_step()

    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    launches0 = model.kernel_launches()
    dev_ms = 0.0
    for _ in range(args.steps):
        ids, ms = one_step()
        dev_ms += ms
        assert np.array_equal(ids, ref_ids), "greedy decode is not deterministic"
    barrier()
    clocks = sampler.stop()
    launches = model.kernel_launches() - launches0

    # end to end through the reference-shaped per-token call (host buffers, sync per token)
    model.set_len(PROMPT_LEN)
    cur = first
    for _ in range(8):
        cur = model.decode_token_argmax_from_id(cur)
    model.set_len(PROMPT_LEN)
    e2e_tokens = DECODE_TOKENS * min(args.steps, 2)
    barrier()
    t0 = time.perf_counter()
    for s in range(min(args.steps, 2)):
        model.set_len(PROMPT_LEN)
        cur, got = first, []
        for _ in range(DECODE_TOKENS):
            cur = model.decode_token_argmax_from_id(cur)
            got.append(cur)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    assert got == ref_ids.tolist(), "per-token API and device loop disagree"

    times = torch.tensor([dev_ms, e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s = float(times[0]), float(times[1])

    # per-class kernel time of one token at the mean context of the timed region
    model.set_len(PROMPT_LEN + DECODE_TOKENS // 2)
    prof = model.profile_decode_step(int(ref_ids[DECODE_TOKENS // 2 - 1]))
    gemv_ms = sum(prof[k][0] for k in ("qkv_gemv", "wo_gemv", "w13_gemv", "w2_gemv", "head_gemv"))
    gemv_launches = sum(prof[k][1] for k in ("qkv_gemv", "wo_gemv", "w13_gemv", "w2_gemv", "head_gemv"))
    mean_ctx = PROMPT_LEN + (DECODE_TOKENS + 1) / 2.0
    tok_bytes, weight_bytes = bytes_per_token(mean_ctx)
    peak, peak_kind = measured_peak_gbs()
    tokens = DECODE_TOKENS * args.steps  # one stream, whatever the number of GPUs (tensor parallel)
    value = tokens / (dev_ms / 1e3)
    step_ms = dev_ms / args.steps
    gemv_gbs = weight_bytes / world / (gemv_ms / 1e3) / 1e9  # all five weight-streaming GEMV kinds together (per GPU)
    # dominant kernel: the W1|W3 GEMV (one launch per layer streams the interleaved [2H, D] matrix once)
    w13_bytes = 2 * MODEL["hidden"] * MODEL["dim"] * 2 // world  # this GPU's shard
    w13_ms, w13_launches = prof["w13_gemv"]
    w13_gbs = w13_bytes / (w13_ms / w13_launches / 1e3) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": "single GPU" if world == 1 else "tp%d (heads, FFN columns, LM-head rows; fused push all-reduce)" % world,
                   "l2": "inputs larger than L2: 10.8 GB of weights stream from HBM for every token",
                   "kv_cache_dtype": "fp16 (2 bytes per element, as bf16 would be)",
                   "cuda_graph": not args.no_graph, "ms_per_token": step_ms / DECODE_TOKENS,
                   "prefill_tokens_per_s": PROMPT_LEN / (prefill_ms / 1e3),
                   "prefill_path": ("batched tcgen05 GEMM pass, hi+lo activations" if world == 1 else "batched tcgen05 GEMM pass, hi+lo activations; Wo / W2 partial products all-reduced through peer memory"),
                   "hbm_bytes_per_token": tok_bytes,
                   "token_roofline_frac_of_%s_peak" % peak_kind: tok_bytes / world * value / 1e9 / peak,
                   "token_roofline_frac_of_nominal_8TBs": tok_bytes / world * value / 1e9 / 8000.0,
                   "kernel_ms_by_class_one_token": {k: round(v[0], 4) for k, v in prof.items()}},
        "clocks": clocks,
        "e2e": {"value": e2e_tokens / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 8 * DECODE_TOKENS,
                "d2h_bytes_per_step": 4 * DECODE_TOKENS},
        "gpu_launches": int(launches),
    }
    per_operator = {"kernel": "gemv_tma_kernel<bf16, EpiGate> (W1|W3 GEMV, %d launches per token)" % w13_launches,
                    "achieved": w13_gbs, "frac": w13_gbs / peak, "algorithmic_bytes_per_launch": w13_bytes,
                    "timing": "CUDA events on the launching stream around every launch of one token of the kernel-per-operator "
                              "path (no graph, no overlap with neighbours: includes the per-launch gap)",
                    "all_gemv_kinds_gbs": gemv_gbs}
    peak_source = "MEASURED_PEAKS.json hbm_gbs (of measured)" if peak_kind == "measured" else "6650 (of fallback)"
    if world == 1:
        # The dominant kernel is the whole token: decode_mega_kernel, one launch per token, streams every weight and
        # the cached K/V once.  Its duration is the CUDA-event time of the timed loop per token (the loop's only
        # other kernel is the 3 us head reduction).  `traffic`: dram__bytes_read.sum + dram__bytes_write.sum of one
        # launch on the 3-layer profile case (profiles/decode_mega_5b_profile_case.md) scaled by algorithmic bytes.
        mega_gbs = tok_bytes / (step_ms / DECODE_TOKENS / 1e3) / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": "decode_mega_kernel<bf16, fp16 KV> (one launch per token: all layers and the LM head)",
                            "achieved": mega_gbs, "peak": peak, "unit": "GB/s", "frac": mega_gbs / peak, "peak_source": peak_source,
                            "algorithmic_bytes_per_launch": tok_bytes, "traffic": MEGA_TRAFFIC_RATIO * tok_bytes if MEGA_TRAFFIC_RATIO else None,
                            "timing": "CUDA events on the launching stream around the timed loop, divided by its launches",
                            "kernel_per_operator_path": per_operator}
    else:
        line["roofline"] = dict(per_operator, bound="hbm", peak=peak, unit="GB/s", peak_source=peak_source, traffic=None)
    def side(name, fn):
        """A measurement beside the headline: its failure is recorded in the line, it does not cost the headline."""
        try:
            line["config"][name] = fn()
        except Exception as exc:  # noqa: BLE001
            line["config"][name + "_error"] = repr(exc)[:300]

    if world == 1 and not args.no_extras:
        def samples8():
            # configuration 3's `--samples 8` mode (T 1.0, k 0: block-stats sampler): eight samples share the
            # prompt and advance together; aggregate sampled tokens per second over 128 steps
            firsts = [int(i) for i in np.argsort(-logits)[:8]]
            model.set_len(PROMPT_LEN)
            model.decode_steps_samples(firsts, 16, mode="fullvocab", temperature=1.0, rng_states=np.arange(8, dtype=np.uint64) + SEED)
            model.set_len(PROMPT_LEN)
            model.decode_steps_samples(firsts, 128, mode="fullvocab", temperature=1.0, rng_states=np.arange(8, dtype=np.uint64) + SEED)
            return 8 * 128 / (model.last_device_ms() / 1e3)

        def config4():
            # configuration 4 beside the headline: the same architecture with quantised linears (seed 3),
            # the same 1024-token prompt and 512 greedy tokens; device-loop time of one step each
            extra = {}
            for dt in ("fp8", "int4"):
                qm = R.Model.synthetic(cfg, 3, dtype=dt, device=local_rank, use_graph=not args.no_graph)
                qfirst = int(np.argmax(qm.prefill(prompt)))
                qm.decode_steps_greedy(qfirst, 32)
                qm.set_len(PROMPT_LEN)
                qm.decode_steps_greedy(qfirst, DECODE_TOKENS)
                extra[dt + "_tokens_per_s"] = DECODE_TOKENS / (qm.last_device_ms() / 1e3)
                qm.close()
            return extra

        def prefill4096():
            # configuration 3's prefill-only mode: 4096 prompt tokens through the tensor-core pass (second run: the first allocates)
            p4 = R.synth_prompt(SEED, MODEL["vocab"], 4096)
            for _ in range(2):
                model.set_len(0)
                model.prefill(p4)
            return 4096 / (model.last_device_ms() / 1e3)

        side("samples8_fullvocab_tokens_per_s", samples8)
        side("config4_quantised_linears", config4)
        side("prefill4096_tokens_per_s", prefill4096)
        model.close()
        side("config5_moe_mla", lambda: bench_moe(R, np, local_rank, 0, 1, not args.no_graph))
    elif world > 1 and not args.no_extras:
        model.close()

        def config4_tp():
            # configuration 4 at this rank count: quantised linears under tensor parallelism (every rank's shard is a byte
            # slice of the single-GPU model's rows), prompt fed one token at a time, 512 greedy tokens; max over ranks
            extra = {}
            for dt in ("fp8", "int4"):
                qm = R.Model.synthetic(cfg, 3, dtype=dt, device=local_rank, use_graph=not args.no_graph, tp_rank=rank, tp_world=world)
                qm.tp_connect_group()
                qm.prefill(prompt[:-1], want_logits=False)
                qfirst = qm.decode_token_argmax_from_id(int(prompt[-1]))
                qm.decode_steps_greedy(qfirst, 32)
                qm.set_len(PROMPT_LEN)
                barrier()
                qm.decode_steps_greedy(qfirst, DECODE_TOKENS)
                t = torch.tensor([qm.last_device_ms()], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                extra[dt + "_tokens_per_s"] = DECODE_TOKENS / (float(t.item()) / 1e3)
                qm.close()
            return extra

        side("config4_quantised_linears", config4_tp)
        side("config5_moe_mla", lambda: bench_moe(R, np, local_rank, rank, world, not args.no_graph))
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            cpu = CpuDecoder()
            done, secs = cpu.decode(96, budget_s=25.0)
            line["cpu_baseline"] = {"value": cpu.scale(done / secs), "unit": UNIT, "cores": cpu.cores, "kind": "port",
                                    "sample": cpu.describe(done)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
