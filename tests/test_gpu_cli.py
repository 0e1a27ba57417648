"""The `generate` binary end to end on the GPU: checkpoint -> session -> report lines
(bin/generate.rs:493-729), against the Python session on the same checkpoint."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ids(line):
    return [int(x) for x in re.findall(r"\d+", line.split("=", 1)[1])]


@pytest.mark.parametrize("samples,extra", [(1, ["--temperature", "0"]), (3, ["--temperature", "0.8", "--top-k", "8"]),
                                           (3, ["--temperature", "0", "--dtype", "fp8"])])
def test_generate_cli_matches_python_session(R, tmp_path, samples, extra):
    cfg = R.Config(256, 640, 2, 128, 96, 2, 1500)
    path = str(tmp_path / "tiny.rstk")
    R.write_synthetic_checkpoint(path, cfg, dtype="bf16", seed=4)
    prompt = [5, 6, 7, 8, 9, 10, 11, 12, 13]
    cmd = [os.path.join(ROOT, "rustane_b200", "generate"), "--checkpoint", path, "--prompt-ids", ",".join(map(str, prompt)),
           "--decode-backend", "cuda", "--steps", "12", "--samples", str(samples), "--seed", "3"] + extra
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = out.stdout.splitlines()
    key = "generated_ids=" if samples == 1 else "_generated_ids="
    got = [_ids(l) for l in lines if key in l]
    assert len(got) == samples and all(len(g) == 12 for g in got)
    t = float(extra[extra.index("--temperature") + 1])
    k = int(extra[extra.index("--top-k") + 1]) if "--top-k" in extra else 0
    dtype = extra[extra.index("--dtype") + 1] if "--dtype" in extra else None
    gm = R.Model.from_checkpoint(path, dtype=dtype, max_samples=samples)
    sess = R.InferenceSession(gm, prompt)
    ref = sess.generate(R.GenerationRequest("cuda", 12, t, k, samples, 3))
    assert got == [r.sampled for r in ref.results]
    assert any(l.startswith("total_generation_time=") for l in lines)


def test_jsonl_session_contract(R, tmp_path):
    """`generate --jsonl-session` (bin/generate.rs:413-491): one JSON response per request line; a request
    without fields takes the CLI defaults (generate.rs:758-778); an unknown backend, samples = 0, mixed
    suffix inputs and malformed JSON come back as {"error": ...} lines (generate.rs:85-88, :780-821) and
    the session goes on; a suffix request equals a fresh session on prompt + suffix."""
    import json
    cfg = R.Config(256, 640, 2, 128, 96, 2, 1500)
    path = str(tmp_path / "tiny.rstk")
    R.write_synthetic_checkpoint(path, cfg, dtype="bf16", seed=4)
    prompt = [5, 6, 7, 8, 9, 10, 11, 12, 13]
    suffix = [20, 21, 22, 23, 24, 25, 26, 27, 28, 29]      # long enough to go through the chunked prompt pass
    requests = [
        "{}",
        '{"decode_backend": "bad"}',
        '{"samples": 0}',
        '{"append_prompt_ids": [1, 2], "append_prompt": "hello"}',
        "this is not json",
        "",
        json.dumps({"append_prompt_ids": suffix, "steps": 6, "temperature": 0.0, "samples": 1, "decode_backend": "cuda"}),
        '{"append_prompt": "text needs a tokenizer"}',
        json.dumps({"steps": 5, "temperature": 0.0, "samples": 1, "seed": 9}),
    ]
    cmd = [os.path.join(ROOT, "rustane_b200", "generate"), "--checkpoint", path, "--prompt-ids", ",".join(map(str, prompt)),
           "--jsonl-session", "--steps", "7", "--temperature", "0.8", "--top-k", "8", "--samples", "2", "--seed", "7"]
    out = subprocess.run(cmd, input="\n".join(requests) + "\n", capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(l) for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 8                                  # the empty line produces nothing
    first = lines[0]                                        # CLI defaults: auto backend, 7 steps, T 0.8, k 8, 2 samples, seed 7
    assert first["decode_backend_request"] == "auto" and len(first["results"]) == 2
    assert [r["seed"] for r in first["results"]] == [7, 8]
    assert all(len(r["generated_ids"]) == 7 and r["full_sequence"] == prompt + r["generated_ids"] for r in first["results"])
    assert first["base_prompt_ids"] == prompt and first["prompt_ids"] == prompt and first["request_prefill_ms"] == 0.0
    for key in ("decode_mode", "fallback_reason", "auto_reason", "base_prefill_ms", "base_prefill_tok_per_s", "total_prefill_ms",
                "request_decode_ms_total", "request_decode_ms_avg", "request_avg_decode_tok_per_s",
                "end_to_end_ms_including_prefill", "end_to_end_tok_per_s_including_prefill", "base_prompt_text", "prompt_text"):
        assert key in first
    assert "decode_backend must be one of" in lines[1]["error"]
    assert lines[2]["error"] == "samples must be >= 1"
    assert "either append_prompt_ids or append_prompt" in lines[3]["error"]
    assert lines[4]["error"].startswith("invalid json request")
    sfx = lines[5]
    assert sfx["decode_mode"] == "kv_cache_cuda" and sfx["prompt_ids"] == prompt + suffix and sfx["request_prefill_ms"] > 0.0
    assert "requires the session to be started with --tokenizer" in lines[6]["error"]
    # the same answers from the Python session: defaults, suffix == fresh (inference.rs:1001-1033), and after the suffix request
    gm = R.Model.from_checkpoint(path, max_samples=2)
    sess = R.InferenceSession(gm, prompt)
    ref = sess.generate(R.GenerationRequest("auto", 7, 0.8, 8, 2, 7))
    assert [r["generated_ids"] for r in first["results"]] == [r.sampled for r in ref.results]
    fresh = R.InferenceSession(gm, prompt + suffix).generate(R.GenerationRequest("cuda", 6, 0.0, 8, 1, 7))
    assert sfx["results"][0]["generated_ids"] == fresh.results[0].sampled
    again = R.InferenceSession(gm, prompt).generate(R.GenerationRequest("auto", 5, 0.0, 8, 1, 9))
    assert lines[7]["results"][0]["generated_ids"] == again.results[0].sampled and lines[7]["prompt_ids"] == prompt


def test_generate_cli_converts_and_runs_a_quantised_checkpoint(R, tmp_path):
    """`generate --convert-to OUT --dtype int4` writes the quantised file once; generating from OUT gives the ids of
    generating from the plain file with --dtype int4 (quantised at load)."""
    cfg = R.Config(256, 640, 2, 128, 96, 2, 1500)
    plain, quant = str(tmp_path / "plain.rstk"), str(tmp_path / "int4.rstk")
    R.write_synthetic_checkpoint(plain, cfg, dtype="bf16", seed=4)
    exe = os.path.join(ROOT, "rustane_b200", "generate")
    out = subprocess.run([exe, "--checkpoint", plain, "--convert-to", quant, "--dtype", "int4"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "wrote" in out.stdout, out.stderr[-2000:]
    assert R.checkpoint_info(quant)["quantised_linears"] and os.path.getsize(quant) < os.path.getsize(plain)
    bad = subprocess.run([exe, "--checkpoint", plain, "--convert-to", quant, "--dtype", "bf16"], capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and "--convert-to needs --dtype fp8 or --dtype int4" in bad.stderr
    common = ["--prompt-ids", "5,6,7,8", "--decode-backend", "cuda", "--steps", "10", "--temperature", "0"]
    a = subprocess.run([exe, "--checkpoint", plain, "--dtype", "int4"] + common, capture_output=True, text=True, timeout=300)
    b = subprocess.run([exe, "--checkpoint", quant] + common, capture_output=True, text=True, timeout=300)
    assert a.returncode == 0 and b.returncode == 0, (a.stderr[-1000:], b.stderr[-1000:])
    ids = lambda o: [_ids(l) for l in o.stdout.splitlines() if l.startswith("generated_ids=")]
    assert ids(a) == ids(b) and len(ids(a)[0]) == 10
