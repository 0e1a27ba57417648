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
