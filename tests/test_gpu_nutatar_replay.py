"""A Nutatar folder through the two programs a user runs: `bin/trace_run` (whole, last tokens one by one, a batch
of unequal requests) and `bin/qstream` (greedy generation), against the plain model."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_nutatar as P
from nutatar_util import assert_close, load_plain, make_folder
from util import random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("C", "bfloat16")])
def test_replay_and_command_line(tmp_path, which, dtype):
    folder, cfg = make_folder(tmp_path, which, dtype)
    pcfg, w = load_plain(folder)
    V = cfg["vocab"]
    rng = np.random.default_rng(8)
    reqs = {f"q{i}": random_tokens(rng, n, V) for i, n in enumerate((70, 1, 131))}
    refs = {k: P.forward(pcfg, w, t) for k, t in reqs.items()}
    steps, where = [], {}
    # each alone: whole; then all but the last 5 tokens and those one by one; then all three as one batch
    for k, t in reqs.items():
        steps.append({"step": len(steps), "entries": [{"id": k, "tokens": t, "want": list(range(len(t)))}], "end": [k]})
        where[len(steps) - 1] = [(k, p) for p in range(len(t))]
    t = reqs["q2"]
    steps.append({"step": len(steps), "entries": [{"id": "tail", "tokens": t[:-5], "want": [len(t) - 6]}], "end": []})
    where[len(steps) - 1] = [("q2", len(t) - 6)]
    for p in range(len(t) - 5, len(t)):
        steps.append({"step": len(steps), "entries": [{"id": "tail", "tokens": [t[p]], "want": [0]}], "end": ["tail"] if p == len(t) - 1 else []})
        where[len(steps) - 1] = [("q2", p)]
    prompt = {"q0": 60, "q1": 1, "q2": 100}
    steps.append({"step": len(steps), "end": ["q1"],
                  "entries": [{"id": k + "b", "tokens": reqs[k][:n], "want": [n - 1]} for k, n in prompt.items()]})
    where[len(steps) - 1] = [(k, n - 1) for k, n in prompt.items()]
    for j in range(10):
        steps.append({"step": len(steps), "end": ["q0b"] if j == 9 else [], "entries": [
            {"id": k + "b", "tokens": [reqs[k][prompt[k] + j]], "want": [0] if j % 2 else []} for k in ("q0", "q2")]})
        if j % 2:
            where[len(steps) - 1] = [(k, prompt[k] + j) for k in ("q0", "q2")]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "512"], input=text, text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [x for s in steps for x in ("done", str(s["step"]))]
    for s in steps:
        path = out / f"{s['step']}.f32"
        if s["step"] not in where:
            assert not path.exists()
            continue
        got = np.fromfile(path, dtype="<f4").reshape(-1, V)
        ref = np.stack([refs[k][p] for k, p in where[s["step"]]])
        assert_close(got, ref, dtype, f"step {s['step']}")

    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "qstream"), str(folder), "-p", "5,17,3;1 2 3 4", "-n", "6", "-t", "0",
                           "--dtype", dtype, "--max-ctx", "128", "--stop-token", "none", "--repeat-penalty", "1.0"], text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [[int(x) for x in line.split()] for line in proc.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(line) == 6 for line in lines)
    if dtype == "float32":
        assert lines[0] == P.greedy(pcfg, w, [5, 17, 3], 6) and lines[1] == P.greedy(pcfg, w, [1, 2, 3, 4], 6)
