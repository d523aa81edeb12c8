"""bin/trace_run as a program: a short trace through its command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import (model_dir, plain_logits, rel_err, trace_batches, write_trace)
from tiny import TINY, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-6), ("bfloat16", 2e-2)])
def test_trace_run(tmp_path, dtype, tol):
    rng = np.random.default_rng(21)
    v = TINY["B"]["vocab_size"]
    batch = [(tokens(rng, 40, v), 30), (tokens(rng, 9, v), 2), (tokens(rng, 70, v), 66)]
    steps = trace_batches([batch], want_prompt_all=False)
    steps[1]["entries"][0]["want"] = []            # a step may want nothing of a request
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
                        model_dir("B"), "--dtype", dtype, "--out", str(out), "--max-tokens",
                        "256"], stdin=open(trace), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    pos = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        path = out / f"{st['step']}.f32"
        if n_want == 0:
            assert not path.exists()
            continue
        got = np.fromfile(path, dtype="<f4").reshape(n_want, v)
        row = 0
        for e in st["entries"]:
            i = int(e["id"][3:])
            base = pos.get(e["id"], 0)
            for w_ in e["want"]:
                want = plain_logits("B", batch[i][0])[base + w_]
                assert rel_err(got[row], want) <= tol, (st["step"], e["id"])
                row += 1
            pos[e["id"]] = base + len(e["tokens"])


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
def test_trace_run_zuzelorn(tmp_path, dtype, tol):
    """The same program on a model of the Zuzelorn design: the class is chosen by config.json."""
    import plain_zuzelorn as pz
    from zuzelorn_models import model
    folder, c, w = model("ZA")
    rng = np.random.default_rng(22)
    v = c["vocab"]
    batch = [(tokens(rng, 140, v), 131), (tokens(rng, 3, v), 1), (tokens(rng, 66, v), 64)]
    steps = trace_batches([batch], want_prompt_all=False)
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    # 140 + 3 + 66 tokens are alive at once: the runner makes room for the pages' slack itself
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", str(out), "--max-tokens", "209"],
                       stdin=open(trace), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    plain = [pz.forward(c, w, t, None if dtype == "float32" else "bfloat16").numpy() for t, _ in batch]
    pos = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        got = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(n_want, v)
        row = 0
        for e in st["entries"]:
            i = int(e["id"][3:])
            base = pos.get(e["id"], 0)
            for w_ in e["want"]:
                assert rel_err(got[row], plain[i][base + w_]) <= tol, (st["step"], e["id"])
                row += 1
            pos[e["id"]] = base + len(e["tokens"])


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 5e-2)])
def test_trace_run_dunavik(tmp_path, dtype, tol):
    """The same program on a model of the Dunavik design (latent rows in the cache, repeated passes),
    and the command line's generation on the same folder."""
    import plain_dunavik as pd
    from dunavik_models import model
    folder, c, w = model("DA")
    rng = np.random.default_rng(23)
    v = c["vocab"]
    batch = [(tokens(rng, 150, v), 131), (tokens(rng, 3, v), 1), (tokens(rng, 66, v), 64)]
    steps = trace_batches([batch], want_prompt_all=False)
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", str(out), "--max-tokens", "219"],
                       stdin=open(trace), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    plain = [pd.forward(c, w, t, None if dtype == "float32" else "bfloat16").numpy() for t, _ in batch]
    pos = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        got = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(n_want, v)
        row = 0
        for e in st["entries"]:
            i = int(e["id"][3:])
            base = pos.get(e["id"], 0)
            for w_ in e["want"]:
                assert rel_err(got[row], plain[i][base + w_]) <= tol, (st["step"], e["id"])
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    if dtype == "float32":
        # greedy generation through the command line: the plain model's own choices
        prompt = batch[2][0][:20]
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "janas-b200"), folder, "--tokens",
                            " ".join(map(str, prompt)), "--max", "6", "--dtype", "float32"],
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        import torch
        seq = list(prompt)
        for _ in range(6):
            lg = pd.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]) < 1e-4 * lg.abs().max():
                break                                   # a tie within rounding: stop comparing
            seq.append(int(lg.argmax()))
        assert len(seq) > 21 and " ".join(map(str, seq[20:])) in r.stdout, r.stdout[-500:]


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 5e-2)])
def test_trace_run_kefesun(tmp_path, dtype, tol):
    """The same program on a model of the Kefesun design (recurrent state and the convolutions' last
    inputs in the cache's slots, a window with kept first tokens, a routed feed-forward),
    and the command line's generation on the same folder."""
    import plain_kefesun as pd
    from kefesun_models import model
    folder, c, w = model("KA")
    rng = np.random.default_rng(23)
    v = c["vocab"]
    batch = [(tokens(rng, 150, v), 131), (tokens(rng, 3, v), 1), (tokens(rng, 66, v), 64)]
    steps = trace_batches([batch], want_prompt_all=False)
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", str(out), "--max-tokens", "219"],
                       stdin=open(trace), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    plain = [pd.forward(c, w, t, None if dtype == "float32" else "bfloat16").numpy() for t, _ in batch]
    pos = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        got = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(n_want, v)
        row = 0
        for e in st["entries"]:
            i = int(e["id"][3:])
            base = pos.get(e["id"], 0)
            for w_ in e["want"]:
                assert rel_err(got[row], plain[i][base + w_]) <= tol, (st["step"], e["id"])
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    if dtype == "float32":
        # greedy generation through the command line: the plain model's own choices
        prompt = batch[2][0][:20]
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "janas-b200"), folder, "--tokens",
                            " ".join(map(str, prompt)), "--max", "6", "--dtype", "float32"],
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        import torch
        seq = list(prompt)
        for _ in range(6):
            lg = pd.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]) < 1e-4 * lg.abs().max():
                break                                   # a tie within rounding: stop comparing
            seq.append(int(lg.argmax()))
        assert len(seq) > 21 and " ".join(map(str, seq[20:])) in r.stdout, r.stdout[-500:]


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 5e-2)])
def test_trace_run_munisun(tmp_path, dtype, tol):
    """The same program on a model of the Munisun design: pages for the attention side, a state row per
    request for the convolutions and the recurrences, a batch of unequal requests decoded together,
    and the command line's generation on the same folder."""
    import plain_munisun as pm
    from munisun_models import model
    folder, c, w = model("MD")
    rng = np.random.default_rng(25)
    v = c["vocab"]
    batch = [(tokens(rng, 140, v), 131), (tokens(rng, 3, v), 1), (tokens(rng, 66, v), 64)]
    steps = trace_batches([batch], want_prompt_all=False)
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", str(out), "--max-tokens", "209"],
                       stdin=open(trace), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    plain = [pm.forward(c, w, t, None if dtype == "float32" else "bfloat16").numpy() for t, _ in batch]
    pos = {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        got = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(n_want, v)
        row = 0
        for e in st["entries"]:
            i = int(e["id"][3:])
            base = pos.get(e["id"], 0)
            for w_ in e["want"]:
                assert rel_err(got[row], plain[i][base + w_]) <= tol, (st["step"], e["id"])
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    if dtype == "float32":
        # greedy generation through the command line: the plain model's own choices
        prompt = batch[2][0][:20]
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "janas-b200"), folder, "--tokens",
                            " ".join(map(str, prompt)), "--max", "6", "--dtype", "float32"],
                           capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        import torch
        seq = list(prompt)
        for _ in range(6):
            lg = pm.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            if (top[0] - top[1]) < 1e-4 * lg.abs().max():
                break                                   # a tie within rounding: stop comparing
            seq.append(int(lg.argmax()))
        assert len(seq) > 21 and " ".join(map(str, seq[20:])) in r.stdout, r.stdout[-500:]
