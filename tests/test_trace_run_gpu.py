"""bin/trace_run as a user runs it: the same requests whole, with the last 32
tokens one by one, and in batches of unequal lengths whose shorter requests end
earlier, one batch after another; float32 and bfloat16; against the plain
implementation."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import TINY, TOL, oracle_logits, prompts_for, rel_err, write_folder

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def build_trace(reqs):
    """(steps, expectations): expectations[step] = list of (request, position) in file order."""
    steps, expect = [], {}
    n = 0

    def add(entries, end):
        nonlocal n
        steps.append({"step": n, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w, _ in entries], "end": end})
        exp = [(r, p) for _, _, w, pos in entries for r, p in pos]
        if exp:
            expect[n] = exp
        n += 1

    # 1. each request alone and whole, logits everywhere
    for r, toks in enumerate(reqs):
        add([(f"w{r}", toks, list(range(len(toks))), [(r, p) for p in range(len(toks))])], [f"w{r}"])
    # 2. each request alone: all but the last 32 tokens, then one by one
    for r, toks in enumerate(reqs):
        head = len(toks) - 32
        add([(f"t{r}", toks[:head], [head - 1], [(r, head - 1)])], [])
        for p in range(head, len(toks)):
            add([(f"t{r}", [toks[p]], [0], [(r, p)])], [f"t{r}"] if p == len(toks) - 1 else [])
    # 3. two batches of unequal lengths; every request is cut so that its last k tokens are decoded
    for batch_no, members in enumerate([[0, 1, 2], [2, 0]]):
        tails = {0: 5, 1: 12, 2: 2}
        heads = {r: len(reqs[r]) - tails[r] for r in members}
        ids = {r: f"b{batch_no}_{r}" for r in members}
        add([(ids[r], reqs[r][:heads[r]], [heads[r] - 1], [(r, heads[r] - 1)]) for r in members], [])
        for s in range(max(tails[r] for r in members)):
            live = [r for r in members if s < tails[r]]
            done = [ids[r] for r in live if s == tails[r] - 1]
            add([(ids[r], [reqs[r][heads[r] + s]], [0], [(r, heads[r] + s)]) for r in live], done)
    # 4. a step in which nothing is wanted, and an empty step
    add([("n0", reqs[0][:4], [], [])], ["n0"])
    add([], [])
    return steps, expect


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths", [("C", [40, 75, 33]), ("E", [140, 300, 70])])
def test_replay(tmp_path, dtype, name, lengths):
    """C: odd sizes (the CUDA-core attention in both dtypes).  E: head size 128, a window on one layer and
    prompts longer than a 128-row tile (in bfloat16 the tcgen05 products and attention, the tensor-core decode
    attention and the weight-streaming decode products)."""
    folder = write_folder(tmp_path, name, seed=9)
    V = TINY[name]["vocab_size"]
    reqs = prompts_for(V, lengths, seed=12)
    steps, expect = build_trace(reqs)
    out_dir = tmp_path / f"out_{dtype}"
    # live tokens at any time: at most three requests, each rounded up to a multiple of 64
    max_tokens = sum(-(-len(r) // 64) * 64 for r in reqs)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    files = sorted(int(p.stem) for p in out_dir.glob("*.f32"))
    assert files == sorted(expect)                    # a file exactly for the steps that want something
    import hashlib
    manifest = json.loads((out_dir / "manifest.json").read_text())
    assert manifest["config_sha256"] == hashlib.sha256((folder / "config.json").read_bytes()).hexdigest()
    assert manifest["dtype"] == dtype and manifest["vocab_size"] == V and manifest["steps"] == len(steps)
    assert [(f["step"], f["rows"]) for f in manifest["files"]] == [(st, len(expect[st])) for st in sorted(expect)]
    worst = 0.0
    for step, exp in expect.items():
        got = torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(len(exp), V))
        for row, (r, p) in zip(got, exp):
            err = rel_err(row, oracle_logits(folder, reqs[r])[p])
            worst = max(worst, err)
            assert err < TOL[dtype], f"step {step}, request {r}, position {p}"
    print(f"{dtype}: worst relative error {worst:.2e}")
