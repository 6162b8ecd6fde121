"""The plain implementation itself: against logits of the reference's own
engine (committed under tests/golden/, made by tests/golden/make_golden.py),
and against closed forms of its parts."""

import json
import math
from pathlib import Path

import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.weights import load_checkpoint, read_file
from helpers import TINY
from plain import qwen2_plain as P

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_matches_the_reference_engine(tmp_path):
    golden = read_file(GOLDEN / "reference_logits.safetensors")
    meta = json.loads((GOLDEN / "reference_logits.json").read_text())
    seen = 0
    for name, info in meta.items():
        folder = fd.write_random_model(tmp_path / name, TINY[name], info["seed"])
        weights = load_checkpoint(folder)
        for i, prompt in enumerate(info["prompts"]):
            mine = P.logits(TINY[name], weights, prompt, dtype=torch.float32)
            for key, row in golden.items():
                case, idx, kind, n = key.split(".")
                if case != name or int(idx) != i:
                    continue
                pos = int(n) - 1 if kind == "prefill" else int(n)
                assert torch.allclose(mine[pos], row, atol=2e-5, rtol=0), key
                seen += 1
    assert seen == len(golden) > 50


def test_rmsnorm_closed_form():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    out = P.rmsnorm(x, torch.tensor([2.0, 0.5], dtype=torch.float64), 0.0)
    rms = math.sqrt((9 + 16) / 2)
    assert torch.allclose(out, torch.tensor([[2 * 3 / rms, 0.5 * 4 / rms]], dtype=torch.float64))


def test_rope_pairs_j_with_j_plus_half():
    cos, sin = P.rope_tables(4, 3, 10000.0)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]]).repeat(3, 1, 1)
    y = P.apply_rope(x, cos, sin)
    assert torch.allclose(y[0], x[0])                                  # position 0: no rotation
    a0, a1 = 1.0, 1.0 / 10000.0 ** 0.5                                 # angles of position 1
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)]
    assert torch.allclose(y[1, 0], torch.tensor(want), atol=1e-6)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)   # a rotation keeps the norm


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(6, n, 8, generator=g, dtype=torch.float64) for n in (4, 2, 2))
    out = P.causal_gqa_attention(q, k, v, 0.3, None)
    assert torch.allclose(out[0, 3], v[0, 1])                          # the first token sees itself only; head 3 -> kv head 1
    k2, v2 = k.clone(), v.clone()
    k2[5], v2[5] = 9.0, -9.0                                            # the future does not leak back
    assert torch.allclose(P.causal_gqa_attention(q, k2, v2, 0.3, None)[:5], out[:5])
    w1 = P.causal_gqa_attention(q, k, v, 0.3, 1)                        # a window of 1: every token sees itself only
    assert torch.allclose(w1[:, 0], v[:, 0]) and torch.allclose(w1[:, 2], v[:, 1])
    w3 = P.causal_gqa_attention(q, k, v, 0.3, 3)
    assert torch.allclose(w3[:3], out[:3]) and not torch.allclose(w3[5], out[5])


def test_window_layers_follow_the_config():
    cfg = TINY["C"]
    assert [P.layer_window(cfg, i) for i in range(4)] == [None, None, 24, 24]
    assert P.layer_window(TINY["A"], 1) is None


def test_philox_known_answer_and_sampling():
    # Random123 known-answer vectors for philox4x32-10
    assert P.philox4x32((0, 0, 0, 0), (0, 0)) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert P.philox4x32((0xffffffff,) * 4, (0xffffffff, 0xffffffff)) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    row = torch.tensor([0.1, 2.0, 2.0, -1.0])
    assert P.sample(row, 0.0, 0, 0, 0) == 1                             # ties: the lowest index
    draws = [P.sample(row, 1.0, 3, r, 0) for r in range(300)]
    freq = torch.bincount(torch.tensor(draws), minlength=4).double() / 300
    assert float((freq - torch.softmax(row.double(), 0)).abs().max()) < 0.08
    assert P.sample(row, 1.0, 3, 5, 2) == P.sample(row, 1.0, 3, 5, 2)
    g = P.gumbel_noise(9, 1, 2, 3)
    assert torch.isfinite(g).all()
