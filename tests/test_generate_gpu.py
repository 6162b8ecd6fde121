"""Generation through the Python entry point and the command line, against the
plain implementation."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import flashdecode_cuda_b200 as fd
from helpers import TINY, TOL, oracle_logits, prompts_for, raw_config, weights_of, write_folder
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen")
    return {n: write_folder(tmp, n, seed=5) for n in ("B", "C")}


@pytest.mark.parametrize("name", ["B", "C"])
def test_greedy_float32_equals_the_plain_implementation(folders, name):
    eng = fd.load(folders[name], device="cuda", dtype="float32")
    raw, w = raw_config(folders[name]), weights_of(folders[name])
    prompts = prompts_for(raw["vocab_size"], [3, 14, 1, 30, 9], seed=1)
    want = [P.generate(raw, w, p, 12) for p in prompts]
    got = eng.generate(prompts, 12, max_batch=3)            # 5 requests, 3 at a time: two batches on one cache
    assert [r.tokens for r in got] == want
    assert all(r.finish_reason == "length" for r in got)
    eng.model.check_status()
    # the reference's form: a [B, S] tensor in, a [B, max_new_tokens] tensor out (engine/model.py:315-329)
    same_len = prompts_for(raw["vocab_size"], [7, 7], seed=2)
    out = eng.generate(torch.tensor(same_len), 6)
    assert out.shape == (2, 6) and out.tolist() == [P.generate(raw, w, p, 6) for p in same_len]


@pytest.mark.parametrize("name", ["B", "C"])
def test_greedy_bfloat16_picks_a_best_token(folders, name):
    """In bfloat16 near-ties may fall the other way: every chosen token must be
    a best one of the plain implementation up to the bfloat16 tolerance."""
    eng = fd.load(folders[name], device="cuda", dtype="bfloat16")
    raw = raw_config(folders[name])
    prompts = prompts_for(raw["vocab_size"], [5, 21, 2], seed=3)
    got = eng.generate(prompts, 10)
    for p, r in zip(prompts, got):
        assert len(r.tokens) == 10
        full = p + r.tokens
        ref = oracle_logits(folders[name], full[:-1])
        scale = float(ref.abs().max())
        for i, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 2 * TOL["bfloat16"] * scale, f"token {i}"


def test_temperature_stop_tokens_and_early_end(folders):
    eng = fd.load(folders["B"], device="cuda", dtype="float32")
    raw, w = raw_config(folders["B"]), weights_of(folders["B"])
    prompts = prompts_for(raw["vocab_size"], [4, 9, 2], seed=4)
    want = [P.generate(raw, w, p, 8, temperature=0.8, seed=77, request=i) for i, p in enumerate(prompts)]
    got = eng.generate(prompts, 8, temperature=0.8, seed=77)
    assert [r.tokens for r in got] == want
    assert len({tuple(t) for t in want}) == 3
    # a request's draws do not depend on its batch: alone it gives the same tokens
    cache = eng.new_paged_cache(1, 64)
    eng.cache, eng.seed = cache, 77
    from flashdecode_cuda_b200.engine.generate import GenerationLoop, Request
    alone = GenerationLoop(eng, 1).run([Request(prompts[1], 8, 0.8, (), request_id=1)])
    assert alone[0].tokens == want[1]
    # the stop token ends its sequence at once and is kept; the others go on
    stop = want[0][2]
    got = eng.generate(prompts, 8, temperature=0.8, seed=77, stop_token_ids=[stop])
    for r, full in zip(got, want):
        cut = full.index(stop) + 1 if stop in full else len(full)
        assert r.tokens == full[:cut]
        assert r.finish_reason == ("stop" if stop in full else "length")
    assert got[0].finish_reason == "stop" and len(got[0].tokens) == 3
    # another seed, also one beyond 63 bits: other draws, through the graphs captured for the first seed
    n_graphs = len(eng._decoder().graphs)
    for seed in (78, (1 << 63) + 5):
        want2 = [P.generate(raw, w, p, 8, temperature=0.8, seed=seed, request=i) for i, p in enumerate(prompts)]
        assert [r.tokens for r in eng.generate(prompts, 8, temperature=0.8, seed=seed)] == want2
        assert want2 != want
    assert len(eng._decoder().graphs) == n_graphs
    eng.model.check_status()


def test_graph_replay_equals_eager_steps(folders):
    """Decode steps replayed from CUDA graphs give the tokens of eager steps."""
    eng = fd.load(folders["C"], device="cuda", dtype="bfloat16")
    prompts = prompts_for(TINY["C"]["vocab_size"], [6, 40, 17], seed=6)
    assert eng.use_graphs
    a = [r.tokens for r in eng.generate(prompts, 40)]
    eng.use_graphs = False
    b = [r.tokens for r in eng.generate(prompts, 40)]
    assert a == b


def test_new_sequences_in_the_same_slots_of_the_same_graph(folders):
    """The decoder fills in the next step's slots and lengths while a step runs.  When the
    sequences end instead and new ones start in the same slots, in the same order, with the
    same graph, what it filled in is stale and must not be used."""
    from flashdecode_cuda_b200.engine.decode import GraphDecoder
    eng = fd.load(folders["B"], device="cuda", dtype="float32")
    raw, w = raw_config(folders["B"]), weights_of(folders["B"])
    model = eng.model
    cache = model.new_cache(max_tokens=256, block_size=8)
    dec = GraphDecoder(model, cache)

    def run(prompts, n_new):
        slots = [cache.admit() for _ in prompts]
        toks = eng.sampler.sample(model.step(cache, slots, prompts, "last")).tolist()
        out = [[t] for t in toks]
        for _ in range(n_new - 1):
            dec.run(slots, toks)
            toks = dec.read_tokens(len(slots))
            for o, t in zip(out, toks):
                o.append(t)
        for s in reversed(slots):            # the allocator hands the last freed slot out first
            cache.release(s)
        return slots, out

    first = prompts_for(raw["vocab_size"], [9, 4], seed=11)
    second = prompts_for(raw["vocab_size"], [3, 17], seed=12)
    slots_a, got_a = run(first, 6)
    slots_b, got_b = run(second, 6)
    assert slots_a == slots_b and len(dec.graphs) == 1      # the case this test is about
    assert got_a == [P.generate(raw, w, p, 6) for p in first]
    assert got_b == [P.generate(raw, w, p, 6) for p in second]
    model.check_status()


def test_engine_uses_a_decoder_it_is_given(folders):
    """``Engine.use_decoder``: generation over a decoder's cache goes through that decoder and the graphs it has
    captured - none is captured anew - and a decoder's length bounds are powers of two."""
    from flashdecode_cuda_b200.engine.decode import GraphDecoder, KV_BOUND_MIN
    eng = fd.load(folders["B"], device="cuda", dtype="float32")
    raw, w = raw_config(folders["B"]), weights_of(folders["B"])
    model = eng.model
    cache = model.new_cache(batch_size=2, max_len=128, block_size=8)
    dec = GraphDecoder(model, cache)
    assert dec._key(2, 5, True, 0)[1] == min(KV_BOUND_MIN, cache.max_len)
    import types
    probe = GraphDecoder(model, cache)
    probe.cache = types.SimpleNamespace(max_len=5000)        # _key reads nothing else of the cache
    bounds = [probe._key(1, n, True, 0)[1] for n in (1, 1024, 1025, 2048, 2049, 4096, 4097, 5000)]
    assert bounds == [1024, 1024, 2048, 2048, 4096, 4096, 5000, 5000]
    prompts = prompts_for(raw["vocab_size"], [9, 4], seed=21)
    slots = [cache.admit() for _ in prompts]
    toks = eng.sampler.sample(model.step(cache, slots, prompts, "last")).tolist()
    dec.run(slots, toks)                                     # captures the graph of this bucket and bound
    for s_ in slots:
        cache.release(s_)
    captured = dict(dec.graphs)
    eng.use_decoder(dec)
    got = [r.tokens for r in eng.generate(prompts, 6, cache)]
    assert got == [P.generate(raw, w, p, 6) for p in prompts]
    assert eng._decoder() is dec and dec.graphs == captured      # the same graphs, none added
    other = fd.load(folders["C"], device="cuda", dtype="float32")
    with pytest.raises(ValueError, match="another model"):
        other.use_decoder(dec)
    model.check_status()


def test_engine_keeps_its_cache_and_graphs_between_calls(folders):
    """A call that is given no cache makes one; the next call uses it again if it is large enough and empty, and with
    it the decode graphs captured over it; a call that needs more gets a new one."""
    eng = fd.load(folders["B"], device="cuda", dtype="float32")
    raw, w = raw_config(folders["B"]), weights_of(folders["B"])
    first = prompts_for(raw["vocab_size"], [9, 4, 12], seed=31)
    second = prompts_for(raw["vocab_size"], [5, 7], seed=32)
    assert [r.tokens for r in eng.generate(first, 8)] == [P.generate(raw, w, p, 8) for p in first]
    cache, dec = eng.cache, eng._decoder()
    graphs = dict(dec.graphs)
    assert graphs
    assert [r.tokens for r in eng.generate(second, 6)] == [P.generate(raw, w, p, 6) for p in second]
    assert eng.cache is cache and eng._decoder() is dec and not cache.active_slots()
    longer = prompts_for(raw["vocab_size"], [30], seed=33)
    assert [r.tokens for r in eng.generate(longer, 20)] == [P.generate(raw, w, p, 20) for p in longer]
    assert eng.cache is not cache                      # 50 tokens did not fit the first cache's longest sequence
    eng.model.check_status()


def test_command_line(folders, tmp_path):
    cmd = [sys.executable, "-m", "flashdecode_cuda_b200", "generate", "--model", str(folders["B"]),
           "--prompt-ids", "5,6,7", "--prompt-ids", "300,2", "--max-new-tokens", "5", "--dtype", "float32",
           "--block-size", "8"]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [json.loads(l) for l in out.stdout.strip().splitlines()]
    raw, w = raw_config(folders["B"]), weights_of(folders["B"])
    assert [l["tokens"] for l in lines] == [P.generate(raw, w, p, 5) for p in ([5, 6, 7], [300, 2])]
    made = tmp_path / "made"
    cmd = [sys.executable, "-m", "flashdecode_cuda_b200", "random-weights", "--config", "tiny-a", "--seed", "3",
           "--out", str(made)]
    assert subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=120).returncode == 0
    assert (made / "config.json").exists() and (made / "model.safetensors").exists()
