"""The engine against the plain implementation, on the GPU, in float32 and
bfloat16: whole requests, the last tokens one by one, unequal batches whose
shorter requests end earlier with slots used again, long decoding, first
tokens."""

import pytest
import torch

import flashdecode_cuda_b200 as fd
from helpers import TINY, TOL, oracle_logits, prompts_for, rel_err, write_folder

pytestmark = pytest.mark.gpu

CONFIGS = ["A", "B", "C", "D", "E"]
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {name: write_folder(tmp, name, seed=11) for name in CONFIGS}


@pytest.fixture(scope="module")
def engines(folders):
    return {(n, d): fd.load(folders[n], device="cuda", dtype=d) for n in CONFIGS for d in DTYPES}


def _lengths(name):
    return {"A": [5, 11, 17, 64], "B": [1, 7, 16, 33, 100], "C": [3, 24, 25, 49, 130], "D": [2, 63, 64, 65, 200],
            "E": [3, 128, 129, 300]}[name]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
@pytest.mark.parametrize("block_size", [4, 16])
def test_each_request_alone_and_whole(engines, folders, name, dtype, block_size):
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=-(-max(_lengths(name)) // 64) * 64, block_size=block_size)
    for p in prompts_for(TINY[name]["vocab_size"], _lengths(name), seed=1):
        slot = cache.admit()
        got = eng.model.step(cache, [slot], [p], "all")
        assert rel_err(got, oracle_logits(folders[name], p)) < TOL[dtype]
        cache.release(slot)
    eng.model.check_status()
    cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_last_32_tokens_one_by_one(engines, folders, name, dtype):
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=256, block_size=16)
    for p in prompts_for(TINY[name]["vocab_size"], [33, 70, 127], seed=2):
        want = oracle_logits(folders[name], p)
        slot = cache.admit()
        head = len(p) - 32
        got = eng.model.step(cache, [slot], [p[:head]], "last")
        assert rel_err(got[0], want[head - 1]) < TOL[dtype]
        for i in range(head, len(p)):
            got = eng.model.step(cache, [slot], [[p[i]]], "last")
            assert rel_err(got[0], want[i]) < TOL[dtype], f"decoded token {i - head} of a {len(p)}-token request"
        cache.release(slot)
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_unequal_batches_one_after_another(engines, folders, name, dtype):
    """Batches of unequal lengths; prompts in one step, then one token each;
    shorter requests end earlier; the next batch reuses slots and blocks."""
    eng = engines[(name, dtype)]
    V = TINY[name]["vocab_size"]
    cache = eng.model.new_cache(max_tokens=64 * 6, block_size=8, max_slots=4)
    for batch_no, lengths in enumerate([[9, 30, 17, 44], [40, 3, 21], [5, 5, 62, 13]]):
        reqs = prompts_for(V, lengths, seed=10 + batch_no)
        decode = [min(k, len(p) - 1) for k, p in zip([6, 14, 2, 9], reqs)]   # tokens of each request fed one by one
        slots = [cache.admit() for _ in reqs]
        live = list(range(len(reqs)))
        heads = [len(p) - k for p, k in zip(reqs, decode)]
        got = eng.model.step(cache, slots, [p[:h] for p, h in zip(reqs, heads)], "last")
        for j, i in enumerate(live):
            assert rel_err(got[j], oracle_logits(folders[name], reqs[i])[heads[i] - 1]) < TOL[dtype]
        for step in range(max(decode)):
            done = [i for i in live if step >= decode[i]]
            for i in done:
                cache.release(slots[i])
            live = [i for i in live if step < decode[i]]
            got = eng.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + step]] for i in live], "last")
            for j, i in enumerate(live):
                want = oracle_logits(folders[name], reqs[i])[heads[i] + step]
                assert rel_err(got[j], want) < TOL[dtype], f"batch {batch_no} request {i} step {step}"
        for i in live:
            cache.release(slots[i])
        cache.check_invariants()
        assert cache.blocks_in_use() == [0] * len(cache.groups)
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C", "D", "E"])
def test_long_decoding(engines, folders, name, dtype):
    """Two tokens of prompt, then 200 decoded one by one in a batch of two."""
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=512, block_size=16)
    reqs = prompts_for(TINY[name]["vocab_size"], [202, 150], seed=5)
    slots = [cache.admit(), cache.admit()]
    eng.model.step(cache, slots, [r[:2] for r in reqs], None)
    for i in range(2, 202):
        live = [j for j in range(2) if i < len(reqs[j])]
        got = eng.model.step(cache, [slots[j] for j in live], [[reqs[j][i]] for j in live], "last")
        if i % 7 == 0 or i > 195:
            for k, j in enumerate(live):
                assert rel_err(got[k], oracle_logits(folders[name], reqs[j])[i]) < TOL[dtype], f"position {i}"
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_first_tokens_of_a_sequence(engines, folders, name, dtype):
    """A one-token prompt, then every following token alone."""
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=64, block_size=4)
    (p,) = prompts_for(TINY[name]["vocab_size"], [12], seed=8)
    want = oracle_logits(folders[name], p)
    slot = cache.admit()
    for i, t in enumerate(p):
        got = eng.model.step(cache, [slot], [[t]], "all")
        assert rel_err(got[0], want[i]) < TOL[dtype], f"token {i}"
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_neighbours_change_nothing(engines, folders, dtype):
    """A request's logits are the same alone and among others (float32: to the bit)."""
    eng = engines[("B", dtype)]
    cache = eng.model.new_cache(max_tokens=512, block_size=16)
    reqs = prompts_for(TINY["B"]["vocab_size"], [20, 9, 41], seed=3)
    s = cache.admit()
    alone = eng.model.step(cache, [s], [reqs[0]], "all").clone()
    cache.release(s)
    slots = [cache.admit() for _ in reqs]
    together = eng.model.step(cache, [slots[2], slots[0], slots[1]], [reqs[2], reqs[0], reqs[1]], "all")
    mine = together[len(reqs[2]):len(reqs[2]) + len(reqs[0])]
    if dtype == "float32":
        assert torch.equal(alone, mine)
    else:
        assert rel_err(mine, alone) < TOL[dtype]
