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


@pytest.mark.parametrize("name", ["D", "E"])
def test_asking_l2_for_what_comes_next_changes_no_bit(engines, folders, name, monkeypatch):
    """Decode steps hand ``ctx.upcoming`` (the weights the step streams next) to their kernels, which ask L2
    for its beginning.  With that switched off, with the usual size and with a size that is no multiple of
    anything, the logits are the same bits."""
    from flashdecode_cuda_b200.parts import attention as A, linear as L
    eng = engines[(name, "bfloat16")]
    reqs = prompts_for(TINY[name]["vocab_size"], [40, 23, 31], seed=9)
    outs = []
    for nbytes, o_bytes in ((0, 0), (L.UPCOMING_BYTES, A.PREFETCH_BYTES), (1000, 1 << 30)):
        monkeypatch.setattr(A, "UPCOMING_BYTES", nbytes)
        monkeypatch.setattr(L, "UPCOMING_BYTES", nbytes)
        monkeypatch.setattr(A, "PREFETCH_BYTES", o_bytes)
        cache = eng.model.new_cache(max_tokens=256, block_size=16)
        slots = [cache.admit() for _ in reqs]
        eng.model.step(cache, slots, [r[:20] for r in reqs], None)
        got = []
        for i in range(20, 23):
            got.append(eng.model.step(cache, slots, [[r[i]] for r in reqs], "last").clone())
        outs.append(torch.stack(got))
        for s_ in slots:
            cache.release(s_)
    eng.model.check_status()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    for j, r in enumerate(reqs):
        assert rel_err(outs[1][2][j], oracle_logits(folders[name], r)[22]) < TOL["bfloat16"]


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


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n_seqs", [("D", 17), ("E", 24), ("E", 33), ("D", 64)])
def test_decode_batches_beyond_16_through_graphs(engines, folders, name, dtype, n_seqs):
    """Decode steps of 17 to 64 sequences of unequal lengths replayed from captured graphs (the buckets above 16,
    whose products are the streaming tcgen05 kernel in bfloat16), with sequences that end earlier, so that
    the batch falls into smaller buckets; every step's logits against the plain implementation."""
    from flashdecode_cuda_b200.engine.decode import GraphDecoder
    eng = engines[(name, dtype)]
    V = TINY[name]["vocab_size"]
    lens = [2 + (37 * i) % 90 for i in range(n_seqs)]
    n_dec = [3 + (5 * i) % 7 for i in range(n_seqs)]                 # tokens fed one by one: 3 .. 9
    reqs = prompts_for(V, [l + k for l, k in zip(lens, n_dec)], seed=31)
    cache = eng.model.new_cache(max_tokens=64 * 3 * n_seqs, block_size=16, max_slots=n_seqs)
    slots = [cache.admit() for _ in reqs]
    eng.model.step(cache, slots, [r[:l] for r, l in zip(reqs, lens)], None)
    dec = GraphDecoder(eng.model, cache)
    live = list(range(n_seqs))
    buckets = set()
    for step in range(max(n_dec)):
        for i in [i for i in live if step >= n_dec[i]]:
            cache.release(slots[i])
        live = [i for i in live if step < n_dec[i]]
        dec.run([slots[i] for i in live], [reqs[i][lens[i] + step] for i in live])
        got = dec.last_logits(len(live)).clone()
        buckets.add(dec.last.ctx.n_rows)
        for j, i in enumerate(live):
            if (i + step) % 3 == 0 or i in (live[0], live[-1]):
                want = oracle_logits(folders[name], reqs[i])[lens[i] + step]
                assert rel_err(got[j], want) < TOL[dtype], f"request {i} step {step} among {len(live)}"
    assert max(buckets) >= n_seqs and len(buckets) >= 2
    for i in live:
        cache.release(slots[i])
    cache.check_invariants()
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "E"])
def test_mixed_steps(engines, folders, name, dtype):
    """Steps in which some sequences bring one token and another brings a prompt, or the next part of a
    prompt: two sequences decode while a third brings its 200 tokens at once, then a fourth its 300 tokens
    as 128 + 172."""
    eng = engines[(name, dtype)]
    V = TINY[name]["vocab_size"]
    a, b, c, d = prompts_for(V, [30, 61, 200, 300], seed=41)
    want = {k: oracle_logits(folders[name], r) for k, r in zip("abcd", (a, b, c, d))}
    cache = eng.model.new_cache(max_tokens=64 * 12, block_size=16, max_slots=4)
    sa, sb, sc, sd = (cache.admit() for _ in range(4))
    pa, pb = 20, 50                                   # tokens of a and b that are in the cache
    eng.model.step(cache, [sa, sb], [a[:pa], b[:pb]], None)

    def check(got, rows):
        for g, (k, p) in zip(got, rows):
            assert rel_err(g, want[k][p]) < TOL[dtype], f"request {k} position {p}"

    # a and b go on by one token each while c brings its whole prompt
    got = eng.model.step(cache, [sa, sc, sb], [[a[pa]], c, [b[pb]]], [[0], [0, 99, 199], [0]])
    check(got, [("a", pa), ("c", 0), ("c", 99), ("c", 199), ("b", pb)])
    # a and b go on while d brings the first 128 tokens of its prompt, then the other 172
    got = eng.model.step(cache, [sd, sa, sb], [d[:128], [a[pa + 1]], [b[pb + 1]]], "last")
    check(got, [("d", 127), ("a", pa + 1), ("b", pb + 1)])
    got = eng.model.step(cache, [sb, sd, sa], [[b[pb + 2]], d[128:], [a[pa + 2]]], [[0], [0, 100, 171], [0]])
    check(got, [("b", pb + 2), ("d", 128), ("d", 228), ("d", 299), ("a", pa + 2)])
    # and a chunk of several tokens for a sequence that already decodes, beside single tokens
    got = eng.model.step(cache, [sa, sb], [a[pa + 3:pa + 8], [b[pb + 3]]], "all")
    check(got, [("a", pa + 3 + i) for i in range(5)] + [("b", pb + 3)])
    eng.model.check_status()
    cache.check_invariants()


def test_float32_decode_does_not_depend_on_the_batch(engines, folders):
    """In float32 a decoded token's logits are the same bits alone and in a batch of eight with longer
    neighbours: the keys are cut into splits of a fixed length, whatever else is in the step."""
    eng = engines[("D", "float32")]
    V = TINY["D"]["vocab_size"]
    reqs = prompts_for(V, [600, 900, 300, 14, 610, 1000, 257, 512], seed=51)
    cache = eng.model.new_cache(max_tokens=64 * 70, block_size=16, max_slots=9)
    s = cache.admit()
    eng.model.step(cache, [s], [reqs[0][:590]], None)
    alone = [eng.model.step(cache, [s], [[reqs[0][590 + i]]], "last").clone() for i in range(4)]
    assert rel_err(alone[3][0], oracle_logits(folders["D"], reqs[0])[593]) < TOL["float32"]
    cache.release(s)
    slots = [cache.admit() for _ in reqs]
    heads = [len(r) - 10 for r in reqs]
    eng.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], None)
    order = [3, 5, 0, 1, 2, 4, 6, 7]
    for i in range(4):
        got = eng.model.step(cache, [slots[j] for j in order], [[reqs[j][heads[j] + i]] for j in order], "last")
        assert torch.equal(got[2], alone[i][0]), f"decoded token {i}"
    eng.model.check_status()


REAL_WIDTHS = {
    # the layer sizes of the three presets (two layers each, the whole vocabulary): groups of 6, 7 and 5 query heads
    "qwen2.5-1.5b": [40, 33, 140],
    "qwen2.5-7b": [40, 25, 37],
    "qwen2.5-14b": [40, 19, 31],
}


@pytest.mark.parametrize("preset", list(REAL_WIDTHS))
def test_two_layers_at_real_widths(preset):
    """Two layers at the real widths of a preset with its whole vocabulary, in bfloat16: prompts in one
    unequal batch (one of them longer than a 128-row tile at the smallest preset), then eight tokens one by
    one, against the plain implementation (layers in float64 on the CPU; the output head, whose matrix alone is
    gigabytes in float64, as one float64 product on the GPU)."""
    from flashdecode_cuda_b200.config import config_from_dict, preset_dict
    from flashdecode_cuda_b200.engine import Model, random_weights
    from plain import qwen2_plain as P
    raw = preset_dict(preset)
    raw["num_hidden_layers"] = 2
    if "max_window_layers" in raw:
        raw["max_window_layers"] = min(raw["max_window_layers"], 2)
    cfg = config_from_dict(raw)
    model = Model.from_config(cfg, torch.bfloat16, "cuda")
    tensors = random_weights(model, 5, torch.bfloat16, device="cuda")
    model.bind(tensors)
    V = cfg.vocab_size
    lens = REAL_WIDTHS[preset]
    reqs = prompts_for(V, [l + 8 for l in lens], seed=61)

    head = tensors.get("lm_head.weight", tensors["model.embed_tokens.weight"]).double()      # on the GPU

    layers = {k: v.cpu().double() for k, v in tensors.items() if k not in ("lm_head.weight", "model.embed_tokens.weight")}

    def plain_logits(tokens, rows):
        ids = sorted(set(tokens))                    # only the rows of the embedding table that the request uses
        small = dict(layers)
        small["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"][torch.tensor(ids, device="cuda")].cpu().double()
        hn = P.hidden_states(raw, small, [ids.index(t) for t in tokens])
        return (hn[rows].cuda() @ head.T).cpu()

    cache = model.new_cache(max_tokens=64 * 8, block_size=16, max_slots=3)
    slots = [cache.admit() for _ in reqs]
    got = [model.step(cache, slots, [r[:l] for r, l in zip(reqs, lens)], "last").clone()]
    for i in range(8):
        got.append(model.step(cache, slots, [[r[l + i]] for r, l in zip(reqs, lens)], "last").clone())
    model.check_status()
    got = torch.stack(got)                                    # [9, 3, V]
    for j, (r, l) in enumerate(zip(reqs, lens)):
        want = plain_logits(r, list(range(l - 1, l + 8)))
        assert rel_err(got[:, j], want) < TOL["bfloat16"], f"request {j}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "E"])
def test_trace_of_every_layer(engines, folders, name, dtype, monkeypatch):
    """``Model.trace = {}`` records the embedding and the residual stream after every layer; each tensor
    against the plain implementation's trace of the same name, in execution order, so that the first
    difference names the layer (the manner of testing/diff.py:98-122 of the reference).  With the trace off
    (the default) a step records nothing and copies nothing to the host."""
    from helpers import raw_config, weights_of
    from plain import qwen2_plain as P
    eng = engines[(name, dtype)]
    model = eng.model
    (p,) = prompts_for(TINY[name]["vocab_size"], [150], seed=71)
    want = {}
    P.hidden_states(raw_config(folders[name]), weights_of(folders[name]), p, trace=want)
    cache = model.new_cache(max_tokens=256, block_size=16)
    slot = cache.admit()
    assert model.trace is None
    copies = []
    real_cpu = torch.Tensor.cpu
    monkeypatch.setattr(torch.Tensor, "cpu", lambda t, *a, **k: (copies.append(1), real_cpu(t, *a, **k))[1])
    model.step(cache, [slot], [p[:100]], None)
    assert model.trace is None and not copies                    # off: nothing recorded, nothing read back
    monkeypatch.undo()
    cache.release(slot)
    slot = cache.admit()
    model.trace = {}
    try:
        model.step(cache, [slot], [p], "last")
        got = model.trace
    finally:
        model.trace = None
    names = ["embed"] + [f"layer.{i}" for i in range(TINY[name]["num_hidden_layers"])]
    assert list(got) == names and list(want) == names
    tol = {"float32": 2e-5, "bfloat16": 2e-2}[dtype]
    for n in names:                                              # the first failing name is the layer to look at
        assert rel_err(got[n], want[n]) < tol, f"first difference at {n}"
    # decode steps record too (one row per sequence): the last layer of the next token
    model.trace = {}
    try:
        model.step(cache, [slot], [[p[-1]]], "last")
        assert model.trace["layer.0"].shape == (1, TINY[name]["hidden_size"])
    finally:
        model.trace = None
    model.check_status()
