"""Each part alone against the plain function of the same name, and two toy
architectures defined here - a mixer with fixed-size state of its own, mixed
with attention layers, one layer run twice, one entry reading another's cache;
a feed-forward with routing, a position encoding that is not rotary, layers
that differ in mixer and in feed-forward - registered, built and stepped
without touching the framework's files."""

import json
import math
from dataclasses import dataclass
from typing import Dict, List

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.cache import StateSpec
from flashdecode_cuda_b200.engine import LayerSpec, Model, ModelBlueprint, PartSpec, RunSpec
from flashdecode_cuda_b200.parts import LayerCache, Mixer
from flashdecode_cuda_b200.weights import TensorSpec
from helpers import TINY, TOL, prompts_for, raw_config, rel_err, weights_of, write_folder
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
PART_TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return write_folder(tmp_path_factory.mktemp("parts"), "C", seed=4)


def setup(folder, dtype, lengths):
    eng = fd.load(folder, device="cuda", dtype=dtype)
    model = eng.model
    cache = model.new_cache(max_tokens=512, block_size=8)
    prompts = prompts_for(TINY["C"]["vocab_size"], lengths, seed=2)
    slots = [cache.admit() for _ in prompts]
    cache.reserve([(s, len(p)) for s, p in zip(slots, prompts)])
    cache.sync()
    ctx = model.make_context(cache, slots, prompts, "all")
    return model, cache, ctx, prompts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_norm_feed_forward_head(folder, dtype):
    model, cache, ctx, prompts = setup(folder, dtype, [9, 30])
    raw, w = raw_config(folder), {k: v.double() for k, v in weights_of(folder).items()}
    T, H = ctx.T, model.hidden_size
    flat = [t for p in prompts for t in p]
    resid = torch.empty(T, H, device="cuda")
    model.embedding.forward(ctx, resid)
    assert torch.equal(resid.cpu().double(), P.embedding(torch.tensor(flat), w["model.embed_tokens.weight"]))

    g = torch.Generator().manual_seed(0)
    delta = torch.randn(T, H, generator=g).to(DT[dtype]).cuda()
    before = resid.clone()
    xn = torch.empty(T, H, dtype=DT[dtype], device="cuda")
    norm = model.blocks[1].norm2
    norm.forward(ctx, delta, resid, xn)
    summed = before.double().cpu() + delta.double().cpu()
    assert rel_err(resid, summed) < 1e-6
    want = P.rmsnorm(summed, w["model.layers.1.post_attention_layernorm.weight"], raw["rms_norm_eps"])
    assert rel_err(xn, want) < PART_TOL[dtype]

    x = (0.5 * torch.randn(T, H, generator=g)).to(DT[dtype]).cuda()
    got = model.blocks[2].feed_forward.forward(ctx, x)
    assert rel_err(got, P.mlp_block(w, 2, x.double().cpu())) < PART_TOL[dtype]

    logits = model.head.forward(ctx, x[:5].contiguous())
    assert logits.dtype == torch.float32
    assert rel_err(logits, P.linear(x[:5].double().cpu(), w["lm_head.weight"])) < PART_TOL[dtype]


def test_rotary_tables(folder):
    model, cache, ctx, _ = setup(folder, "float32", [3])
    rope = model.positions["rope"]
    cos, sin = P.rope_tables(TINY["C"]["head_dim"], rope.cos.shape[0], TINY["C"]["rope_theta"])
    half = TINY["C"]["head_dim"] // 2
    assert torch.equal(rope.cos.cpu(), cos[:, :half]) and torch.equal(rope.sin.cpu(), sin[:, :half])
    assert rope.cos.shape[0] == TINY["C"]["max_position_embeddings"] >= cache.max_len


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", [0, 3])           # full attention, and a window of 24
def test_attention_mixer_and_block(folder, dtype, layer):
    lengths = [9, 30, 41]
    model, cache, ctx, prompts = setup(folder, dtype, lengths)
    raw, w = raw_config(folder), {k: v.double() for k, v in weights_of(folder).items()}
    T, H = ctx.T, model.hidden_size
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(DT[dtype]).cuda()
    lc = model._layer_caches(cache)[layer]
    got = model.blocks[layer].mixer.forward(ctx, x, lc)
    cos, sin = P.rope_tables(raw["head_dim"], max(lengths), raw["rope_theta"])
    o = 0
    for n in lengths:
        want = P.attention_block(raw, w, layer, x[o:o + n].double().cpu(), cos[:n], sin[:n])
        assert rel_err(got[o:o + n], want) < PART_TOL[dtype]
        o += n
    # the whole arrangement: x += mixer(norm(x)); x += ff(norm(x)), handed on as (resid, delta)
    resid = x.float().clone()
    delta = model.blocks[layer].forward(ctx, resid, None, lc)
    o = 0
    for n in lengths:
        xs = x[o:o + n].double().cpu()
        p = f"model.layers.{layer}"
        mid = xs + P.attention_block(raw, w, layer, P.rmsnorm(xs, w[f"{p}.input_layernorm.weight"], raw["rms_norm_eps"]),
                                     cos[:n], sin[:n])
        ff = P.mlp_block(w, layer, P.rmsnorm(mid, w[f"{p}.post_attention_layernorm.weight"], raw["rms_norm_eps"]))
        assert rel_err(resid[o:o + n], mid) < PART_TOL[dtype]
        assert rel_err(delta[o:o + n], ff) < 2 * PART_TOL[dtype]
        o += n
    model.check_status()


# ---------------------------------------------------------------------------
# a toy architecture, defined and registered here
# ---------------------------------------------------------------------------

@fd.register_part("mixer", "toy_running_mean")
class RunningMean(Mixer):
    """delta_t = W * mean(x_0 .. x_t): its cache is one running sum per
    sequence (fixed size), not keys.  Written with torch on the device and the
    step's host mirrors, so its steps are not replayed from CUDA graphs."""
    graph_safe = False

    def __init__(self, prefix, hidden_size):
        self.prefix, self.H = prefix, hidden_size

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.mix.weight", (self.H, self.H))]

    def state_requests(self):
        return [StateSpec("sum", (self.H,), torch.float32)]

    def bind(self, tensors, rt):
        self.rt = rt
        self.w = tensors[f"{self.prefix}.mix.weight"]

    def forward(self, ctx, x, lc: LayerCache):
        out = ctx.ws.get("toy_out", tuple(x.shape), x.dtype)
        state = lc.states["sum"]
        o = 0
        for slot, n, cached in zip(ctx.h_slots, ctx.h_q_len, ctx.h_ctx_len):
            sums = torch.cumsum(x[o:o + n].float(), 0) + state[slot]
            counts = torch.arange(cached + 1, cached + n + 1, device=x.device, dtype=torch.float32)
            out[o:o + n] = ((sums / counts[:, None]) @ self.w.float().T).to(x.dtype)
            if lc.writes:
                state[slot] = sums[-1]
            o += n
        return out


@dataclass
class ToyConfig:
    hidden_size: int
    vocab_size: int
    intermediate_size: int
    eps: float
    architecture: str = "ToyForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(d["hidden_size"], d["vocab_size"], d["intermediate_size"], d["eps"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "intermediate_size": self.intermediate_size, "eps": self.eps}


def toy_blueprint(cfg: ToyConfig) -> ModelBlueprint:
    H = cfg.hidden_size

    def layer(i, mixer):
        p = f"toy.layers.{i}"
        return LayerSpec("prenorm", PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.eps), f"{p}.n1"), mixer,
                         PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.eps), f"{p}.n2"),
                         PartSpec("feed_forward", "swiglu", dict(hidden_size=H, intermediate_size=cfg.intermediate_size),
                                  f"{p}.ff"))
    attn = lambda i: PartSpec("mixer", "gqa_attention", dict(hidden_size=H, n_heads=2, n_kv_heads=1, head_dim=16,
                                                            position="rope", bias=False), f"toy.layers.{i}.attn")
    return ModelBlueprint(
        hidden_size=H, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab_size, hidden_size=H), "toy.embed"),
        positions={"rope": PartSpec("position", "rotary_half", dict(head_dim=16, theta=100.0, max_positions=256))},
        layers=[layer(0, PartSpec("mixer", "toy_running_mean", dict(hidden_size=H), "toy.layers.0")),
                layer(1, attn(1)),
                layer(2, PartSpec("mixer", "toy_running_mean", dict(hidden_size=H), "toy.layers.2"))],
        # layer 0 runs twice (shared weights, separate state); the last entry reads the keys of entry 1
        schedule=[RunSpec(0), RunSpec(1), RunSpec(2), RunSpec(0), RunSpec(1, cache_from=1)],
        final_norm=PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.eps), "toy.norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=H, tied_to="toy.embed.weight"),
                      "toy.head"),
        max_positions=256)


fd.register_architecture("ToyForCausalLM", ToyConfig, toy_blueprint)


def toy_plain(w: Dict[str, torch.Tensor], cfg: ToyConfig, tokens: List[int]) -> torch.Tensor:
    """The toy model on one whole sequence, in float64, with the plain parts."""
    w = {k: v.double() for k, v in w.items()}
    x = w["toy.embed.weight"][torch.tensor(tokens)]
    S = len(tokens)
    cos, sin = P.rope_tables(16, S, 100.0)
    kept = {}

    def ff(i, h):
        p = f"toy.layers.{i}.ff"
        return P.linear(P.swiglu(P.linear(h, w[f"{p}.gate_proj.weight"]), P.linear(h, w[f"{p}.up_proj.weight"])),
                        w[f"{p}.down_proj.weight"])

    def mean_mixer(i, h):
        means = torch.cumsum(h, 0) / torch.arange(1, S + 1, dtype=torch.float64)[:, None]
        return means @ w[f"toy.layers.{i}.mix.weight"].T

    def attn(i, h, own_kv):
        p = f"toy.layers.{i}.attn"
        q = P.apply_rope(P.linear(h, w[f"{p}.q_proj.weight"]).view(S, 2, 16), cos, sin)
        if own_kv:
            k = P.apply_rope(P.linear(h, w[f"{p}.k_proj.weight"]).view(S, 1, 16), cos, sin)
            kept[i] = (k, P.linear(h, w[f"{p}.v_proj.weight"]).view(S, 1, 16))
        k, v = kept[i]
        o = P.causal_gqa_attention(q, k, v, 1 / math.sqrt(16), None)
        return P.linear(o.reshape(S, 32), w[f"{p}.o_proj.weight"])

    for layer, own in [(0, True), (1, True), (2, True), (0, True), (1, False)]:
        p = f"toy.layers.{layer}"
        h = P.rmsnorm(x, w[f"{p}.n1.weight"], cfg.eps)
        x = x + (attn(layer, h, own) if layer == 1 else mean_mixer(layer, h))
        x = x + ff(layer, P.rmsnorm(x, w[f"{p}.n2.weight"], cfg.eps))
    return P.rmsnorm(x, w["toy.norm.weight"], cfg.eps) @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_registers_builds_and_steps(tmp_path, dtype):
    cfg = ToyConfig(48, 101, 80, 1e-5)
    folder = tmp_path / "toy"
    probe = Model.from_config(cfg, torch.float32, "cpu")
    tensors = fd.weights.random_tensors(probe.tensor_specs(), 3)
    fd.weights.write_model_folder(folder, cfg.to_dict(), tensors)

    eng = fd.load(folder, device="cuda", dtype=dtype)         # chosen by config.json, like any model
    model = eng.model
    assert isinstance(model.blocks[0].mixer, RunningMean) and not model.graph_safe and not eng.use_graphs
    groups = model.cache_groups()
    assert len(groups) == 1 and groups[0].n_layers == 1       # entry 4 shares entry 1's keys
    cache = model.new_cache(max_tokens=256, block_size=8)
    assert sorted(cache.states) == ["run0.sum", "run2.sum", "run3.sum"]

    prompts = prompts_for(101, [23, 5, 40], seed=1)
    want = [toy_plain(tensors, cfg, p) for p in prompts]
    # whole prompts in one unequal batch
    slots = [cache.admit() for _ in prompts]
    got = model.step(cache, slots, prompts, "all")
    o = 0
    for p, ref in zip(prompts, want):
        assert rel_err(got[o:o + len(p)], ref) < TOL[dtype]
        o += len(p)
    for s in slots:
        cache.release(s)
    # a cut prompt, then token by token, in slots that are used again (state must start from zero)
    slots = [cache.admit() for _ in prompts]
    heads = [len(p) - 4 for p in prompts]
    model.step(cache, slots, [p[:h] for p, h in zip(prompts, heads)], None)
    for i in range(4):
        got = model.step(cache, slots, [[p[h + i]] for p, h in zip(prompts, heads)], "last")
        for j, (p, ref) in enumerate(zip(prompts, want)):
            assert rel_err(got[j], ref[heads[j] + i]) < TOL[dtype]
    # and through the generation loop (eager steps, since the toy mixer decides on the host)
    res = eng.generate(prompts[:2], 5)
    assert all(len(r.tokens) == 5 for r in res)
    model.check_status()


# ---------------------------------------------------------------------------
# a second toy architecture: another position encoding and a feed-forward with routing
# ---------------------------------------------------------------------------

@fd.register_part("position", "toy_sinusoid_table")
class SinusoidTable(fd.parts.Position):
    """table[p, i] = 1 + amp * sin(p / period + i): multiplied into the activations by the mixer below.
    No weights; built for as many positions as the cache holds."""

    def __init__(self, size, period, amp, max_positions):
        self.size, self.period, self.amp, self.max_positions = size, float(period), float(amp), max_positions
        self.table = None

    def prepare(self, n_positions, rt):
        n = min(n_positions, self.max_positions)
        if self.table is None or self.table.shape[0] < n:
            p = torch.arange(n, dtype=torch.float32)[:, None]
            i = torch.arange(self.size, dtype=torch.float32)[None, :]
            self.table = (1.0 + self.amp * torch.sin(p / self.period + i)).to(rt.device)


@fd.register_part("mixer", "toy_position_gate")
class PositionGate(Mixer):
    """delta_t = W (x_t * table[pos_t]): no cache at all, the position comes from the step's index arrays."""

    def __init__(self, prefix, hidden_size, position):
        self.prefix, self.H, self.position = prefix, hidden_size, position

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.gate.weight", (self.H, self.H))]

    def bind(self, tensors, rt):
        self.rt = rt
        self.w = tensors[f"{self.prefix}.gate.weight"]

    def forward(self, ctx, x, lc: LayerCache):
        gate = self.position.table[ctx.tok_pos.long()]
        return ((x.float() * gate) @ self.w.float().T).to(x.dtype)


@fd.register_part("feed_forward", "toy_top1_experts")
class Top1Experts(fd.parts.FeedForward):
    """Router logits in float32, the best expert alone (lowest index wins ties), one matrix per expert."""

    def __init__(self, prefix, hidden_size, n_experts):
        self.prefix, self.H, self.E = prefix, hidden_size, n_experts

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.router.weight", (self.E, self.H), "vector"),      # stays 32-bit if stored so
                TensorSpec(f"{self.prefix}.experts.weight", (self.E * self.H, self.H))]

    def bind(self, tensors, rt):
        self.rt = rt
        self.router = tensors[f"{self.prefix}.router.weight"]
        self.experts = tensors[f"{self.prefix}.experts.weight"].view(self.E, self.H, self.H)

    def forward(self, ctx, x):
        choice = (x.float() @ self.router.float().T).argmax(-1)
        return torch.bmm(self.experts[choice].float(), x.float()[:, :, None])[:, :, 0].to(x.dtype)


@dataclass
class Toy2Config:
    hidden_size: int
    vocab_size: int
    n_experts: int
    eps: float
    architecture: str = "Toy2ForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(d["hidden_size"], d["vocab_size"], d["n_experts"], d["eps"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "n_experts": self.n_experts, "eps": self.eps}


def toy2_blueprint(cfg: Toy2Config) -> ModelBlueprint:
    H = cfg.hidden_size
    norm = lambda name: PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.eps), name)

    def layer(i, mixer, ff):
        return LayerSpec("prenorm", norm(f"t2.layers.{i}.n1"), mixer, norm(f"t2.layers.{i}.n2"), ff)
    gate = lambda i: PartSpec("mixer", "toy_position_gate", dict(hidden_size=H, position="sinus"), f"t2.layers.{i}")
    attn = lambda i: PartSpec("mixer", "gqa_attention", dict(hidden_size=H, n_heads=2, n_kv_heads=2, head_dim=16,
                                                            position="rope", bias=False), f"t2.layers.{i}.attn")
    routed = lambda i: PartSpec("feed_forward", "toy_top1_experts", dict(hidden_size=H, n_experts=cfg.n_experts),
                                f"t2.layers.{i}.moe")
    dense = lambda i: PartSpec("feed_forward", "swiglu", dict(hidden_size=H, intermediate_size=2 * H), f"t2.layers.{i}.ff")
    return ModelBlueprint(
        hidden_size=H, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab_size, hidden_size=H), "t2.embed"),
        positions={"rope": PartSpec("position", "rotary_half", dict(head_dim=16, theta=50.0, max_positions=128)),
                   "sinus": PartSpec("position", "toy_sinusoid_table", dict(size=H, period=3.0, amp=0.5, max_positions=128))},
        # different mixers AND different feed-forwards from layer to layer
        layers=[layer(0, gate(0), routed(0)), layer(1, attn(1), routed(1)), layer(2, gate(2), dense(2))],
        schedule=[RunSpec(0), RunSpec(1), RunSpec(2)],
        final_norm=norm("t2.norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=H, tied_to=None), "t2.head"),
        max_positions=128)


fd.register_architecture("Toy2ForCausalLM", Toy2Config, toy2_blueprint)


def toy2_plain(w: Dict[str, torch.Tensor], cfg: Toy2Config, tokens: List[int]) -> torch.Tensor:
    w = {k: v.double() for k, v in w.items()}
    H, S = cfg.hidden_size, len(tokens)
    x = w["t2.embed.weight"][torch.tensor(tokens)]
    pos = torch.arange(S, dtype=torch.float32)[:, None]
    table = (1.0 + 0.5 * torch.sin(pos / 3.0 + torch.arange(H, dtype=torch.float32)[None, :])).double()
    cos, sin = P.rope_tables(16, S, 50.0)

    def gate(i, h):
        return (h * table) @ w[f"t2.layers.{i}.gate.weight"].T

    def attn(i, h):
        p = f"t2.layers.{i}.attn"
        q = P.apply_rope(P.linear(h, w[f"{p}.q_proj.weight"]).view(S, 2, 16), cos, sin)
        k = P.apply_rope(P.linear(h, w[f"{p}.k_proj.weight"]).view(S, 2, 16), cos, sin)
        v = P.linear(h, w[f"{p}.v_proj.weight"]).view(S, 2, 16)
        return P.linear(P.causal_gqa_attention(q, k, v, 0.25, None).reshape(S, 32), w[f"{p}.o_proj.weight"])

    def routed(i, h):
        choice = (h @ w[f"t2.layers.{i}.moe.router.weight"].T).argmax(-1)
        experts = w[f"t2.layers.{i}.moe.experts.weight"].view(cfg.n_experts, H, H)
        return torch.stack([experts[c] @ h[t] for t, c in enumerate(choice.tolist())])

    def dense(i, h):
        p = f"t2.layers.{i}.ff"
        return P.linear(P.swiglu(P.linear(h, w[f"{p}.gate_proj.weight"]), P.linear(h, w[f"{p}.up_proj.weight"])),
                        w[f"{p}.down_proj.weight"])

    for i, (mix, ff) in enumerate([(gate, routed), (attn, routed), (gate, dense)]):
        x = x + mix(i, P.rmsnorm(x, w[f"t2.layers.{i}.n1.weight"], cfg.eps))
        x = x + ff(i, P.rmsnorm(x, w[f"t2.layers.{i}.n2.weight"], cfg.eps))
    return P.rmsnorm(x, w["t2.norm.weight"], cfg.eps) @ w["t2.head.weight"].T


def test_toy_routing_and_another_position_encoding(tmp_path):
    """A feed-forward with routing, a position encoding that is not rotary, and layers that differ in both
    mixer and feed-forward: registered here, built from config.json and stepped like any model (float32,
    where the router's choice is the same as the plain implementation's)."""
    cfg = Toy2Config(32, 77, 3, 1e-5)
    folder = tmp_path / "toy2"
    probe = Model.from_config(cfg, torch.float32, "cpu")
    tensors = fd.weights.random_tensors(probe.tensor_specs(), 9, dtype=torch.float32)
    # well separated router logits, so that rounding cannot change a choice
    for k in tensors:
        if k.endswith("router.weight"):
            tensors[k] = tensors[k] * 40
    fd.weights.write_model_folder(folder, cfg.to_dict(), tensors)
    eng = fd.load(folder, device="cuda", dtype="float32")
    model = eng.model
    assert isinstance(model.blocks[0].feed_forward, Top1Experts) and isinstance(model.blocks[2].mixer, PositionGate)
    assert len(model.cache_groups()) == 1 and model.cache_groups()[0].n_layers == 1      # only layer 1 keeps keys
    cache = model.new_cache(max_tokens=256, block_size=8)
    prompts = prompts_for(77, [19, 6, 33], seed=4)
    want = [toy2_plain(tensors, cfg, p) for p in prompts]
    slots = [cache.admit() for _ in prompts]
    heads = [len(p) - 3 for p in prompts]
    got = model.step(cache, slots, [p[:h] for p, h in zip(prompts, heads)], "all")
    o = 0
    for h, ref in zip(heads, want):
        assert rel_err(got[o:o + h], ref[:h]) < 1e-4
        o += h
    for i in range(3):
        got = model.step(cache, slots, [[p[h + i]] for p, h in zip(prompts, heads)], "last")
        for j, ref in enumerate(want):
            assert rel_err(got[j], ref[heads[j] + i]) < 1e-4
    model.check_status()


# ---------------------------------------------------------------------------
# a third toy architecture: a mixer whose state lives on the device only (its decode steps are replayed from
# CUDA graphs), a norm and a block that know nothing of partial sums, a block of three norms
# ---------------------------------------------------------------------------

@fd.register_part("mixer", "toy_running_mean_device")
class RunningMeanDevice(Mixer):
    """The same function as ``RunningMean`` above, written with device index arrays only (no host mirror of the
    step), so ``graph_safe`` stays True and decode steps are captured.  Padding rows (slot -1) change nothing."""

    def __init__(self, prefix, hidden_size):
        self.prefix, self.H = prefix, hidden_size

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.mix.weight", (self.H, self.H))]

    def state_requests(self):
        return [StateSpec("sum", (self.H,), torch.float32)]

    def bind(self, tensors, rt):
        self.rt = rt
        self.w = tensors[f"{self.prefix}.mix.weight"]

    def forward(self, ctx, x, lc: LayerCache):
        state = lc.states["sum"]
        row = ctx.tok_row.long()
        slot = ctx.row_slot.long()
        live = (slot >= 0).float()[:, None]                          # [rows, 1]
        safe = slot.clamp(min=0)
        xf = x.float() * live[row]
        cs = torch.cumsum(xf, 0)
        start = ctx.row_q_start.long()
        before = cs[start] - xf[start]                                # sum of all tokens before each row's first
        sums = cs - before[row] + state[safe][row] * live[row]        # running sum inside each sequence
        counts = (ctx.tok_pos + 1).float()[:, None]
        out = ((sums / counts) @ self.w.float().T).to(x.dtype)
        if lc.writes:
            last = start + ctx.row_q_len.long() - 1
            state.index_add_(0, safe, (cs[last] - before) * live)      # padding rows add zero to slot 0
        return out


@fd.register_part("norm", "toy_centered_norm")
class CenteredNorm(fd.parts.Norm):
    """resid += delta; out = (resid - mean) * rsqrt(var + eps) * weight, with torch on the device.  It knows
    nothing of partial sums (``accepts_parts`` stays False), so no part may hand it any."""

    def __init__(self, prefix, size, eps):
        self.name, self.size, self.eps = f"{prefix}.weight", size, float(eps)

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), "vector", init="norm")]

    def bind(self, tensors, rt):
        self.rt = rt
        self.weight = tensors[self.name]

    def forward(self, ctx, delta, resid, out, rows=None, n_out=None, write_resid=True):
        assert delta is None or delta.dim() == 2, "partial sums were handed to a norm that never asked for them"
        r = resid if rows is None else resid[rows.long()]
        if delta is not None:
            r = r + (delta if rows is None else delta[rows.long()]).float()
            if write_resid:
                if rows is None:
                    resid.copy_(r)
                else:
                    resid[rows.long()] = r
        c = r - r.mean(-1, keepdim=True)
        out.copy_((c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(out.dtype))


@fd.register_part("block", "toy_sandwich")
class SandwichBlock(fd.parts.Block):
    """Three norms: x += norm_mid(mixer(norm1(x))); x += feed_forward(norm2(x)).  The mixer's output is normed
    before it is added, so this block does that add itself; its feed-forward's output is handed on as delta."""

    def __init__(self, norm1, mixer, norm_mid, norm2, feed_forward):
        self.norm1, self.mixer, self.norm_mid, self.norm2, self.feed_forward = norm1, mixer, norm_mid, norm2, feed_forward

    def parts(self):
        return [self.norm1, self.mixer, self.norm_mid, self.norm2, self.feed_forward]

    def forward(self, ctx, resid, delta, lc):
        assert delta is None or delta.dim() == 2, "partial sums were handed to a block that never asked for them"
        xn = ctx.ws.get("normed", tuple(resid.shape), ctx.rt.dtype)
        self.norm1.forward(ctx, delta, resid, xn)
        d1 = self.mixer.forward(ctx, xn, lc)
        zeros = torch.zeros_like(resid)
        mid = ctx.ws.get("sandwich_mid", tuple(resid.shape), ctx.rt.dtype)
        self.norm_mid.forward(ctx, d1, zeros, mid)                    # norm of the mixer's output alone
        self.norm2.forward(ctx, mid, resid, xn)                       # resid += mid; xn = norm2(resid)
        return self.feed_forward.forward(ctx, xn)


@dataclass
class Toy3Config:
    hidden_size: int
    vocab_size: int
    intermediate_size: int
    eps: float
    architecture: str = "Toy3ForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(d["hidden_size"], d["vocab_size"], d["intermediate_size"], d["eps"])

    def to_dict(self):
        return {"architectures": [self.architecture], "hidden_size": self.hidden_size, "vocab_size": self.vocab_size,
                "intermediate_size": self.intermediate_size, "eps": self.eps}


def toy3_blueprint(cfg: Toy3Config) -> ModelBlueprint:
    H = cfg.hidden_size
    rms = lambda name: PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.eps), name)
    centered = lambda name: PartSpec("norm", "toy_centered_norm", dict(size=H, eps=cfg.eps), name)
    ff = lambda i: PartSpec("feed_forward", "swiglu", dict(hidden_size=H, intermediate_size=cfg.intermediate_size),
                            f"t3.layers.{i}.ff")
    mean = lambda i: PartSpec("mixer", "toy_running_mean_device", dict(hidden_size=H), f"t3.layers.{i}")
    attn = lambda i: PartSpec("mixer", "gqa_attention", dict(hidden_size=H, n_heads=2, n_kv_heads=1, head_dim=16,
                                                            position="rope", bias=False), f"t3.layers.{i}.attn")
    layers = [
        # the built-in arrangement with a stateful mixer; its feed-forward's output goes to the sandwich block
        LayerSpec("prenorm", norm1=rms("t3.layers.0.n1"), mixer=mean(0), norm2=rms("t3.layers.0.n2"), feed_forward=ff(0)),
        # five named parts, three of them norms, one of another kind
        LayerSpec("toy_sandwich", {"norm1": centered("t3.layers.1.n1"), "mixer": attn(1), "norm_mid": rms("t3.layers.1.nm"),
                                   "norm2": rms("t3.layers.1.n2"), "feed_forward": ff(1)}),
        # the built-in arrangement whose first norm is the foreign one
        LayerSpec("prenorm", centered("t3.layers.2.n1"), mean(2), rms("t3.layers.2.n2"), ff(2)),
    ]
    return ModelBlueprint(
        hidden_size=H, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab_size, hidden_size=H), "t3.embed"),
        positions={"rope": PartSpec("position", "rotary_half", dict(head_dim=16, theta=100.0, max_positions=256))},
        layers=layers, schedule=[RunSpec(0), RunSpec(1), RunSpec(2)],
        final_norm=centered("t3.norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=H, tied_to="t3.embed.weight"),
                      "t3.head"),
        max_positions=256)


fd.register_architecture("Toy3ForCausalLM", Toy3Config, toy3_blueprint)


def toy3_plain(w: Dict[str, torch.Tensor], cfg: Toy3Config, tokens: List[int]) -> torch.Tensor:
    w = {k: v.double() for k, v in w.items()}
    S = len(tokens)
    x = w["t3.embed.weight"][torch.tensor(tokens)]
    cos, sin = P.rope_tables(16, S, 100.0)

    def centered(h, name):
        c = h - h.mean(-1, keepdim=True)
        return c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + cfg.eps) * w[name]

    def ff(i, h):
        p = f"t3.layers.{i}.ff"
        return P.linear(P.swiglu(P.linear(h, w[f"{p}.gate_proj.weight"]), P.linear(h, w[f"{p}.up_proj.weight"])),
                        w[f"{p}.down_proj.weight"])

    def mean_mixer(i, h):
        return (torch.cumsum(h, 0) / torch.arange(1, S + 1, dtype=torch.float64)[:, None]) @ w[f"t3.layers.{i}.mix.weight"].T

    def attn(i, h):
        p = f"t3.layers.{i}.attn"
        q = P.apply_rope(P.linear(h, w[f"{p}.q_proj.weight"]).view(S, 2, 16), cos, sin)
        k = P.apply_rope(P.linear(h, w[f"{p}.k_proj.weight"]).view(S, 1, 16), cos, sin)
        v = P.linear(h, w[f"{p}.v_proj.weight"]).view(S, 1, 16)
        return P.linear(P.causal_gqa_attention(q, k, v, 0.25, None).reshape(S, 32), w[f"{p}.o_proj.weight"])

    x = x + mean_mixer(0, P.rmsnorm(x, w["t3.layers.0.n1.weight"], cfg.eps))
    x = x + ff(0, P.rmsnorm(x, w["t3.layers.0.n2.weight"], cfg.eps))
    x = x + P.rmsnorm(attn(1, centered(x, "t3.layers.1.n1.weight")), w["t3.layers.1.nm.weight"], cfg.eps)
    x = x + ff(1, P.rmsnorm(x, w["t3.layers.1.n2.weight"], cfg.eps))
    x = x + mean_mixer(2, centered(x, "t3.layers.2.n1.weight"))
    x = x + ff(2, P.rmsnorm(x, w["t3.layers.2.n2.weight"], cfg.eps))
    return centered(x, "t3.norm.weight") @ w["t3.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_that_know_nothing_of_partial_sums_and_state_under_graphs(tmp_path, dtype):
    """Layers given as named parts (a block of three norms among them); a norm and a block without
    ``accepts_parts`` next to the built-in feed-forward, which offers partial sums in decode steps: one-token
    steps must hand them plain tensors.  The stateful mixer keeps its state on the device only, so decode
    steps are replayed from CUDA graphs: a graph's first step must not run twice on that state."""
    from flashdecode_cuda_b200.engine.decode import GraphDecoder
    cfg = Toy3Config(64, 97, 96, 1e-5)
    folder = tmp_path / "toy3"
    probe = Model.from_config(cfg, torch.float32, "cpu")
    assert [type(b).__name__ for b in probe.blocks] == ["PreNormBlock", "SandwichBlock", "PreNormBlock"]
    assert probe.blocks[0].accepts_parts and not probe.blocks[1].accepts_parts and not probe.blocks[2].accepts_parts
    tensors = fd.weights.random_tensors(probe.tensor_specs(), 7)
    fd.weights.write_model_folder(folder, cfg.to_dict(), tensors)
    eng = fd.load(folder, device="cuda", dtype=dtype)
    model = eng.model
    assert model.graph_safe and eng.use_graphs
    prompts = prompts_for(97, [21, 4, 37], seed=3)
    n_dec = 9
    reqs = [p + q for p, q in zip(prompts, prompts_for(97, [n_dec] * 3, seed=4))]
    want = [toy3_plain(tensors, cfg, r) for r in reqs]
    tol = TOL[dtype]
    # eager: whole prompts, then one token each (up to 16 rows: the feed-forward would offer partial sums)
    cache = model.new_cache(max_tokens=512, block_size=8)
    slots = [cache.admit() for _ in reqs]
    got = model.step(cache, slots, prompts, "last")
    for j, p in enumerate(prompts):
        assert rel_err(got[j], want[j][len(p) - 1]) < tol
    for i in range(n_dec):
        got = model.step(cache, slots, [[r[len(p) + i]] for r, p in zip(reqs, prompts)], "last")
        for j, p in enumerate(prompts):
            assert rel_err(got[j], want[j][len(p) + i]) < tol, f"eager, request {j}, decoded token {i}"
    for s in slots:
        cache.release(s)
    # the same through captured graphs: the step that captures a graph is a real step of the sequences, and a
    # sequence that ends changes the bucket, so graphs are captured in the middle of sequences too
    slots = [cache.admit() for _ in reqs]
    model.step(cache, slots, prompts, None)
    dec = GraphDecoder(model, cache)
    live = [0, 1, 2]
    for i in range(n_dec):
        if i == 4:
            cache.release(slots[1])
            live = [0, 2]
        dec.run([slots[j] for j in live], [reqs[j][len(prompts[j]) + i] for j in live])
        got = dec.last_logits(len(live)).clone()
        for k, j in enumerate(live):
            assert rel_err(got[k], want[j][len(prompts[j]) + i]) < tol, f"graphs, request {j}, decoded token {i}"
    # and through the entry point, greedy: the tokens of the plain implementation
    if dtype == "float32":
        res = eng.generate(prompts, 6)
        for r, p in zip(res, prompts):
            seq = list(p)
            for t in r.tokens:
                assert t == int(toy3_plain(tensors, cfg, seq)[-1].argmax())
                seq.append(t)
    model.check_status()
