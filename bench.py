#!/usr/bin/env python3
"""Throughput of flashdecode_cuda_b200 on one B200: decoded tokens per second.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The default run has the layer
sizes of Qwen2.5-1.5B (28 layers, hidden 1536, 12/2 heads of 128, intermediate
8960, vocabulary 151936, tied head) with random bfloat16 weights, 8 sequences
whose prompts have unequal lengths drawn from [1024, 2048], prefilled for real
and decoded until the longest reaches the context length 4096 at the end of the
timed steps.  It prints ONE JSON line:

* ``value``: decoded tokens per second, timed on the device with CUDA events
  around K graph-replayed steps whose tokens never leave the device;
* ``e2e``: the same through ``Engine.stream`` (the Python entry point): every
  step uploads that step's token ids from pinned host memory and reads the
  sampled ids back;
* ``prefill``: one 2,048-token prompt in one step, with the fraction of the
  bfloat16 tensor peak its floating-point operations reach;
* ``roofline``: bytes a decode step has to read (every weight once, and the
  cached keys and values of the live sequences) / step time / HBM peak;
* ``points``: decoded tokens per second at batch 1 and 64.

Every device-timed number is the best of up to five trials of K steps each (the
discipline of testing/phase1.py:312-351 of davidjoyme/flashdecode-cuda); the
trials and their spread are in the line, and ``"jitter": true`` marks a spread
above 15 % (testing/phase1.py:425-434).  The cache block is 16 tokens, as the
benchmark configuration says; the library's own default of 64 is measured
beside it (``points.decode_b8_block64``, ``points.prefill_block64_ms``).

Peaks come from MEASURED_PEAKS.json beside this file when present, else from
the stated fallback.  Only one GPU is used: for --gpus > 1 it says so and exits
with 2.

``--impl reference`` runs davidjoyme/flashdecode-cuda itself, unmodified, from
its source tree (``baseline/_ref``, else ``$FLASHDECODE_REFERENCE``, else the
``reference_path`` of BASELINE.json) through its own public API:
``LlamaEngine(cfg, weights, "cuda", bfloat16)``, ``new_paged_cache``,
``prefill`` and ``decode_step`` + ``argmax`` with its stock "ref" (PyTorch)
ops, at the same sizes, batch, per-sequence contexts and block size, timed the
way its own testing/phase1.py does.  Its CUDA extension builds for sm_120 only
and is not used.  None of this library's code is on that path.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BLOCK_SIZE = 16          # tokens of a cache block: what the benchmark configuration names
LIB_BLOCK_SIZE = 64      # the library's own default, measured beside it
TRIALS = 5
JITTER = 0.15
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            out = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the
    timed regions run (read only; nothing is set)."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        rows = [l.strip().split(", ") for l in open(self.file.name) if l.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(int(float(r[0])))
                mx = max(mx, int(float(r[1])))
                for name, v in zip(names, r[3:7]):
                    if v.strip().lower().startswith("active"):
                        reasons.add(name)
            except (ValueError, IndexError):
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_engine(preset: str, layers: int, seed: int, dtype=None):
    import torch
    dtype = dtype or torch.bfloat16
    import flashdecode_cuda_b200 as fd
    from flashdecode_cuda_b200.config import config_from_dict, preset_dict
    from flashdecode_cuda_b200.engine import Engine, Model, random_weights
    cfgd = preset_dict(preset)
    full_layers = cfgd["num_hidden_layers"]
    if layers:
        cfgd["num_hidden_layers"] = layers
        if "max_window_layers" in cfgd:
            cfgd["max_window_layers"] = min(cfgd["max_window_layers"], layers)
    cfg = config_from_dict(cfgd)
    model = Model.from_config(cfg, dtype, "cuda")
    model.bind(random_weights(model, seed, dtype, device="cuda"))
    return Engine(model), cfg, full_layers


def ragged_prompts(batch: int, lo: int, hi: int, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    if batch > 1:
        lens[0] = hi            # the longest prompt is as long as allowed, so the context bound is reached
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def plan_trials(context: int, longest_prompt: int, steps: int, warmup: int, trials: int) -> int:
    """As many trials of ``steps`` steps as fit before the longest sequence reaches the context."""
    room = context - longest_prompt - 1 - warmup
    return max(1, min(trials, room // max(1, steps)))


def decode_run(engine, batch: int, context: int, steps: int, warmup: int, seed: int, e2e: bool,
               prompt_range=None, profile: bool = False, block_size: int = BLOCK_SIZE, trials: int = TRIALS, decoder=None):
    """Prefill ragged prompts, decode untimed until ``trials * steps + warmup`` steps are left before the
    longest sequence reaches ``context``, then time ``trials`` runs of ``steps`` steps each.  ``decoder``: run in this
    decoder's (empty) cache with the graphs it has captured already, instead of a new cache and new captures; the
    device-timed run returns its decoder as ``out["decoder"]``."""
    import torch
    from flashdecode_cuda_b200 import kernels as K
    from flashdecode_cuda_b200.engine.decode import GraphDecoder
    model = engine.model
    vocab = model.vocab_size
    lo, hi = prompt_range or (context // 4, context // 2)
    prompts = ragged_prompts(batch, lo, hi, vocab, seed)
    longest = max(len(p) for p in prompts)
    if decoder is not None:
        cache = decoder.cache
        engine.use_decoder(decoder)
    else:
        cache = model.new_cache(batch_size=batch, max_len=context, block_size=block_size)
    out = {}
    if e2e:
        # the public entry point: host token ids in, host token ids out, every step
        trials = plan_trials(context, longest, steps, warmup, min(trials, 3))
        total_new = context - longest
        it = engine.stream(prompts, total_new, cache, max_batch=batch, block_size=block_size)
        n_fast = total_new - trials * steps - warmup
        for _ in range(n_fast):
            next(it)
        torch.cuda.synchronize()
        for _ in range(warmup):
            next(it)
        times = []
        for _ in range(trials):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                next(it)
            torch.cuda.synchronize()
            times.append((time.perf_counter() - t0) / steps * 1e3)
        it.close()
        out["e2e_ms"] = min(times)
        out["e2e_tok_s"] = batch * 1e3 / min(times)
        out["e2e_trials_ms"] = [round(t, 4) for t in times]
        return out
    trials = plan_trials(context, longest, steps, warmup, trials)
    slots = [cache.admit() for _ in prompts]
    logits = model.step(cache, slots, prompts, "last")
    first = engine.sampler.sample(logits).tolist()
    dec = decoder if decoder is not None else GraphDecoder(model, cache)
    dec.run(slots, first)
    n_fast = context - longest - 1 - trials * steps - warmup
    for _ in range(n_fast + warmup):
        dec.run(slots, None)
    torch.cuda.synchronize()
    times, kv = [], []
    if profile:
        torch.cuda.profiler.start()       # for `ncu --profile-from-start off`: only the timed steps are seen
    for _ in range(trials):
        kv_start = cache.kv_bytes(slots)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            dec.run(slots, None)
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / steps)
        kv.append((kv_start + cache.kv_bytes(slots)) / 2)
    if profile:
        torch.cuda.profiler.stop()
    best = min(range(trials), key=lambda i: times[i])
    ms = times[best]
    model.check_status()
    out.update(ms_per_step=ms, tok_s=batch * 1e3 / ms, kv_bytes=kv[best],
               weight_bytes=model.weight_bytes(), launches_per_step=dec.launches_per_step,
               mean_context=sum(cache.length(s) for s in slots) / batch,
               trials_ms=[round(t, 4) for t in times], spread=(max(times) - min(times)) / min(times))
    for s in slots:
        cache.release(s)
    out["decoder"] = dec
    return out


def prefill_run(engine, cfg, tokens: int, warmup: int, seed: int, pk: dict, block_size: int = BLOCK_SIZE):
    import torch
    model = engine.model
    cache = model.new_cache(batch_size=1, max_len=tokens, block_size=block_size)
    (prompt,) = ragged_prompts(1, tokens, tokens, model.vocab_size, seed)
    times = []
    for i in range(warmup + TRIALS):
        slot = cache.admit()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.step(cache, [slot], [prompt], "last")
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
        cache.release(slot)
    ms = min(times)
    spread = (max(times) - ms) / ms
    flops = prefill_flops(cfg, tokens)
    return {"value": tokens / ms * 1e3, "tokens": tokens, "ms": ms, "flops": flops, "spread": spread,
            "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}


def prefill_flops(cfg, tokens: int) -> float:
    L, H, I = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    lin = L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    return 2.0 * tokens * lin + 2.0 * H * cfg.vocab_size + L * 4.0 * nq * d * tokens * (tokens + 1) / 2


# ---------------------------------------------------------------------------
# the reference arm: davidjoyme/flashdecode-cuda itself, from its source tree

def find_reference():
    """(path, places tried): the first folder that holds the reference's engine/model.py and config.py."""
    tried = [ROOT / "baseline" / "_ref"]
    if os.environ.get("FLASHDECODE_REFERENCE"):
        tried.append(Path(os.environ["FLASHDECODE_REFERENCE"]))
    try:
        ref = json.loads((ROOT / "BASELINE.json").read_text()).get("reference_path")
        if ref:
            tried.append(Path(ref))
    except Exception:
        pass
    for cand in tried:
        if (cand / "engine" / "model.py").exists() and (cand / "config.py").exists():
            return cand, tried
    return None, tried


def reference_weights(raw: dict, device, dtype, seed: int):
    """Random weights under the checkpoint's names (engine/model.py:100,166,175-232 of the reference):
    matrices N(0, 0.02), norm weights 1 + N(0, 0.1), q/k/v biases N(0, 0.02); a tied head is the
    embedding table (engine/loader.py:39-40)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    H, I, V = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    nq, nkv = raw["num_attention_heads"], raw["num_key_value_heads"]
    d = raw.get("head_dim") or H // nq

    def mat(*shape, std=0.02, mean=0.0):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std + mean).to(dtype)
    w = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": mat(H, std=0.1, mean=1.0)}
    for i in range(raw["num_hidden_layers"]):
        p = f"model.layers.{i}"
        w[f"{p}.input_layernorm.weight"] = mat(H, std=0.1, mean=1.0)
        w[f"{p}.post_attention_layernorm.weight"] = mat(H, std=0.1, mean=1.0)
        for name, rows in (("q", nq * d), ("k", nkv * d), ("v", nkv * d)):
            w[f"{p}.self_attn.{name}_proj.weight"] = mat(rows, H)
            w[f"{p}.self_attn.{name}_proj.bias"] = mat(rows)
        w[f"{p}.self_attn.o_proj.weight"] = mat(H, nq * d)
        w[f"{p}.mlp.gate_proj.weight"] = mat(I, H)
        w[f"{p}.mlp.up_proj.weight"] = mat(I, H)
        w[f"{p}.mlp.down_proj.weight"] = mat(H, I)
    w["lm_head.weight"] = w["model.embed_tokens.weight"] if raw.get("tie_word_embeddings") else mat(V, H)
    return w


def reference_main(args) -> int:
    ref_root, tried = find_reference()
    if ref_root is None:
        print(json.dumps({"impl": "reference", "unavailable":
                          "no source tree of davidjoyme/flashdecode-cuda found (engine/model.py + config.py); looked at "
                          + ", ".join(str(t) for t in tried)}))
        return 0
    import torch
    from flashdecode_cuda_b200.config import preset_dict      # the sizes of the preset only: plain JSON
    raw = preset_dict(args.preset)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    on_gpu = args.device == "cuda"
    if on_gpu and not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device"}))
        return 0
    dtype = torch.bfloat16 if on_gpu else torch.float32
    sys.path.insert(0, str(ref_root))
    try:
        import config as ref_config                 # the reference's own modules, unmodified
        from engine.model import LlamaEngine
    except Exception as e:          # pragma: no cover - depends on the tree found
        print(json.dumps({"impl": "reference", "unavailable": f"the reference at {ref_root} does not import: {e!r}"[:300]}))
        return 0
    nq = raw["num_attention_heads"]
    cfg = ref_config.LlamaConfig(
        hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"],
        num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=nq,
        num_key_value_heads=raw["num_key_value_heads"], head_dim=raw.get("head_dim") or raw["hidden_size"] // nq,
        vocab_size=raw["vocab_size"], rms_norm_eps=raw["rms_norm_eps"], rope_theta=raw["rope_theta"],
        max_position_embeddings=raw["max_position_embeddings"],
        tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)), rope_scaling=None, qkv_bias=True)
    weights = reference_weights(raw, args.device, dtype, args.seed)
    eng = LlamaEngine(cfg, weights, args.device, dtype, rope_max_pos=max(8192, args.context + 64))
    warmup = max(3, args.warmup)
    sync = torch.cuda.synchronize if on_gpu else (lambda: None)

    def timed(fn, n):
        """ms per call of n calls: CUDA events on the GPU, the host clock otherwise."""
        if on_gpu:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sync()
            a.record()
            for _ in range(n):
                fn()
            b.record()
            sync()
            return a.elapsed_time(b) / n
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        return (time.perf_counter() - t0) / n * 1e3

    def decode(batch: int, steps: int, seed: int, e2e: bool, budget_s: float = 20.0):
        """The reference's decode loop at the contexts this library's own arm has when its timed steps begin:
        cache filled without a prefill the way testing/phase1.py:256-274 does, then decode_step + argmax."""
        lo, hi = args.prompt_min or args.context // 4, args.prompt_max or args.context // 2
        g = torch.Generator().manual_seed(seed)
        lens = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
        if batch > 1:
            lens[0] = hi
        trials = plan_trials(args.context, max(lens), steps, warmup, TRIALS)
        done_before = args.context - max(lens) - trials * steps - warmup          # steps this library decodes untimed
        ctx = [n + done_before for n in lens]
        cache = eng.new_paged_cache(batch, args.context + 40, block_size=BLOCK_SIZE)
        for b_, c in enumerate(ctx):
            cache.ensure_capacity([b_], extra=c)
        for i in range(cfg.num_hidden_layers):
            cache.k[i].normal_(0, 0.5)
            cache.v[i].normal_(0, 0.5)
        cache.seq_lens[:batch] = torch.tensor(ctx, dtype=torch.int32, device=cache.seq_lens.device)
        tok = torch.randint(0, cfg.vocab_size, (batch,), device=args.device)
        host = torch.empty(batch, dtype=torch.int64)
        if on_gpu:
            host = host.pin_memory()
        state = {"tok": tok}

        def step():
            if e2e:         # host token ids in from pinned memory, sampled ids out to the host, every step
                state["tok"] = host.to(args.device, non_blocking=True)
            state["tok"] = eng.decode_step(state["tok"], cache).argmax(-1)
            if e2e:
                host.copy_(state["tok"])
        with torch.inference_mode():
            host.copy_(tok)
            one = timed(step, warmup)                                  # warm-up, and a first idea of the step's time
            trials = max(1, min(trials, int(budget_s * 1e3 / max(one * steps, 1e-3))))
            times = [timed(step, steps) for _ in range(trials)]
        mean_ctx = float(cache.seq_lens[:batch].float().mean()) if trials else 0.0
        del cache
        return min(times), times, mean_ctx

    def prefill(tokens: int):
        ids = torch.randint(0, cfg.vocab_size, (1, tokens), device=args.device)
        times = []
        with torch.inference_mode():
            for i in range(2 + 3):
                cache = eng.new_paged_cache(1, tokens + 40, block_size=BLOCK_SIZE)
                t = timed(lambda: eng.prefill(ids, cache), 1)
                if i >= 2:
                    times.append(t)
                del cache
        return min(times)

    clocks = ClockSampler()
    clocks.start()
    ms, times, mean_ctx = decode(args.batch, args.steps, args.seed, e2e=False)
    line = {
        "metric": f"decode_tokens_per_s_batch{args.batch}", "value": round(args.batch * 1e3 / ms, 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "trials_ms": [round(t, 4) for t in times], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if on_gpu else "fp32 (cpu)",
        "data": "synthetic: random weights N(0, 0.02), random cache contents, token ids uniform in [0, vocab)",
        "impl": "reference",
        "ops": "the reference's stock \"ref\" ops (PyTorch); its CUDA extension builds for sm_120 only and is not used",
        "reference_path": str(ref_root),
        "config": {
            "model": args.preset, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": args.context,
            "prompt_lens": "uniform[%d,%d]" % (args.prompt_min or args.context // 4, args.prompt_max or args.context // 2),
            "mean_context": round(mean_ctx, 1), "block_size": BLOCK_SIZE, "parallelism": "1 GPU",
            "cache": "filled without a prefill, as testing/phase1.py:256-274 of the reference does",
        },
    }
    if not args.no_points:
        e_ms, e_times, _ = decode(args.batch, args.steps, args.seed, e2e=True)
        line["e2e"] = {"value": round(args.batch * 1e3 / e_ms, 1), "unit": "tok/s", "ms_per_step": round(e_ms, 4),
                       "h2d_bytes_per_step": 8 * args.batch, "d2h_bytes_per_step": 8 * args.batch}
        points = {}
        for b_ in (1, 64):
            p_ms, _, _ = decode(b_, min(args.steps, 16), args.seed + b_, e2e=False, budget_s=10.0)
            points[f"decode_b{b_}"] = round(b_ * 1e3 / p_ms, 1)
            points[f"decode_b{b_}_ms"] = round(p_ms, 4)
        line["points"] = points
        pf = prefill(2048)
        line["prefill"] = {"value": round(2048 / pf * 1e3, 1), "tokens": 2048, "ms": round(pf, 3)}
    line["clocks"] = clocks.stop()
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--preset", default="qwen2.5-1.5b")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the preset (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64, prefill and e2e")
    ap.add_argument("--prompt-min", type=int, default=0, help="shortest prompt (default context/4)")
    ap.add_argument("--prompt-max", type=int, default=0, help="longest prompt (default context/2)")
    ap.add_argument("--profile-range", action="store_true",
                    help="bracket the timed decode steps with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--prefill-only", action="store_true", help="run only the 2,048-token prefill measurement")
    ap.add_argument("--block-size", type=int, default=BLOCK_SIZE, help="tokens of a cache block of the main run")
    ap.add_argument("--no-fp32", action="store_true", help="skip the float32 point (slow at the larger presets)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the main run through the true 32-bit path (with --no-points)")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu: only for --impl reference, to try that arm on a machine without a GPU (float32)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: flashdecode_cuda_b200 is a one-GPU library; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_main(args)
    warmup = max(3, args.warmup)

    import torch
    pk = peaks()
    engine, cfg, full_layers = build_engine(args.preset, args.layers, args.seed,
                                            torch.float32 if args.dtype == "float32" else torch.bfloat16)
    clocks = ClockSampler()
    clocks.start()
    if args.prefill_only:
        if args.profile_range:
            torch.cuda.profiler.start()
        res = prefill_run(engine, cfg, 2048, 1 if args.profile_range else warmup, args.seed, pk)
        if args.profile_range:
            torch.cuda.profiler.stop()
        clocks.stop()                      # a child left running would keep a profiler waiting for it
        print(json.dumps({"prefill": res}))
        return 0
    prange = (args.prompt_min or args.context // 4, args.prompt_max or args.context // 2)
    main_run = decode_run(engine, args.batch, args.context, args.steps, warmup, args.seed, e2e=False,
                          prompt_range=prange, profile=args.profile_range, block_size=args.block_size,
                          trials=1 if args.profile_range else TRIALS)
    points, prefill, e2e = {}, None, None
    if not args.no_points:
        # the end-to-end run goes through the same cache and the decode graphs captured for it
        e2e = decode_run(engine, args.batch, args.context, args.steps, warmup, args.seed, e2e=True,
                         block_size=args.block_size, decoder=main_run["decoder"])
    del main_run["decoder"]
    if not args.no_points:
        for b in (1, 64):
            r = decode_run(engine, b, args.context, args.steps, warmup, args.seed + b, e2e=False,
                           block_size=args.block_size)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_ms"] = round(r["ms_per_step"], 4)
            points[f"decode_b{b}_hbm_frac"] = round((r["weight_bytes"] + r["kv_bytes"]) / (r["ms_per_step"] * 1e-3)
                                                    / (pk["hbm_gbs"] * 1e9), 4)
            points[f"decode_b{b}_spread"] = round(r["spread"], 4)
        prefill = prefill_run(engine, cfg, 2048, warmup, args.seed, pk, block_size=args.block_size)
        # the library's own block size beside the benchmark's
        other = LIB_BLOCK_SIZE if args.block_size != LIB_BLOCK_SIZE else BLOCK_SIZE
        r = decode_run(engine, args.batch, args.context, args.steps, warmup, args.seed, e2e=False, block_size=other)
        points[f"decode_b{args.batch}_block{other}"] = round(r["tok_s"], 1)
        points[f"decode_b{args.batch}_block{other}_ms"] = round(r["ms_per_step"], 4)
        points[f"prefill_block{other}_ms"] = round(prefill_run(engine, cfg, 2048, warmup, args.seed, pk, block_size=other)["ms"], 3)
        # the true 32-bit path (fewer steps: it is there for exactness, not for speed)
        if not args.no_fp32:
            del engine
            torch.cuda.empty_cache()
            engine32, _, _ = build_engine(args.preset, args.layers, args.seed, torch.float32)
            r = decode_run(engine32, args.batch, args.context, min(args.steps, 16), warmup, args.seed, e2e=False,
                           prompt_range=(args.context * 3 // 4, args.context - 256), block_size=args.block_size, trials=2)
            points[f"decode_b{args.batch}_fp32"] = round(r["tok_s"], 1)
            points[f"decode_b{args.batch}_fp32_ms"] = round(r["ms_per_step"], 4)
            points[f"decode_b{args.batch}_fp32_mean_context"] = round(r["mean_context"], 1)
            del engine32
    clk = clocks.stop()

    ms = main_run["ms_per_step"]
    step_bytes = main_run["weight_bytes"] + main_run["kv_bytes"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode_tokens_per_s_batch{args.batch}", "value": round(main_run["tok_s"], 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights N(0, 0.02), token ids uniform in [0, vocab)",
        "impl": "ours",
        "config": {
            "model": args.preset, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": args.context, "prompt_lens": "uniform[%d,%d]" % prange,
            "mean_context": round(main_run["mean_context"], 1), "block_size": args.block_size, "parallelism": "1 GPU",
            "l2": "each step reads %.2f GB, far beyond the 126 MB L2; no flush needed" % (step_bytes / 1e9),
            "peaks": pk["source"], "trials": "best of %d trials of %d steps" % (len(main_run["trials_ms"]), args.steps),
        },
        "trials_ms": main_run["trials_ms"], "spread": round(main_run["spread"], 4),
        "jitter": bool(main_run["spread"] > JITTER),
        "gpu_launches": int(main_run["launches_per_step"] * args.steps),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
        "clocks": clk,
    }
    if e2e:
        line["e2e"] = {"value": round(e2e["e2e_tok_s"], 1), "unit": "tok/s", "ms_per_step": round(e2e["e2e_ms"], 4),
                       "trials_ms": e2e["e2e_trials_ms"],
                       "h2d_bytes_per_step": 4 * (7 * args.batch + args.batch), "d2h_bytes_per_step": 4 * args.batch}
    if prefill:
        line["prefill"] = {"value": round(prefill["value"], 1), "tokens": prefill["tokens"],
                           "ms": round(prefill["ms"], 3), "frac": round(prefill["frac"], 4), "of": pk["source"],
                           "spread": round(prefill["spread"], 4)}
    if points:
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
