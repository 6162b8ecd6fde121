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

Peaks come from MEASURED_PEAKS.json beside this file when present, else from
the stated fallback.  Only one GPU is used: for --gpus > 1 it says so and exits
with 2.  ``--impl reference``: davidjoyme/flashdecode-cuda cannot be installed
offline (it has no build file at its root), so that arm prints ``unavailable``.
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

BLOCK_SIZE = int(os.environ.get("FD_BLOCK_SIZE", "64"))      # tokens of a cache block (the library's default)
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


def build_engine(preset: str, layers: int, seed: int):
    import torch
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
    model = Model.from_config(cfg, torch.bfloat16, "cuda")
    model.bind(random_weights(model, seed, torch.bfloat16, device="cuda"))
    return Engine(model), cfg, full_layers


def ragged_prompts(batch: int, lo: int, hi: int, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    if batch > 1:
        lens[0] = hi            # the longest prompt is as long as allowed, so the context bound is reached
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def decode_run(engine, batch: int, context: int, steps: int, warmup: int, seed: int, e2e: bool,
               prompt_range=None, profile: bool = False):
    """Prefill ragged prompts, decode untimed until ``steps + warmup`` steps are
    left before the longest sequence reaches ``context``, then time."""
    import torch
    from flashdecode_cuda_b200 import kernels as K
    from flashdecode_cuda_b200.engine.decode import GraphDecoder
    model = engine.model
    vocab = model.vocab_size
    lo, hi = prompt_range or (context // 4, context // 2)
    prompts = ragged_prompts(batch, lo, hi, vocab, seed)
    cache = model.new_cache(batch_size=batch, max_len=context, block_size=BLOCK_SIZE)
    out = {}
    if e2e:
        # the public entry point: host token ids in, host token ids out, every step
        total_new = context - max(len(p) for p in prompts)
        it = engine.stream(prompts, total_new, cache, max_batch=batch)
        n_fast = total_new - steps - warmup
        for _ in range(n_fast):
            next(it)
        torch.cuda.synchronize()
        for _ in range(warmup):
            next(it)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            ev = next(it)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        it.close()
        out["e2e_tok_s"] = batch * steps / dt
        out["e2e_ms"] = dt / steps * 1e3
        return out
    slots = [cache.admit() for _ in prompts]
    logits = model.step(cache, slots, prompts, "last")
    first = engine.sampler.sample(logits).tolist()
    dec = GraphDecoder(model, cache)
    dec.run(slots, first)
    n_fast = context - max(len(p) for p in prompts) - 1 - steps - warmup
    for _ in range(n_fast + warmup):
        dec.run(slots, None)
    torch.cuda.synchronize()
    kv_start = cache.kv_bytes(slots)
    K.LAUNCHES = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if profile:
        torch.cuda.profiler.start()       # for `ncu --profile-from-start off`: only the timed steps are seen
    start.record()
    for _ in range(steps):
        dec.run(slots, None)
    end.record()
    torch.cuda.synchronize()
    if profile:
        torch.cuda.profiler.stop()
    ms = start.elapsed_time(end) / steps
    kv_end = cache.kv_bytes(slots)
    model.check_status()
    out.update(ms_per_step=ms, tok_s=batch * 1e3 / ms, kv_bytes=(kv_start + kv_end) / 2,
               weight_bytes=model.weight_bytes(), launches_per_step=dec.launches_per_step,
               mean_context=sum(cache.length(s) for s in slots) / batch)
    for s in slots:
        cache.release(s)
    return out


def prefill_run(engine, cfg, tokens: int, warmup: int, seed: int, pk: dict):
    import torch
    model = engine.model
    cache = model.new_cache(batch_size=1, max_len=tokens, block_size=BLOCK_SIZE)
    (prompt,) = ragged_prompts(1, tokens, tokens, model.vocab_size, seed)
    times = []
    for i in range(warmup + 3):
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
    L, H, I = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
    nq, nkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    lin = L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    flops = 2.0 * tokens * lin + 2.0 * H * cfg.vocab_size + L * 4.0 * nq * d * tokens * (tokens + 1) / 2
    return {"value": tokens / ms * 1e3, "tokens": tokens, "ms": ms, "flops": flops,
            "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}


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
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "davidjoyme/flashdecode-cuda has no setup.py or pyproject.toml at its root, so the "
                          "offline pip install into baseline/_ref fails; it also builds for sm_120 only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: flashdecode_cuda_b200 is a one-GPU library; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)

    import torch
    pk = peaks()
    engine, cfg, full_layers = build_engine(args.preset, args.layers, args.seed)
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
                          prompt_range=prange, profile=args.profile_range)
    points, prefill, e2e = {}, None, None
    if not args.no_points:
        e2e = decode_run(engine, args.batch, args.context, args.steps, warmup, args.seed, e2e=True)
        for b in (1, 64):
            r = decode_run(engine, b, args.context, args.steps, warmup, args.seed + b, e2e=False)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            points[f"decode_b{b}_ms"] = round(r["ms_per_step"], 4)
            points[f"decode_b{b}_hbm_frac"] = round((r["weight_bytes"] + r["kv_bytes"]) / (r["ms_per_step"] * 1e-3)
                                                    / (pk["hbm_gbs"] * 1e9), 4)
        prefill = prefill_run(engine, cfg, 2048, warmup, args.seed, pk)
    clk = clocks.stop()

    ms = main_run["ms_per_step"]
    step_bytes = main_run["weight_bytes"] + main_run["kv_bytes"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode_tokens_per_s_batch{args.batch}", "value": round(main_run["tok_s"], 1), "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random bf16 weights N(0, 0.02), token ids uniform in [0, vocab)",
        "impl": "ours",
        "config": {
            "model": args.preset, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "seq_len": args.context, "prompt_lens": "uniform[%d,%d]" % prange,
            "mean_context": round(main_run["mean_context"], 1), "block_size": BLOCK_SIZE, "parallelism": "1 GPU",
            "l2": "each step reads %.2f GB, far beyond the 126 MB L2; no flush needed" % (step_bytes / 1e9),
            "peaks": pk["source"],
        },
        "gpu_launches": int(main_run["launches_per_step"] * args.steps),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
        "clocks": clk,
    }
    if e2e:
        line["e2e"] = {"value": round(e2e["e2e_tok_s"], 1), "unit": "tok/s", "ms_per_step": round(e2e["e2e_ms"], 4),
                       "h2d_bytes_per_step": 4 * (7 * args.batch + args.batch), "d2h_bytes_per_step": 4 * args.batch}
    if prefill:
        line["prefill"] = {"value": round(prefill["value"], 1), "tokens": prefill["tokens"],
                           "ms": round(prefill["ms"], 3), "frac": round(prefill["frac"], 4), "of": pk["source"]}
    if points:
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
