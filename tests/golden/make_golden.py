#!/usr/bin/env python3
"""Makes tests/golden/reference_logits.safetensors: logits of
davidjoyme/flashdecode-cuda's own engine (engine/model.py, run on the CPU in
float32) for two tiny random Qwen2 models.  tests/test_plain.py compares the
plain implementation with them, so the plain implementation rests on the
reference's code as well as on its formulas.

    FLASHDECODE_REFERENCE=<checkout of davidjoyme/flashdecode-cuda> python tests/golden/make_golden.py

The weights are this repository's seeded random weights (bfloat16 values, so
both sides see identical numbers); the reference engine gets them as float32
tensors under the checkpoint's own names.  For each prompt the file holds the
last-position logits of ``prefill`` on several prefixes and the logits of
``decode_step`` for the tokens after the shortest prefix.
"""

import json
import os
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

CASES = {"A": ([5, 11, 17], 21), "B": ([1, 7, 16, 33], 22)}      # prompt lengths, weight seed


def main() -> int:
    ref = os.environ.get("FLASHDECODE_REFERENCE")
    if not ref or not (Path(ref) / "engine" / "model.py").exists():
        print("set FLASHDECODE_REFERENCE to a checkout of davidjoyme/flashdecode-cuda", file=sys.stderr)
        return 1
    sys.path.insert(0, ref)
    sys.dont_write_bytecode = True
    from config import LlamaConfig                      # the reference's modules
    from engine.model import LlamaEngine
    import flashdecode_cuda_b200 as fd
    from flashdecode_cuda_b200.weights import load_checkpoint, write_file
    from helpers import TINY, prompts_for

    out, meta = {}, {}
    for name, (lengths, seed) in CASES.items():
        raw = TINY[name]
        with tempfile.TemporaryDirectory() as d:
            fd.write_random_model(d, raw, seed)
            weights = {k: v.float() for k, v in load_checkpoint(d).items()}
        head_dim = raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"]
        cfg = LlamaConfig(hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"],
                          num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=raw["num_attention_heads"],
                          num_key_value_heads=raw["num_key_value_heads"], head_dim=head_dim,
                          vocab_size=raw["vocab_size"], rms_norm_eps=raw["rms_norm_eps"], rope_theta=raw["rope_theta"],
                          max_position_embeddings=raw["max_position_embeddings"],
                          tie_word_embeddings=raw["tie_word_embeddings"], qkv_bias=True)
        if "lm_head.weight" not in weights:
            weights["lm_head.weight"] = weights["model.embed_tokens.weight"]     # engine/loader.py:39-40
        eng = LlamaEngine(cfg, weights, "cpu", torch.float32, rope_max_pos=cfg.max_position_embeddings)
        prompts = prompts_for(raw["vocab_size"], lengths, seed=seed)
        meta[name] = {"seed": seed, "prompts": prompts}
        for i, p in enumerate(prompts):
            ids = torch.tensor([p])
            for n in sorted({1, max(1, len(p) // 2), len(p)}):
                cache = eng.new_cache(1, len(p) + 2)
                out[f"{name}.{i}.prefill.{n}"] = eng.prefill(ids[:, :n], cache)[0].clone()
            cache = eng.new_cache(1, len(p) + 2)
            eng.prefill(ids[:, :1], cache)
            for t in range(1, len(p)):
                out[f"{name}.{i}.decode.{t}"] = eng.decode_step(ids[:, t], cache)[0].clone()
    write_file(HERE / "reference_logits.safetensors", out)
    (HERE / "reference_logits.json").write_text(json.dumps(meta))
    print(f"wrote {len(out)} logit rows")
    return 0


if __name__ == "__main__":
    sys.exit(main())
