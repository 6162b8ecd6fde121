"""Shared by the tests: tiny configurations, model folders in temporary
directories, the plain implementation as ground truth, error measures."""

from __future__ import annotations

import json
from functools import lru_cache
from pathlib import Path
from typing import Dict, List

import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.weights import load_checkpoint
from plain import qwen2_plain as P


def _qwen2(**kw) -> dict:
    base = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu",
            "use_sliding_window": False, "torch_dtype": "bfloat16"}
    base.update(kw)
    return base


# Tiny configurations that differ in every size and option.
TINY = {
    # 2 layers, group 2, head_dim = hidden/heads, tied head, powers of two
    "A": _qwen2(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=True, max_position_embeddings=128),
    # 3 layers, one KV head with group 3, sizes that are no power of two, separate head
    "B": _qwen2(num_hidden_layers=3, hidden_size=96, num_attention_heads=3, num_key_value_heads=1,
                head_dim=32, intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
                tie_word_embeddings=False, max_position_embeddings=256),
    # 4 layers, head_dim 48 != hidden/heads, odd vocabulary, no q/k/v bias, a window of 24 from layer 2 on
    "C": _qwen2(num_hidden_layers=4, hidden_size=80, num_attention_heads=6, num_key_value_heads=2,
                head_dim=48, intermediate_size=176, vocab_size=333, rope_theta=500000.0, rms_norm_eps=3e-6,
                tie_word_embeddings=False, max_position_embeddings=512, use_sliding_window=True,
                sliding_window=24, max_window_layers=2),
    # head_dim 64 with group 3: the size at which the tensor-core attention kernels take over
    "D": _qwen2(num_hidden_layers=2, hidden_size=128, num_attention_heads=6, num_key_value_heads=2,
                head_dim=64, intermediate_size=192, vocab_size=320, rope_theta=250000.0, rms_norm_eps=2e-6,
                tie_word_embeddings=True, max_position_embeddings=1024),
    # head_dim 128 (the tcgen05 attention and, from 128 prompt tokens on, the tcgen05 products), one KV
    # head shared by 3 query heads, a window of 40 keys on the second layer
    "E": _qwen2(num_hidden_layers=2, hidden_size=192, num_attention_heads=3, num_key_value_heads=1,
                head_dim=128, intermediate_size=320, vocab_size=288, rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=False, max_position_embeddings=1024, use_sliding_window=True,
                sliding_window=40, max_window_layers=1),
}
NO_BIAS = {"C"}


def write_folder(tmp: Path, name: str, seed: int = 0) -> Path:
    """A model folder for tiny configuration ``name`` with weights from ``seed``."""
    folder = Path(tmp) / f"tiny_{name}_{seed}"
    if not (folder / "model.safetensors").exists():
        fd.write_random_model(folder, TINY[name], seed, qkv_bias=name not in NO_BIAS)
    return folder


def raw_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


def weights_of(folder: Path) -> Dict[str, torch.Tensor]:
    return {k: v.clone() for k, v in load_checkpoint(folder).items()}


def prompts_for(vocab: int, lengths: List[int], seed: int = 0) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


_ORACLE: dict = {}


def oracle_logits(folder: Path, tokens: List[int]) -> torch.Tensor:
    """float64 logits [len, vocab] of one whole sequence from the plain implementation."""
    key = (str(folder), tuple(tokens))
    if key not in _ORACLE:
        _ORACLE[key] = P.logits(raw_config(folder), weights_of(folder), tokens)
    return _ORACLE[key]


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| relative to the scale of ``want`` (its largest magnitude)."""
    got, want = got.detach().double().cpu(), want.detach().double().cpu()
    scale = max(float(want.abs().max()), 1e-6)
    return float((got - want).abs().max()) / scale


# Relative to the scale of the logits.  Set from what the replay tests measure (tests/test_trace_run_gpu.py prints
# its worst error: 9.5e-7 in float32, where only the order of summation differs from the float64 ground truth, and
# 8.3e-3 in bfloat16), with a factor of about ten and 2.4 over them; 2e-2 is also the gate of the reference's own
# layer-by-layer diff (testing/diff.py:44-50,113).
TOL = {"float32": 1e-5, "bfloat16": 2e-2}
