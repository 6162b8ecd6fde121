"""Weights by tensor name: checking a checkpoint against what the model's
parts declare, casting, and a seeded random-weights mode.

The checks of ``loader.validate`` in davidjoyme/flashdecode-cuda
(engine/loader.py:46-95) look at layer 0 only and raise on the first problem;
``check`` here looks at every declared tensor and raises ONE error that lists
all missing tensors, all unexpected ones and all wrong shapes.  The refusals
the reference spells out (o_proj / MLP biases, Qwen3 q_norm, :80-95) fall out
of "unexpected": a tensor no part claims is an error, never dropped silently.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Iterable, List, Optional

import torch

from .safetensors_io import read_folder, write_file
from .spec import TensorSpec


class WeightError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` hold the details that the message lists."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str], other: List[str] = ()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.other = list(wrong_shape), list(other)
        lines = ["checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def check(specs: Iterable[TensorSpec], tensors: Dict[str, torch.Tensor]) -> None:
    """Raise ``WeightError`` unless ``tensors`` holds exactly what ``specs``
    declare (optional ones may be absent), each with the declared shape."""
    specs = list(specs)
    by_name = {s.name: s for s in specs}
    missing = [s.name for s in specs if not s.optional and s.name not in tensors]
    unexpected = sorted(n for n in tensors if n not in by_name)
    wrong = []
    for s in specs:
        t = tensors.get(s.name)
        if t is not None and tuple(t.shape) != tuple(s.shape):
            wrong.append(f"{s.name}: expected {tuple(s.shape)}, got {tuple(t.shape)}")
        if t is not None and s.kind != "table" and not t.dtype.is_floating_point:
            wrong.append(f"{s.name}: expected a floating-point tensor, got {t.dtype}")
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)


def cast(spec: TensorSpec, t: torch.Tensor, dtype: torch.dtype, device) -> torch.Tensor:
    """Storage dtype of a tensor on the device.  float32 mode: everything in
    float32.  bfloat16 mode: matrices in bfloat16; a vector stored in 32-bit
    stays in 32-bit; integer tables become int32 in both modes."""
    if spec.kind == "table":
        return t.to(device=device, dtype=torch.int32).contiguous()
    if dtype == torch.float32:
        target = torch.float32
    elif spec.kind == "vector" and t.dtype in (torch.float32, torch.float64):
        target = torch.float32
    else:
        target = dtype
    return t.to(device=device, dtype=target).contiguous()


def load_checkpoint(folder) -> Dict[str, torch.Tensor]:
    """Tensors of a model folder by name, on the CPU, as stored."""
    return read_folder(Path(folder))


# ---------------------------------------------------------------------------
# random weights
# ---------------------------------------------------------------------------

def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """One tensor drawn from (seed, tensor name): the order in which tensors
    are made does not matter.  Values are drawn in float32 and rounded."""
    if spec.kind == "table":
        raise ValueError(f"{spec.name}: integer tables have no random initialiser")
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    if spec.init == "zeros":
        t = torch.zeros(spec.shape, dtype=torch.float32, device=device)
    else:
        t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
        if spec.init == "norm":
            t = 1.0 + 0.1 * t
        elif spec.init in ("normal", "bias"):
            t = 0.02 * t
        else:
            raise ValueError(f"{spec.name}: unknown initialiser {spec.init!r}")
    return t.to(dtype)


def random_tensors(specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu", skip: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    skip = set(skip)
    return {s.name: random_tensor(s, seed, dtype, device) for s in specs if s.name not in skip}


def write_model_folder(folder, config_dict: dict, tensors: Dict[str, torch.Tensor]) -> Path:
    """``config.json`` + ``model.safetensors`` in ``folder``."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config_dict, indent=1))
    write_file(folder / "model.safetensors", tensors, metadata={"format": "pt"})
    return folder
