"""flashdecode_cuda_b200: a small generation library for the Qwen2 dense
decoder on one NVIDIA B200 (sm_100a), with hand-written CUDA kernels.

    import flashdecode_cuda_b200 as fd
    engine = fd.load("/path/to/model_folder", device="cuda", dtype="bfloat16")
    results = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)

The model class is chosen by ``config.json``; see ``registry`` for adding
architectures and parts.
"""

from . import architectures, parts  # noqa: F401  (register the shipped parts and architectures)
from .config import load_config
from .engine import Engine, Model, build_model, load, random_weights, write_random_model
from .registry import register_architecture, register_part

__all__ = ["load", "load_config", "build_model", "random_weights", "write_random_model", "Engine", "Model",
           "register_architecture", "register_part"]
