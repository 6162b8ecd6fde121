"""The Python entry point: load a model folder, generate.

In the manner of davidjoyme/flashdecode-cuda, where a user writes
``cfg, w = loader.load(model_id, device, dtype)``, ``eng = LlamaEngine(cfg, w,
device, dtype)``, ``cache = eng.new_paged_cache(batch_size, max_len,
block_size)`` and ``eng.generate(input_ids, max_new_tokens, cache)``
(engine/loader.py:12, engine/model.py:75,115,316): the same names and meanings,
with the model chosen by ``config.json`` and with what that engine lacks
(unequal prompts, stop tokens, temperature, several batches).
"""

from __future__ import annotations

import time
from pathlib import Path
from typing import Dict, Iterator, List, Optional, Sequence, Tuple, Union

import torch

from .. import kernels as K
from ..cache.paged import DEFAULT_BLOCK_SIZE, PagedCache
from ..config import load_config
from ..sampling.sampler import Sampler
from ..weights import loader as W
from .decode import GraphDecoder
from .generate import Backend, GenerationLoop, Request, Result
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def as_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}") from None


class Engine(Backend):
    """A bound model with a sampler; the object ``load`` returns."""

    def __init__(self, model: Model):
        self.model = model
        self.config = model.config
        self.device, self.dtype = model.device, model.dtype
        self.sampler = Sampler(model.device)
        self.cache: Optional[PagedCache] = None
        self.seed = 0
        # decode steps replay captured CUDA graphs unless a part decides on the host
        self.use_graphs = model.device.type == "cuda" and model.graph_safe
        self._graph_decoder: Optional[GraphDecoder] = None
        self._own_cache: Optional[PagedCache] = None       # the cache made by a call that was given none

    # -- caches -----------------------------------------------------------
    def new_paged_cache(self, batch_size: int, max_len: int, block_size: int = DEFAULT_BLOCK_SIZE,
                        slack_blocks: int = 8) -> PagedCache:
        """A cache for ``batch_size`` sequences of up to ``max_len`` tokens
        (engine/model.py:115-135 of the reference, same arguments)."""
        return self.model.new_cache(batch_size=batch_size, max_len=max_len, block_size=block_size,
                                    slack_blocks=slack_blocks)

    def new_cache(self, max_tokens: int, block_size: int = DEFAULT_BLOCK_SIZE, **kw) -> PagedCache:
        return self.model.new_cache(max_tokens, block_size=block_size, **kw)

    # -- Backend of the generation loop -------------------------------------
    def capacity(self) -> Tuple[int, int]:
        c = self.cache
        return c.max_slots, c.num_blocks * c.block_size

    def tokens_held(self, n_tokens: int) -> int:
        bs = self.cache.block_size
        return -(-n_tokens // bs) * bs

    def admit(self) -> int:
        return self.cache.admit()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def run(self, slots, tokens, requests, steps) -> List[int]:
        temps = [r.temperature for r in requests]
        rids = [r.request_id for r in requests]
        if self.use_graphs and all(len(t) == 1 for t in tokens):
            dec = self._decoder()
            dec.run(slots, [t[0] for t in tokens], temps, rids, steps, self.seed)
            return dec.read_tokens(len(slots))
        logits = self.model.step(self.cache, slots, tokens, "last")
        toks = self.sampler.sample(logits, temps, rids, steps, self.seed)
        return toks.tolist()

    def _decoder(self) -> GraphDecoder:
        if self._graph_decoder is None or self._graph_decoder.cache is not self.cache:
            self._graph_decoder = GraphDecoder(self.model, self.cache)
        return self._graph_decoder

    def use_decoder(self, decoder: GraphDecoder) -> None:
        """Decode steps over ``decoder.cache`` go through this decoder from now on, with the graphs it has captured
        already (a graph is tied to its cache's tensors; capturing one costs tens of milliseconds).  Pass that cache to
        ``generate`` / ``stream``."""
        if decoder.model is not self.model:
            raise ValueError("the decoder belongs to another model")
        self._graph_decoder = decoder

    # -- generation ---------------------------------------------------------
    def _requests(self, input_ids, max_new_tokens, temperature, stop_token_ids) -> List[Request]:
        if isinstance(input_ids, torch.Tensor):
            prompts = input_ids.tolist()
            if input_ids.dim() == 1:
                prompts = [prompts]
        else:
            prompts = [list(map(int, p)) for p in input_ids]
        if stop_token_ids is None:
            stop_token_ids = ()
        n = len(prompts)
        mx = max_new_tokens if isinstance(max_new_tokens, (list, tuple)) else [max_new_tokens] * n
        tp = temperature if isinstance(temperature, (list, tuple)) else [temperature] * n
        return [Request(p, int(m), float(t), tuple(int(s) for s in stop_token_ids), i)
                for i, (p, m, t) in enumerate(zip(prompts, mx, tp))]

    def _ensure_cache(self, requests: Sequence[Request], cache, max_batch, block_size) -> int:
        max_batch = max_batch or min(len(requests), 64)
        if cache is None:
            longest = max(len(r.prompt) + r.max_new_tokens for r in requests)
            own = self._own_cache
            # the cache this engine made for an earlier call serves again if it is large enough and empty: no new
            # allocation, and the decode graphs captured over it are used again instead of being captured anew
            if (own is not None and own.block_size == block_size and own.max_slots >= max_batch
                    and own.max_len >= longest and not own.active_slots()):
                cache = own
            else:
                cache = self._own_cache = self.new_paged_cache(max_batch, longest, block_size)
        self.cache = cache
        return max_batch

    def generate(self, input_ids, max_new_tokens, cache: Optional[PagedCache] = None, *,
                 temperature=0.0, seed: int = 0, stop_token_ids: Optional[Sequence[int]] = None,
                 max_batch: Optional[int] = None, block_size: int = DEFAULT_BLOCK_SIZE):
        """Generate up to ``max_new_tokens`` tokens for every prompt.

        ``input_ids``: a [B, S] tensor (the reference's form; returns a
        [B, max_new_tokens] int64 tensor, positions after an early stop filled
        with -1) or a list of token lists of unequal lengths (returns a list of
        ``Result``).  ``temperature`` 0 is greedy.  More prompts than
        ``max_batch`` run as several batches on the same cache."""
        requests = self._requests(input_ids, max_new_tokens, temperature, stop_token_ids)
        max_batch = self._ensure_cache(requests, cache, max_batch, block_size)
        self.seed = seed
        results = GenerationLoop(self, max_batch).run(requests)
        if isinstance(input_ids, torch.Tensor):
            width = max(r.max_new_tokens for r in requests)
            out = torch.full((len(results), width), -1, dtype=torch.int64)
            for i, r in enumerate(results):
                out[i, :len(r.tokens)] = torch.tensor(r.tokens, dtype=torch.int64)
            return out
        return results

    def stream(self, input_ids, max_new_tokens, cache: Optional[PagedCache] = None, *, temperature=0.0,
               seed: int = 0, stop_token_ids: Optional[Sequence[int]] = None, max_batch: Optional[int] = None,
               block_size: int = DEFAULT_BLOCK_SIZE) -> Iterator[List[Tuple[int, int, Optional[str]]]]:
        """Like ``generate`` but yields, step by step, the new token of every
        live sequence as host integers: (prompt index, token, finish reason)."""
        requests = self._requests(input_ids, max_new_tokens, temperature, stop_token_ids)
        max_batch = self._ensure_cache(requests, cache, max_batch, block_size)
        self.seed = seed
        return GenerationLoop(self, max_batch).events(requests)

    def step(self, cache, slots, tokens, want="last"):
        return self.model.step(cache, slots, tokens, want)


def build_model(config, tensors: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16) -> Model:
    model = Model.from_config(config, as_dtype(dtype), device)
    return model.bind(tensors)


def load(model: Union[str, Path], device="cuda", dtype=torch.bfloat16, seed: Optional[int] = None) -> Engine:
    """An engine for a model folder (``config.json`` + ``model.safetensors``);
    the model class is chosen by ``config.json["architectures"]``.  With
    ``seed`` given, ``model`` may instead name a preset (or a folder with only a
    ``config.json``) and the weights are drawn at random from the seed."""
    dtype = as_dtype(dtype)
    config = load_config(model)
    m = Model.from_config(config, dtype, device)
    folder = Path(model)
    has_weights = folder.is_dir() and ((folder / "model.safetensors").exists() or
                                       (folder / "model.safetensors.index.json").exists())
    if has_weights:
        tensors = W.load_checkpoint(folder)
    elif seed is not None:
        dev = device if torch.device(device).type == "cuda" else "cpu"
        tensors = random_weights(m, seed, device=dev)
    else:
        raise FileNotFoundError(f"{model}: no model.safetensors (give seed= to draw random weights)")
    m.bind(tensors)
    return Engine(m)


def random_weights(model: Model, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                   qkv_bias: bool = True) -> Dict[str, torch.Tensor]:
    """Every tensor the model declares, drawn from (seed, tensor name).
    Optional tensors (the q/k/v biases) are drawn unless ``qkv_bias`` is off."""
    specs = [s for s in model.tensor_specs() if qkv_bias or not s.optional]
    return W.random_tensors(specs, seed, dtype, device)


def write_random_model(folder, config_source, seed: int, dtype=torch.bfloat16, qkv_bias: bool = True) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a configuration
    (preset name, dictionary, folder) with weights drawn from ``seed``."""
    config = load_config(config_source)
    model = Model.from_config(config, torch.float32, "cpu")
    tensors = random_weights(model, seed, as_dtype(dtype), "cpu", qkv_bias)
    return W.write_model_folder(folder, config.to_dict(), tensors)
