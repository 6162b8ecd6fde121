"""Plain, slow implementation of the Qwen2 dense decoder: whole sequences, no
cache, one function per part.  It shares no code with the product package; it
reads a raw ``config.json`` dictionary and a ``{tensor name: tensor}`` dict.

Every function cites the place in davidjoyme/flashdecode-cuda whose formula it
restates (paths are relative to that project's root).  The arithmetic dtype is
a parameter (float64 by default) so the same text serves as a ground truth for
the engine's float32 and bfloat16 paths.  The rotation angles are always built
in float32, as the reference builds them, and then cast.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ---------------------------------------------------------------------------
# configuration helpers (plain dictionary access; nothing typed on purpose)
# ---------------------------------------------------------------------------

def head_dim_of(cfg: dict) -> int:
    """``head_dim`` if given, else hidden/heads (config.py:122)."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


def rope_theta_of(cfg: dict) -> float:
    """Flat ``rope_theta`` or ``rope_parameters.rope_theta`` (config.py:99-118)."""
    if cfg.get("rope_theta") is not None:
        return float(cfg["rope_theta"])
    params = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
    return float(params["rope_theta"])


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """Sliding window of a layer, or None for full attention.

    The reference never reads these keys (it has no window).  The meaning is
    the one the keys' names carry in a Qwen2 ``config.json``: with
    ``use_sliding_window`` true, layers with index >= ``max_window_layers``
    see only the last ``sliding_window`` keys (the query's own included).
    """
    if not cfg.get("use_sliding_window", False):
        return None
    if layer < int(cfg.get("max_window_layers", cfg["num_hidden_layers"])):
        return None
    return int(cfg["sliding_window"])


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------

def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h = W_E[ids], no scaling (engine/model.py:166,255)."""
    return table[ids]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps); out = weight * y (engine/ops.py:61-72).

    The reference casts y back to the input dtype before the weight multiply;
    in one dtype throughout that cast is the identity.
    """
    var = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(var + eps))


def rope_tables(head_dim: int, n_pos: int, theta: float):
    """cos/sin [n_pos, head_dim] in float32 (engine/ops.py:102-110).

    inv_freq_j = 1 / theta^(2j/d); angle[p, j] = p * inv_freq_j computed in
    float32; the table repeats the d/2 angles twice (rotate-half pairing).
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    t = torch.arange(n_pos).float()
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """cat(-x[d/2:], x[:d/2]) (engine/ops.py:132-134)."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x' = x*cos + rotate_half(x)*sin; x [S, heads, d], cos/sin [S, d]
    (engine/model.py:195-197, engine/ops.py:137-146)."""
    c = cos[:, None, :].to(x.dtype)
    s = sin[:, None, :].to(x.dtype)
    return x * c + rotate_half(x) * s


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                         scale: float, window: Optional[int]) -> torch.Tensor:
    """q [S, n_q, d], k/v [S, n_kv, d] -> [S, n_q, d].

    Query head h reads KV head h // G (engine/ops.py:180-185,
    engine/model.py:201-202); scores = scale * q.k, causal mask t <= p
    (engine/model.py:203-205), softmax over keys, weighted sum of values
    (engine/ops.py:185-193).  ``window`` additionally hides keys with
    p - t >= window.
    """
    S, n_q, d = q.shape
    n_kv = k.shape[1]
    G = n_q // n_kv
    out = torch.empty_like(q)
    pos = torch.arange(S)
    visible = pos[None, :] <= pos[:, None]                     # [p, t]
    if window is not None:
        visible &= (pos[:, None] - pos[None, :]) < window
    for h in range(n_q):
        kh = h // G
        scores = (q[:, h, :] @ k[:, kh, :].T) * scale            # [p, t]
        scores = scores.masked_fill(~visible, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ v[:, kh, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up, silu(x) = x * sigmoid(x) (engine/ops.py:201-204)."""
    return gate * torch.sigmoid(gate) * up


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x W^T + b with W [out, in] (engine/model.py:188-190)."""
    y = x @ w.T
    return y if b is None else y + b


# ---------------------------------------------------------------------------
# blocks and the whole model
# ---------------------------------------------------------------------------

def attention_block(cfg: dict, w: Dict[str, torch.Tensor], layer: int,
                    hn: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """q/k/v projections with optional bias, RoPE on q and k, causal GQA
    attention, output projection without bias (engine/model.py:188-208)."""
    p = f"model.layers.{layer}.self_attn"
    S = hn.shape[0]
    d = head_dim_of(cfg)
    n_q, n_kv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    q = linear(hn, w[f"{p}.q_proj.weight"], w.get(f"{p}.q_proj.bias")).view(S, n_q, d)
    k = linear(hn, w[f"{p}.k_proj.weight"], w.get(f"{p}.k_proj.bias")).view(S, n_kv, d)
    v = linear(hn, w[f"{p}.v_proj.weight"], w.get(f"{p}.v_proj.bias")).view(S, n_kv, d)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_gqa_attention(q, k, v, 1.0 / math.sqrt(d), layer_window(cfg, layer))
    return linear(o.reshape(S, n_q * d), w[f"{p}.o_proj.weight"])


def mlp_block(w: Dict[str, torch.Tensor], layer: int, hn: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) (engine/model.py:213-216)."""
    p = f"model.layers.{layer}.mlp"
    return linear(swiglu(linear(hn, w[f"{p}.gate_proj.weight"]),
                         linear(hn, w[f"{p}.up_proj.weight"])),
                  w[f"{p}.down_proj.weight"])


def hidden_states(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
                  dtype=torch.float64, trace: Optional[dict] = None) -> torch.Tensor:
    """Final-normed hidden rows [S, H] of one whole sequence.

    Pre-norm decoder: x += attn(norm(x)); x += mlp(norm(x)); final norm
    (engine/model.py:173-227; its deferred-add threading equals this form).
    """
    w = {k: v.to(dtype) for k, v in weights.items()}
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    S = ids.numel()
    eps = float(cfg["rms_norm_eps"])
    cos, sin = rope_tables(head_dim_of(cfg), S, rope_theta_of(cfg))
    x = embedding(ids, w["model.embed_tokens.weight"])
    if trace is not None:
        trace["embed"] = x.clone()
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        x = x + attention_block(cfg, w, i, rmsnorm(x, w[f"{p}.input_layernorm.weight"], eps), cos, sin)
        x = x + mlp_block(w, i, rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], eps))
        if trace is not None:
            trace[f"layer.{i}"] = x.clone()
    return rmsnorm(x, w["model.norm.weight"], eps)


def logits(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int],
           dtype=torch.float64) -> torch.Tensor:
    """Logits [S, V] at every position of one whole sequence.  The output
    head is ``lm_head.weight`` or, when the checkpoint has none, the
    embedding table (engine/loader.py:39-40, engine/model.py:229-234)."""
    hn = hidden_states(cfg, weights, tokens, dtype)
    head = weights.get("lm_head.weight")
    if head is None:
        head = weights["model.embed_tokens.weight"]
    return linear(hn, head.to(dtype))


# ---------------------------------------------------------------------------
# sampling: greedy, and temperature by the Gumbel-max rule with Philox noise
# ---------------------------------------------------------------------------

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32(counter: Sequence[int], key: Sequence[int]) -> List[int]:
    """Philox-4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as
    easy as 1, 2, 3"), scalar form."""
    c0, c1, c2, c3 = [int(c) & _MASK for c in counter]
    k0, k1 = [int(k) & _MASK for k in key]
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, \
                         ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return [c0, c1, c2, c3]


def gumbel_noise(vocab: int, seed: int, request: int, step: int) -> torch.Tensor:
    """float32 [vocab]: g_i = -log(-log(u_i)); u_i = ((x_i >> 9) + 0.5) / 2^23
    with x_{4j..4j+3} = philox(counter=(j, step, request_lo, request_hi),
    key=(seed_lo, seed_hi)).  A draw depends only on (seed, request, step,
    vocabulary index), never on batch neighbours."""
    out = torch.empty(vocab, dtype=torch.float32)
    key = (seed & _MASK, (seed >> 32) & _MASK)
    for j in range((vocab + 3) // 4):
        xs = philox4x32((j, step, request & _MASK, (request >> 32) & _MASK), key)
        for r, x in enumerate(xs):
            if 4 * j + r < vocab:
                out[4 * j + r] = ((x >> 9) + 0.5) / 8388608.0
    return -torch.log(-torch.log(out))


def sample(logits_row: torch.Tensor, temperature: float, seed: int, request: int, step: int) -> int:
    """Greedy argmax for temperature 0 (engine/model.py:324,327; the lowest
    index wins a tie); else argmax(logits/T + gumbel) in float32."""
    row = logits_row.to(torch.float32)
    if temperature <= 0.0:
        score = row
    else:
        score = row / torch.tensor(temperature, dtype=torch.float32) + \
            gumbel_noise(row.numel(), seed, request, step)
    best = score.max()
    return int(torch.nonzero(score == best)[0, 0])


def generate(cfg: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int],
             max_new_tokens: int, temperature: float = 0.0, seed: int = 0, request: int = 0,
             stop_token_ids: Sequence[int] = (), dtype=torch.float64) -> List[int]:
    """Recompute the whole sequence for every new token (no cache).  The stop
    token is kept in the output and ends the sequence."""
    seq = list(prompt)
    out: List[int] = []
    for step in range(max_new_tokens):
        tok = sample(logits(cfg, weights, seq, dtype)[-1], temperature, seed, request, step)
        out.append(tok)
        seq.append(tok)
        if tok in stop_token_ids:
            break
    return out
