"""Python side of the CUDA kernel library: one thin function per launcher.

The role of ``engine/ops_cuda.py`` + ``kernels/bindings.cpp`` in
davidjoyme/flashdecode-cuda (bindings.cpp:24-63,79-164), without an op
registry or an alternative backend: these functions are the only
implementation, they check what the kernels assume (device, dtype,
contiguity) and raise with the kernel library's own message when a launcher
refuses a size.  There is no CPU path; importing this module on a machine
without the built library builds it, and calling any function without a CUDA
device fails.

Tensors are passed as raw pointers on torch's current stream, so launches are
ordered with torch's own work and can be captured into a CUDA graph.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

STATUS_BAD_TOKEN = 1
STATUS_BAD_BLOCK = 2
STATUS_BAD_POSITION = 4
STATUS_WAIT_TIMEOUT = 8
_STATUS_TEXT = {
    STATUS_BAD_TOKEN: "a token id lies outside the embedding table",
    STATUS_BAD_BLOCK: "a cached token maps to no allocated block",
    STATUS_BAD_POSITION: "a position lies beyond the rotation table",
    STATUS_WAIT_TIMEOUT: "a bounded wait inside a kernel ran out",
}

_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    """A launcher refused its arguments or a launch failed."""


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return 0
    if t == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t}")


def lib() -> ctypes.CDLL:
    """The loaded kernel library; built on first use if it is missing or stale."""
    global _lib
    if _lib is None:
        path = _build.build()
        try:
            _lib = ctypes.CDLL(str(path))
        except OSError as e:  # pragma: no cover - environment failure
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from e
        _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    P, I, F, LL = c_void_p, c_int, c_float, c_longlong
    L.fd_last_error.restype = ctypes.c_char_p
    L.fd_last_error.argtypes = []
    sigs = {
        "fd_device_arch": [],
        "fd_set_pdl": [I],
        "fd_sm_count": [],
        "fd_embed": [P, P, I, P, I, I, I, P, P],
        "fd_add_rmsnorm": [P, I, I, LL, P, I, P, I, F, P, I, P, I, I, P],
        "fd_silu_mul": [P, P, I, I, I, I, P],
        "fd_rope_append": [P, I, I, LL, P, I, P, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
        "fd_gemv_qkv_rope": [P, P, P, I, P, I, I, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P, c_ulonglong, P],
        "fd_gemm_tc_supported": [I, I, I],
        "fd_gemm_tc_set_wide": [I],
        "fd_attn_prefill_set_form": [I],
        "fd_attn_decode_set_form": [I],
        "fd_gemm_tc": [P, P, P, I, P, I, I, I, I, P, P],
        "fd_gemm_tc_qkv_rope": [P, P, P, I, P, I, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
        "fd_gemm_stream_splits": [I, I, I],
        "fd_gemm_stream_force_2d": [I],
        "fd_gemm_stream_set_pdl": [I],
        "fd_gemm_stream_last_map3d": [],
        "fd_gemm_stream": [P, P, P, I, P, I, I, I, I, I, P, P],
        "fd_gemm_stream_qkv_rope": [P, P, P, I, P, I, I, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
        "fd_tc_test_hook": [LL, I],
        "fd_gemv_splits": [I, I, I, I, I],
        "fd_gemv": [P, P, P, I, P, I, I, I, I, I, P, c_ulonglong, P],
        "fd_gemm_simt": [P, P, P, P, I, I, I, I, I, I, P],
        "fd_attn_simt_qt": [I],
        "fd_attention_simt": [P, P, P, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P, P, P],
        "fd_attention": [P, P, P, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P, P, P, P, c_ulonglong, P],
        "fd_attention_mma_sync": [P, P, P, P, I, P, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, I, I, I, P, P, P, P],
        "fd_sample": [P, I, I, P, P, P, c_ulonglong, P, P, P, P],
        "fd_copy_h2d_async": [P, P, LL, P],
        "fd_copy_d2h_sync": [P, P, LL, P],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = I
    L.fd_attn_scratch_floats.argtypes = [I, I, I, I]
    L.fd_launch_count.restype = c_ulonglong
    L.fd_launch_count.argtypes = []
    L.fd_attn_scratch_floats.restype = LL
    L.fd_sample_scratch_words.argtypes = [I, I]
    L.fd_sample_scratch_words.restype = LL


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(lib().fd_last_error().decode())


def launch_count() -> int:
    """Kernels of this library launched so far by this process, counted where they are launched (a kernel
    captured into a graph counts once, at capture)."""
    return int(lib().fd_launch_count())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  torch's own accessor for the raw handle costs a fraction of a microsecond;
    ``torch.cuda.current_stream()`` builds a Stream object each time (about 5 us), which in a prompt step of some
    250 launches was a sixth of the host's time."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors only; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    return t.data_ptr()


def require_device() -> None:
    """Fail loudly unless a CUDA device of compute capability 10.x is current."""
    if not torch.cuda.is_available():
        raise KernelError("flashdecode_cuda_b200 needs a CUDA device (B200, sm_100a); none is available "
                          "and there is no CPU fallback")
    arch = lib().fd_device_arch()
    if arch < 0:
        _check(arch)
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a only; this device is sm_{arch}")


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for this library's kernels: a kernel may start, and fetch
    weights, while the previous one is still finishing.  Off by default: measured on B200 inside
    the captured decode graph every programmatic edge made the step slower (all kernels: 2.34
    against 1.46 ms at batch 8; a single kind of product per layer: 1.50 to 1.62 ms)."""
    lib().fd_set_pdl(int(on))


def copy_h2d_async(dst: torch.Tensor, src_pinned: torch.Tensor, n_elements: int) -> None:
    """dst[:n] <- src[:n] from pinned host memory, asynchronously on the current stream."""
    rc = lib().fd_copy_h2d_async(dst.data_ptr(), src_pinned.data_ptr(), n_elements * dst.element_size(), _stream())
    if rc != 0:
        raise KernelError(lib().fd_last_error().decode())


def copy_d2h_sync(dst_pinned: torch.Tensor, src: torch.Tensor, n_elements: int) -> None:
    """dst[:n] <- src[:n] into pinned host memory on the current stream, waited for."""
    rc = lib().fd_copy_d2h_sync(dst_pinned.data_ptr(), src.data_ptr(), n_elements * src.element_size(), _stream())
    if rc != 0:
        raise KernelError(lib().fd_last_error().decode())


def sm_count() -> int:
    return lib().fd_sm_count()


def status_message(word: int) -> str:
    return "; ".join(text for bit, text in _STATUS_TEXT.items() if word & bit) or "ok"


# ---------------------------------------------------------------------------

def embed(tokens: torch.Tensor, table: torch.Tensor, resid: torch.Tensor, status: torch.Tensor) -> None:
    """resid[t] = float(table[tokens[t]]); tokens int32 [T], resid float32 [T, H]."""
    T = tokens.numel()
    V, H = table.shape
    assert tokens.dtype == torch.int32 and resid.dtype == torch.float32 and resid.shape[-1] == H
    _check(lib().fd_embed(_ptr(tokens), _ptr(table), _dt(table.dtype), _ptr(resid), T, H, V,
                          _ptr(status), _stream()))


def add_rmsnorm(delta: Optional[torch.Tensor], resid: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, n_out: Optional[int] = None,
                write_resid: bool = True, n_parts: int = 1) -> None:
    """out[j] = rmsnorm(resid[r] + delta[r]) * weight with r = rows[j] (or j);
    resid[r] takes the sum when ``write_resid``.  ``delta`` None: plain norm.
    ``delta`` [parts, rows, H] (or ``n_parts`` > 1) holds partial sums, added in order."""
    H = resid.shape[-1]
    if delta is not None and delta.dim() == 3:
        n_parts = delta.shape[0]
    if n_out is None:
        n_out = rows.numel() if rows is not None else resid.numel() // H
    assert resid.dtype == torch.float32 and out.shape[-1] == H and weight.numel() == H
    part_stride = 0
    if delta is not None and n_parts > 1:
        part_stride = delta.numel() // n_parts
    _check(lib().fd_add_rmsnorm(_ptr(delta), _dt(delta.dtype) if delta is not None else _dt(out.dtype),
                                n_parts, part_stride, _ptr(resid), int(write_resid), _ptr(weight),
                                _dt(weight.dtype), float(eps), _ptr(out), _dt(out.dtype), _ptr(rows),
                                n_out, H, _stream()))


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, tiled: bool = False) -> None:
    """out[m, i] = silu(gate_i) * up_i.  ``gate_up`` [M, 2I] is [gate | up], or
    with ``tiled`` tiles of 16 columns: 8 gate values then the 8 up values."""
    M, I2 = gate_up.shape
    assert out.shape == (M, I2 // 2) and out.dtype == gate_up.dtype
    _check(lib().fd_silu_mul(_ptr(gate_up), _ptr(out), _dt(out.dtype), M, I2 // 2, int(tiled), _stream()))


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                tok_row: torch.Tensor, tok_pos: torch.Tensor, row_slot: torch.Tensor,
                k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor,
                bias: Optional[torch.Tensor] = None, paired: bool = False) -> None:
    """Rotate q and k of every token at its position; append k and v to the
    paged pools [num_blocks, n_kv, block_size, d] (unless ``write_kv`` is off).
    ``qkv`` is [T, (n_q + 2 n_kv) d], or [parts, T, ...] float32 partial sums of
    a split-K product that are added up here, with ``bias`` added on top.
    ``paired``: the columns of each q and k head come in tiles of 8 dims + their
    8 rotation partners (the order ``gemv_qkv_rope`` wants the rows of W in)."""
    n_parts = qkv.shape[0] if qkv.dim() == 3 else 1
    T = qkv.shape[-2]
    assert qkv.shape[-1] == (n_q + 2 * n_kv) * head_dim and q_out.shape == (T, n_q * head_dim)
    assert cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2
    assert k_pool.dtype == q_out.dtype and (n_parts == 1 or qkv.dtype == torch.float32)
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_rope_append(_ptr(qkv), _dt(qkv.dtype), n_parts, qkv.numel() // n_parts, _ptr(bias),
                                _dt(bias.dtype) if bias is not None else 0, _ptr(q_out), _dt(q_out.dtype),
                                _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row), _ptr(tok_pos), _ptr(row_slot),
                                _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], num_blocks,
                                block_size, T, n_q, n_kv, head_dim, int(write_kv), int(paired), _ptr(status),
                                _stream()))


def gemv_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, tok_row: torch.Tensor, tok_pos: torch.Tensor,
                  row_slot: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                  n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor, n_splits: int = 1,
                  prefetch: Optional[torch.Tensor] = None) -> None:
    """The q/k/v projection of a decode step (M <= 64 rows, bfloat16) with bias,
    rotary encoding and the append to the paged cache in its epilogue.  ``w``
    and ``bias`` are in the paired row order (see ``rope_append``).  ``prefetch``: a
    tensor that a later kernel streams (the output projection's weights); the kernel
    asks L2 for it once its own loads are through."""
    M, K = x.shape
    assert w.shape == ((n_q + 2 * n_kv) * head_dim, K) and q_out.shape == (M, n_q * head_dim)
    assert x.dtype == w.dtype == q_out.dtype == k_pool.dtype == torch.bfloat16
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_gemv_qkv_rope(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                  _ptr(q_out), M, K, n_splits, _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row),
                                  _ptr(tok_pos), _ptr(row_slot), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                  block_table.shape[1], num_blocks, block_size, n_q, n_kv, head_dim, int(write_kv),
                                  _ptr(status), *_prefetch_args(prefetch, 1 << 62), _stream()))


GEMV_PARTIAL, GEMV_BF16, GEMV_F32, GEMV_GATED = 0, 1, 2, 3


def gemm_tc_set_wide(on) -> None:
    """Which tiling ``gemm_tc`` and ``gemm_tc_qkv_rope`` use from now on where N >= 256: 2 = two SMs per
    256 x 256 tile (``tcgen05.mma.cta_group::2``), 1 / True = one persistent CTA per SM with 128 x 256
    tiles, or with 128 x 128 tiles where those number no more than the SMs, 3 = 128 x 256 tiles
    always, 0 / False = 128 x 128 tiles, one per CTA, everywhere.  For tests and measurements."""
    lib().fd_gemm_tc_set_wide(int(on))


def attn_prefill_set_form(form: int) -> None:
    """Which form the tcgen05 prompt attention takes from now on: 1 = a CTA takes 256 queries as two query
    tiles that share every key tile; 2 = a CTA takes 128 queries and deals their key tiles to its two groups
    of softmax warps, which add up their results at the end (half the chain of key tiles per query tile:
    for prompts too short to fill the GPU); 0 = the launcher chooses by the number of CTAs.  For tests and
    measurements."""
    lib().fd_attn_prefill_set_form(int(form))


def attn_decode_set_form(form: int) -> None:
    """Which form the tensor-core decode attention takes from now on: 0 = the launcher chooses (keys as
    the rows of the MMAs for groups of up to 8 query heads, CTAs of eight warps where all of them fit the
    GPU at one per SM); bit 0: the heads as rows always; bit 1: four warps always; bit 2: eight warps
    always.  For tests and measurements."""
    lib().fd_attn_decode_set_form(int(form))


def gemm_tc_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                     cos: torch.Tensor, sin: torch.Tensor, tok_row: torch.Tensor, tok_pos: torch.Tensor,
                     row_slot: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                     n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor) -> None:
    """The q/k/v projection of a prompt step on the tcgen05 tensor cores with
    bias, rotary encoding and the append to the paged cache in its epilogue.
    ``w`` and ``bias`` in the paired row order (see ``rope_append``)."""
    M, K = x.shape
    assert w.shape == ((n_q + 2 * n_kv) * head_dim, K) and q_out.shape == (M, n_q * head_dim)
    assert x.dtype == w.dtype == q_out.dtype == k_pool.dtype == torch.bfloat16
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_gemm_tc_qkv_rope(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                     _ptr(q_out), M, K, _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row),
                                     _ptr(tok_pos), _ptr(row_slot), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                     block_table.shape[1], num_blocks, block_size, n_q, n_kv, head_dim,
                                     int(write_kv), _ptr(status), _stream()))


def gemm_tc_supported(M: int, N: int, K: int) -> bool:
    return bool(lib().fd_gemm_tc_supported(M, N, K))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, gated: bool = False,
            status: Optional[torch.Tensor] = None) -> None:
    """out = x w^T (+ bias) on the tcgen05 tensor cores (TMA-fed, accumulator in
    tensor memory); bfloat16 operands, ``out`` bfloat16 or float32 [M, N], or
    with ``gated`` (w rows in tiles of 8 gate + 8 up) bfloat16 [M, N / 2] =
    silu(gate) * up.  Any M and N; K a multiple of 8."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2) and bias is None
        mode = GEMV_GATED
    else:
        assert out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32)
        mode = GEMV_BF16 if out.dtype == torch.bfloat16 else GEMV_F32
    _check(lib().fd_gemm_tc(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                            _ptr(out), mode, M, N, K, _ptr(status), _stream()))


def gemm_stream_splits(M: int, N: int, K: int) -> int:
    """CTAs per cluster (splits of K) the streaming tcgen05 product would use; 0 if it does not take
    the sizes (more than 128 rows of x, K not a multiple of 8)."""
    return int(lib().fd_gemm_stream_splits(M, N, K))


def gemm_stream(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, gated: bool = False,
                splits: int = 0, status: Optional[torch.Tensor] = None) -> None:
    """Weight-streaming product for up to 128 rows of x on the tcgen05 tensor cores (W tiles as the
    M side, the rows of x as the N side, K split over a thread-block cluster for narrow W):
    out = x w^T (+ bias), bfloat16 or float32 [M, N], or with ``gated`` (w rows in tiles of 8 gate +
    8 up) bfloat16 [M, N / 2] = silu(gate) * up.  ``splits`` 0: chosen by the launcher."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K
    if gated:
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2) and bias is None
        mode = GEMV_GATED
    else:
        assert out.shape == (M, N) and out.dtype in (torch.bfloat16, torch.float32)
        mode = GEMV_BF16 if out.dtype == torch.bfloat16 else GEMV_F32
    _check(lib().fd_gemm_stream(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                _ptr(out), mode, M, N, K, splits, _ptr(status), _stream()))


def gemm_stream_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                         cos: torch.Tensor, sin: torch.Tensor, tok_row: torch.Tensor, tok_pos: torch.Tensor,
                         row_slot: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                         n_q: int, n_kv: int, head_dim: int, write_kv: bool, status: torch.Tensor,
                         splits: int = 0) -> None:
    """The q/k/v projection of a step of up to 128 tokens on the streaming tcgen05 product, with bias,
    rotary encoding and the append to the paged cache in its epilogue.  ``w`` and ``bias`` in the
    paired row order (see ``rope_append``)."""
    M, K = x.shape
    assert w.shape == ((n_q + 2 * n_kv) * head_dim, K) and q_out.shape == (M, n_q * head_dim)
    assert x.dtype == w.dtype == q_out.dtype == k_pool.dtype == torch.bfloat16
    num_blocks, _, block_size, _ = k_pool.shape
    _check(lib().fd_gemm_stream_qkv_rope(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                                         _ptr(q_out), M, K, splits, _ptr(cos), _ptr(sin), cos.shape[0], _ptr(tok_row),
                                         _ptr(tok_pos), _ptr(row_slot), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                         block_table.shape[1], num_blocks, block_size, n_q, n_kv, head_dim,
                                         int(write_kv), _ptr(status), _stream()))


def gemm_stream_set_pdl(on: bool) -> None:
    """Whether the streaming product is launched with the programmatic-dependent-launch attribute (the
    default): it may then start and fetch its first weights while the kernel before it in the stream
    still runs, and waits for that kernel before it reads x or writes anything."""
    lib().fd_gemm_stream_set_pdl(int(on))


def gemm_stream_force_2d(on: bool) -> None:
    """Tests: make the streaming product read its operands through two-dimensional tensor maps (one copy per
    k-block) even where K is a multiple of 64 and one three-dimensional copy per stage would do."""
    lib().fd_gemm_stream_force_2d(int(on))


def gemm_stream_last_map3d() -> bool:
    """Whether the last streaming product read its operands through three-dimensional tensor maps."""
    return bool(lib().fd_gemm_stream_last_map3d())


def tc_test_hook(wait_ns: int = 0, skip_last: bool = False) -> None:
    """Tests only.  The limit of every bounded wait of the TMA + tcgen05 kernels (0: the default of
    0.2 s) and whether their producers leave out their very last copy, so that a wait runs out and the
    kernel reports ``STATUS_WAIT_TIMEOUT`` and returns."""
    lib().fd_tc_test_hook(int(wait_ns), int(skip_last))


def gemv_splits(M: int, N: int, K: int, target_ctas: int, allow_split: bool = True) -> int:
    """Splits of K the decode matrix product would use; 0 if it does not take the sizes."""
    return int(lib().fd_gemv_splits(M, N, K, target_ctas, int(allow_split)))


def _prefetch_args(t: Optional[torch.Tensor], limit: int):
    """(pointer, bytes) of the leading ``limit`` bytes of a tensor that a kernel is to ask L2 for.  It is a hint:
    a tensor the kernels cannot take it from (not on the device, not contiguous, not 16-byte aligned) is passed over."""
    if t is None or limit <= 0 or not t.is_cuda or not t.is_contiguous() or t.data_ptr() % 16 != 0:
        return None, 0
    return t.data_ptr(), min(int(limit), t.numel() * t.element_size()) & ~15


def gemv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, mode: int,
         n_splits: int = 1, prefetch: Optional[torch.Tensor] = None, prefetch_bytes: int = 1 << 62) -> None:
    """Weight-streaming product for M <= 64 rows (bfloat16): out = x w^T.
    mode GEMV_PARTIAL: out float32 [n_splits, M, N]; GEMV_BF16 / GEMV_F32: out
    [M, N] (+ bias), with ``n_splits`` <= 8 splits of K added inside a
    thread-block cluster; GEMV_GATED: w rows in tiles of 8 gate + 8 up, out
    bfloat16 [M, N / 2] = silu(gate) * up.  ``prefetch``: a tensor that a later kernel
    streams; the kernel asks L2 for its first ``prefetch_bytes`` once its own loads are through."""
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    want = {GEMV_PARTIAL: (torch.float32, n_splits * M * N), GEMV_BF16: (torch.bfloat16, M * N),
            GEMV_F32: (torch.float32, M * N), GEMV_GATED: (torch.bfloat16, M * N // 2)}[mode]
    assert out.dtype == want[0] and out.numel() == want[1], (out.dtype, out.shape, mode)
    _check(lib().fd_gemv(_ptr(x), _ptr(w), _ptr(bias), int(bias is not None and bias.dtype == torch.float32),
                         _ptr(out), mode, M, N, K, n_splits, *_prefetch_args(prefetch, prefetch_bytes), _stream()))


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] w[N, K]^T + bias on the CUDA cores (fixed k order)."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N) and w.dtype == x.dtype
    _check(lib().fd_gemm_simt(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _dt(x.dtype),
                              _dt(bias.dtype) if bias is not None else 0, _dt(out.dtype), M, N, K, _stream()))


def attention_scratch_floats(n_tokens: int, n_q: int, head_dim: int, n_splits: int) -> int:
    return int(lib().fd_attn_scratch_floats(n_tokens, n_q, head_dim, n_splits))


_attn_counters = {}      # per device: zeroed ints the decode kernel counts arriving splits in (kept alive for good)


def _counters(device, n: int) -> torch.Tensor:
    bufs = _attn_counters.setdefault(device, [])
    if not bufs or bufs[-1].numel() < n:
        bufs.append(torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device))
    return bufs[-1]


def _attention(fn_name, q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start, row_q_len,
               row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits, split_len,
               scratch, status, prefetch=None, prefetch_bytes=0) -> None:
    T = q.shape[0]
    num_blocks, _, block_size, _ = k_pool.shape
    assert q.dtype == k_pool.dtype == out.dtype
    if n_splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= attention_scratch_floats(T, n_q, head_dim, n_splits)
    args = [_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _dt(q.dtype), _ptr(block_table), block_table.shape[1],
            num_blocks, block_size, _ptr(tok_row), _ptr(row_slot), _ptr(row_q_start), _ptr(row_q_len),
            _ptr(row_ctx_len), n_rows, T, max_q_len, n_q, n_kv, head_dim, float(scale), int(window), n_splits,
            split_len, _ptr(scratch)]
    if fn_name != "fd_attention_simt":
        fused = n_splits > 1 and max_q_len == 1 and q.dtype == torch.bfloat16
        args.append(_ptr(_counters(q.device, n_rows * n_kv)) if fused else None)
    args.append(_ptr(status))
    if fn_name == "fd_attention":
        args += list(_prefetch_args(prefetch, prefetch_bytes))
    args.append(_stream())
    _check(getattr(lib(), fn_name)(*args))


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
              block_table: torch.Tensor, tok_row: torch.Tensor, row_slot: torch.Tensor,
              row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx_len: torch.Tensor,
              n_rows: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
              window: int = 0, n_splits: int = 1, split_len: int = 0,
              scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
              prefetch: Optional[torch.Tensor] = None, prefetch_bytes: int = 0) -> None:
    """Causal GQA attention of the step's tokens over the paged cache, by the
    fastest kernel that takes the sizes (tensor cores for bfloat16 decode steps
    with head size 64 or 128; the CUDA-core kernel otherwise).  ``prefetch``: a
    tensor that a later kernel streams; the tensor-core decode kernel asks L2 for its
    first ``prefetch_bytes`` when its own reads are through (the other kernels do not)."""
    _attention("fd_attention", q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start, row_q_len,
               row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits, split_len,
               scratch, status, prefetch, prefetch_bytes)


def attention_mma_sync(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                       block_table: torch.Tensor, tok_row: torch.Tensor, row_slot: torch.Tensor,
                       row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx_len: torch.Tensor,
                       n_rows: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                       window: int = 0, n_splits: int = 1, split_len: int = 0,
                       scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """The same with prompts on the mma.sync kernel even at head size 128, where
    ``attention`` takes the tcgen05 kernel."""
    _attention("fd_attention_mma_sync", q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start,
               row_q_len, row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits,
               split_len, scratch, status)


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, out: torch.Tensor,
                   block_table: torch.Tensor, tok_row: torch.Tensor, row_slot: torch.Tensor,
                   row_q_start: torch.Tensor, row_q_len: torch.Tensor, row_ctx_len: torch.Tensor,
                   n_rows: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                   window: int = 0, n_splits: int = 1, split_len: int = 0,
                   scratch: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """The same on the CUDA cores for every size (the true 32-bit path)."""
    _attention("fd_attention_simt", q, k_pool, v_pool, out, block_table, tok_row, row_slot, row_q_start,
               row_q_len, row_ctx_len, n_rows, max_q_len, n_q, n_kv, head_dim, scale, window, n_splits,
               split_len, scratch, status)


_sample_scratch = {}


def sample_scratch_words(n: int, V: int) -> int:
    return int(lib().fd_sample_scratch_words(n, V))


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           request: Optional[torch.Tensor] = None, step: Optional[torch.Tensor] = None, seed: int = 0,
           scratch: Optional[torch.Tensor] = None, seed_tensor: Optional[torch.Tensor] = None) -> None:
    """out[i] = argmax (greedy) or a Gumbel-max draw from softmax(logits[i] / T_i).
    ``scratch``: int32 tensor of ``sample_scratch_words(n, V)`` entries for large
    vocabularies; when omitted a per-device buffer is kept and reused.  ``seed_tensor``:
    a one-element int64 tensor on the device that holds the seed (its 64 bits) instead of
    ``seed``, so that a captured graph serves any seed."""
    n, V = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32
    if temperature is not None:
        assert temperature.dtype == torch.float32 and request.dtype == torch.int64 and step.dtype == torch.int32
    words = sample_scratch_words(n, V)
    if words and scratch is None:
        key = logits.device
        scratch = _sample_scratch.get(key)
        if scratch is None or scratch.numel() < words:
            scratch = torch.empty(max(words, 4096), dtype=torch.int32, device=logits.device)
            _sample_scratch[key] = scratch
    if words:
        assert scratch.dtype == torch.int32 and scratch.numel() >= words
    assert seed_tensor is None or (seed_tensor.dtype == torch.int64 and seed_tensor.numel() == 1)
    _check(lib().fd_sample(_ptr(logits), n, V, _ptr(temperature), _ptr(request), _ptr(step),
                           seed & 0xFFFFFFFFFFFFFFFF, _ptr(seed_tensor), _ptr(out), _ptr(scratch) if words else None,
                           _stream()))
