"""Each CUDA kernel alone against a plain PyTorch float32/float64 reference of
the same operation, at sizes other than the engine's tiny models: head sizes
in steps of 16, groups that are no power of two, widths and vocabularies that
are no multiple of anything useful."""

import math

import pytest
import torch

from flashdecode_cuda_b200 import kernels as K
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 1.2e-2}


def rel(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return float((got - want).abs().max()) / max(float(want.abs().max()), 1e-9)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("V,H,T", [(100, 48, 7), (333, 1536, 33), (50, 5, 3)])
def test_embed(dtype, V, H, T):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(V, H, generator=g).to(DT[dtype]).to(DEV)
    tokens = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).to(DEV)
    resid = torch.full((T, H), 7.0, device=DEV)
    st = status()
    K.embed(tokens, table, resid, st)
    assert torch.equal(resid, table[tokens.long()].float())
    assert int(st.item()) == 0
    # an id outside the table is skipped and reported, not read
    bad = tokens.clone()
    bad[T // 2] = V + 5
    K.embed(bad, table, resid, st)
    assert int(st.item()) == K.STATUS_BAD_TOKEN
    assert float(resid[T // 2].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,H", [(5, 80), (3, 1537), (64, 4096), (2, 9)])
def test_add_rmsnorm(dtype, rows, H):
    g = torch.Generator().manual_seed(1)
    dt = DT[dtype]
    delta = torch.randn(rows, H, generator=g).to(dt).to(DEV)
    resid = torch.randn(rows, H, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(dt).to(DEV)
    eps = 3e-6
    out = torch.empty(rows, H, dtype=dt, device=DEV)
    r2 = resid.clone()
    K.add_rmsnorm(delta, r2, w, eps, out)
    x = resid.double() + delta.double()
    assert rel(r2, x) < 1e-6
    want = P.rmsnorm(x, w.double(), eps)
    assert rel(out, want) < (1e-5 if dtype == "float32" else 6e-3)
    # plain norm (no delta), only chosen rows, residual untouched
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=dt, device=DEV)
    r3 = resid.clone()
    K.add_rmsnorm(None, r3, w, eps, out2, rows=idx)
    assert torch.equal(r3, resid)
    assert rel(out2, P.rmsnorm(resid.double()[idx.long()], w.double(), eps)) < (1e-5 if dtype == "float32" else 6e-3)
    # chosen rows with a delta that is not written back
    K.add_rmsnorm(delta, r3, w, eps, out2, rows=idx, write_resid=False)
    assert torch.equal(r3, resid)
    assert rel(out2, want[idx.long()]) < (1e-5 if dtype == "float32" else 6e-3)
    # a 32-bit weight vector with 16-bit activations
    if dtype == "bfloat16":
        K.add_rmsnorm(delta, resid.clone(), w.float(), eps, out)
        assert rel(out, want) < 6e-3


def test_add_rmsnorm_partial_sums():
    g = torch.Generator().manual_seed(2)
    parts = torch.randn(3, 6, 200, generator=g).to(DEV)
    resid = torch.randn(6, 200, generator=g).to(DEV)
    w = torch.ones(200, device=DEV)
    out = torch.empty(6, 200, device=DEV)
    r = resid.clone()
    K.add_rmsnorm(parts, r, w, 1e-6, out, n_parts=3, n_out=6)
    x = resid.double() + parts.double().sum(0)
    assert rel(r, x) < 1e-6
    assert rel(out, P.rmsnorm(x, w.double(), 1e-6)) < 1e-5


@pytest.mark.parametrize("n_parts,rows,H", [(1, 8, 1536), (2, 3, 200), (4, 16, 8192), (5, 2, 1536), (3, 4, 1537), (4, 5, 8200),
                                            (8, 8, 3584), (7, 3, 4096), (6, 4, 5120), (8, 2, 8192)])
def test_add_rmsnorm_partial_sums_to_bfloat16(n_parts, rows, H):
    """Float partial sums of a split product, bfloat16 output: the row kernel for up to four parts
    and widths that are multiples of 8 up to 8192, the general kernel otherwise; only chosen rows too."""
    g = torch.Generator().manual_seed(4)
    parts = torch.randn(n_parts, rows, H, generator=g).to(DEV)
    resid = torch.randn(rows, H, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16().to(DEV)
    out = torch.empty(rows, H, dtype=torch.bfloat16, device=DEV)
    r = resid.clone()
    K.add_rmsnorm(parts, r, w, 1e-6, out)
    x = resid.double() + parts.double().sum(0)
    assert rel(r, x) < 1e-6
    want = P.rmsnorm(x, w.double(), 1e-6)
    assert rel(out, want) < 6e-3
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=torch.bfloat16, device=DEV)
    r2 = resid.clone()
    K.add_rmsnorm(parts, r2, w.float(), 1e-6, out2, rows=idx, write_resid=False)
    assert torch.equal(r2, resid)
    assert rel(out2, want[idx.long()]) < 6e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,I", [(3, 176), (65, 8960), (1, 7)])
def test_silu_mul(dtype, M, I):
    g = torch.Generator().manual_seed(3)
    gu = (2 * torch.randn(M, 2 * I, generator=g)).to(DT[dtype]).to(DEV)
    out = torch.empty(M, I, dtype=DT[dtype], device=DEV)
    K.silu_mul(gu, out)
    want = P.swiglu(gu[:, :I].double(), gu[:, I:].double())
    assert rel(out, want) < (1e-6 if dtype == "float32" else 5e-3)
    if I % 8 == 0:                              # tiles of 8 gate + 8 up columns
        tiled = torch.stack([gu[:, :I].reshape(M, I // 8, 8), gu[:, I:].reshape(M, I // 8, 8)], dim=2).reshape(M, 2 * I)
        K.silu_mul(tiled.contiguous(), out, tiled=True)
        assert rel(out, want) < (1e-6 if dtype == "float32" else 5e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K_", [(1, 7, 5), (33, 100, 48), (70, 333, 1537), (8, 2048, 1536), (130, 64, 66)])
@pytest.mark.parametrize("bias", [False, True])
def test_gemm_simt(dtype, M, N, K_, bias):
    g = torch.Generator().manual_seed(4)
    dt = DT[dtype]
    x = torch.randn(M, K_, generator=g).to(dt).to(DEV)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(dt).to(DEV)
    b = torch.randn(N, generator=g).to(dt).to(DEV) if bias else None
    out = torch.empty(M, N, dtype=dt, device=DEV)
    K.gemm_simt(x, w, b, out)
    want = P.linear(x.double(), w.double(), b.double() if bias else None)
    assert rel(out, want) < (2e-6 if dtype == "float32" else 5e-3)
    if dtype == "bfloat16":                      # float32 output from 16-bit operands (logits)
        out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
        K.gemm_simt(x, w, b, out32)
        assert rel(out32, want) < 2e-6


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K_", [(16, 32), (100, 96), (333, 1536), (2048, 224), (1536, 8960)])
def test_gemv_decode_product(M, N, K_):
    """The weight-streaming product of decode steps: every output form, rows of
    W and of x that fill no tile, K cut into partial sums."""
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    want = P.linear(x.double(), w.double())
    assert K.gemv_splits(M, N, K_, 1, allow_split=False) in (0, 1)
    if K.gemv_splits(M, N, K_, 1, allow_split=False) == 1:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        K.gemv(x, w, b, out, K.GEMV_BF16)
        assert rel(out, want + b.double()) < 5e-3
        out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
        K.gemv(x, w, None, out32, K.GEMV_F32)
        assert rel(out32, want) < 2e-5
        K.gemv(x, w, b.float(), out32, K.GEMV_F32)            # a bias kept in 32-bit
        assert rel(out32, want + b.double()) < 2e-5
    for target in (1, 64, 296):
        splits = K.gemv_splits(M, N, K_, target)
        assert 1 <= splits <= K_ // 32
        parts = torch.full((splits, M, N), float("nan"), device=DEV)
        K.gemv(x, w, None, parts, K.GEMV_PARTIAL, splits)
        assert rel(parts.double().sum(0), want) < 2e-5
        # the same splits added inside a thread-block cluster: the finished product comes out
        assert splits <= 8
        out32 = torch.full((M, N), float("nan"), device=DEV)
        K.gemv(x, w, b, out32, K.GEMV_F32, splits)
        assert rel(out32, want + b.double()) < 2e-5
        out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        K.gemv(x, w, None, out16, K.GEMV_BF16, splits)
        assert rel(out16, want) < 5e-3
    if N % 16 == 0 and K.gemv_splits(M, N, K_, 1, allow_split=False) == 1:
        # gated form: rows in tiles of 8 gate + 8 up
        I = N // 2
        gate, up = w[:I], w[I:]
        tiled = torch.stack([gate.view(I // 8, 8, K_), up.view(I // 8, 8, K_)], dim=1).reshape(N, K_).contiguous()
        act = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        K.gemv(x, tiled, None, act, K.GEMV_GATED)
        assert rel(act, P.swiglu(P.linear(x.double(), gate.double()), P.linear(x.double(), up.double()))) < 6e-3


def test_gemv_refuses_what_it_cannot_do():
    assert K.gemv_splits(65, 128, 64, 1) == 0 and K.gemv_splits(4, 128, 80, 1) == 0
    x = torch.zeros(4, 80, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(K.KernelError, match="multiple of 32"):
        K.gemv(x, torch.zeros(16, 80, dtype=torch.bfloat16, device=DEV), None,
               torch.zeros(4, 16, dtype=torch.bfloat16, device=DEV), K.GEMV_BF16)


@pytest.fixture(params=[False, True], ids=["3d", "2d"])
def stream_maps(request):
    """The streaming product's copies: one three-dimensional copy per operand and stage where K is a
    multiple of 64 (the default), or one two-dimensional copy per k-block."""
    K.gemm_stream_force_2d(request.param)
    yield request.param
    K.gemm_stream_force_2d(False)


@pytest.mark.parametrize("M", [1, 8, 17, 24, 33, 48, 64, 100, 128])
@pytest.mark.parametrize("N,K_", [(16, 8), (100, 96), (333, 1536), (2048, 1536), (1536, 8960), (4880, 200), (129, 72),
                                  (300, 320), (40000, 128)])
def test_gemm_stream_decode_product(M, N, K_, stream_maps):
    """The streaming tcgen05 product of decode steps (W tiles as the M side of the MMAs, the rows of x
    as the N side): every output form, rows of W, rows of x and K that fill no tile, K split over
    clusters of 2, 4 and 8 CTAs and unsplit with several tiles per persistent CTA."""
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    want = P.linear(x.double(), w.double())
    assert K.gemm_stream_splits(M, N, K_) in (1, 2, 4, 8)
    st = status()
    for splits in (0, 1, 2, 4, 8):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.gemm_stream(x, w, b, out, splits=splits, status=st)
        assert K.gemm_stream_last_map3d() == (K_ % 64 == 0 and not stream_maps)
        assert rel(out, want + b.double()) < 5e-3, splits
        out32 = torch.full((M, N), float("nan"), device=DEV)
        K.gemm_stream(x, w, None, out32, splits=splits, status=st)
        assert rel(out32, want) < 2e-5, splits
        K.gemm_stream(x, w, b.float(), out32, splits=splits, status=st)            # a bias kept in 32-bit
        assert rel(out32, want + b.double()) < 2e-5, splits
        if N % 16 == 0:
            I = N // 2
            gate, up = w[:I], w[I:]
            tiled = torch.stack([gate.view(I // 8, 8, K_), up.view(I // 8, 8, K_)], dim=1).reshape(N, K_).contiguous()
            act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
            K.gemm_stream(x, tiled, None, act, gated=True, splits=splits, status=st)
            assert rel(act, P.swiglu(P.linear(x.double(), gate.double()), P.linear(x.double(), up.double()))) < 6e-3, splits
    assert int(st.item()) == 0


def test_gemm_stream_sums_do_not_depend_on_the_batch():
    """A row of x gives the same bits alone and among 63 others (the split of K and the order in
    which the cluster adds its partial sums depend on the matrix only)."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(64, 1536, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2048, 1536, generator=g) / 40).to(torch.bfloat16).to(DEV)
    big = torch.empty(64, 2048, device=DEV)
    one = torch.empty(1, 2048, device=DEV)
    K.gemm_stream(x, w, None, big, status=status())
    K.gemm_stream(x[37:38].contiguous(), w, None, one, status=status())
    assert torch.equal(big[37:38], one)


def test_gemm_stream_refuses_what_it_cannot_do():
    assert K.gemm_stream_splits(129, 128, 64) == 0 and K.gemm_stream_splits(4, 128, 12) == 0
    x = torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(K.KernelError, match="multiple of 8"):
        K.gemm_stream(x, torch.zeros(16, 12, dtype=torch.bfloat16, device=DEV), None,
                      torch.zeros(4, 16, dtype=torch.bfloat16, device=DEV))


TC_DEFAULT_TILING = 1


@pytest.fixture(params=[2, 3, 1, 0], ids=["pair", "wide", "auto", "square"])
def tc_tiling(request):
    """The tilings of the tcgen05 product: two SMs per 256 x 256 tile, persistent CTAs with 128 x 256 tiles, the
    default (persistent CTAs with 128 x 128 tiles where those number no more than the SMs: most shapes of these
    tests), and 128 x 128 tiles with one CTA each."""
    K.gemm_tc_set_wide(request.param)
    yield request.param
    K.gemm_tc_set_wide(TC_DEFAULT_TILING)


@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (128, 256, 256), (130, 200, 72), (70, 333, 1536), (2048, 2048, 1536),
                                    (300, 1536, 8960), (17, 16, 8), (1000, 384, 136), (4096, 4864, 256), (129, 257, 64)])
def test_gemm_tcgen05(M, N, K_, tc_tiling):
    """The TMA + tcgen05 product of prompt steps: full tiles, ragged edges in M, N
    and K (zero-filled by TMA), more tiles than SMs (the persistent kernel walks several,
    alternating its two accumulators), bias in either dtype, float output."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16).to(DEV)
    b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
    want = P.linear(x.double(), w.double())
    assert K.gemm_tc_supported(M, N, K_)
    st = status()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.gemm_tc(x, w, None, out, status=st)
    assert rel(out, want) < 5e-3
    K.gemm_tc(x, w, b, out, status=st)
    assert rel(out, want + b.double()) < 5e-3
    out32 = torch.full((M, N), float("nan"), device=DEV)
    K.gemm_tc(x, w, b.float(), out32, status=st)
    assert rel(out32, want + b.double()) < 2e-5
    assert int(st.item()) == 0
    if N % 16 == 0:
        I = N // 2
        gate, up = w[:I], w[I:]
        tiled = torch.stack([gate.view(I // 8, 8, K_), up.view(I // 8, 8, K_)], dim=1).reshape(N, K_).contiguous()
        act = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.gemm_tc(x, tiled, None, act, gated=True, status=st)
        assert rel(act, P.swiglu(P.linear(x.double(), gate.double()), P.linear(x.double(), up.double()))) < 6e-3


@pytest.mark.parametrize("N,K_", [(77, 300), (200, 1537), (10000, 520)])
def test_gemm_simt_rows_do_not_depend_on_the_batch(N, K_):
    """The same row gives the same bits alone, among 8 and among 100 others: the kernels for up to 16 rows (a
    narrow and a wide form) and the one for more keep the same chain of k for every output element."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(101, K_, generator=g).to(DEV)
    w = torch.randn(N, K_, generator=g).to(DEV)
    b = torch.randn(N, generator=g).to(DEV)
    big = torch.empty(101, N, device=DEV)
    some = torch.empty(9, N, device=DEV)
    one = torch.empty(1, N, device=DEV)
    K.gemm_simt(x, w, b, big)
    K.gemm_simt(x[64:73].contiguous(), w, b, some)
    K.gemm_simt(x[70:71].contiguous(), w, b, one)
    assert torch.equal(big[70:71], one) and torch.equal(some[6:7], one)
    assert rel(big, P.linear(x.double(), w.double(), b.double())) < 2e-5


# ---------------------------------------------------------------------------
# paged cache helpers for the rope and attention kernels
# ---------------------------------------------------------------------------

def scrambled_table(lens, block_size, n_slots, gen, spare=3):
    """Block table [n_slots, max_blocks] whose blocks are handed out in a
    random order, so a kernel that ignores the table cannot pass."""
    per = [-(-n // block_size) for n in lens]
    total = sum(per) + spare
    perm = torch.randperm(total, generator=gen).tolist()
    width = max(per) + 1
    table = torch.full((n_slots, width), -1, dtype=torch.int32)
    it = iter(perm)
    slots = torch.randperm(n_slots, generator=gen)[:len(lens)].tolist()
    for s, nb in zip(slots, per):
        for c in range(nb):
            table[s, c] = next(it)
    return table, slots, total


def fill_pools(k_seqs, v_seqs, table, slots, block_size, total_blocks, dtype, poison=None):
    """Pools [blocks, n_kv, block_size, d] holding the given per-sequence keys
    and values; untouched places hold ``poison`` (NaN by default: nothing may
    read beyond a sequence's length)."""
    n_kv, d = k_seqs[0].shape[1:]
    fill = float("nan") if poison is None else poison
    kp = torch.full((total_blocks, n_kv, block_size, d), fill, dtype=dtype)
    vp = torch.full_like(kp, fill)
    for ks, vs, s in zip(k_seqs, v_seqs, slots):
        for pos in range(ks.shape[0]):
            b = int(table[s, pos // block_size])
            kp[b, :, pos % block_size] = ks[pos].to(dtype)
            vp[b, :, pos % block_size] = vs[pos].to(dtype)
    return kp.to(DEV), vp.to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_q,n_kv,d,bs", [(6, 2, 48, 4), (5, 5, 16, 16), (12, 2, 128, 16), (7, 1, 80, 32)])
def test_rope_append(dtype, n_q, n_kv, d, bs):
    g = torch.Generator().manual_seed(6)
    dt = DT[dtype]
    ctx = [3, 0, 37]                 # cached before the step
    new = [5, 9, 1]                  # new tokens of each row
    lens = [c + n for c, n in zip(ctx, new)]
    table, slots, total = scrambled_table(lens, bs, 5, g)
    T = sum(new)
    qkv = torch.randn(T, (n_q + 2 * n_kv) * d, generator=g).to(dt)
    theta = 12345.0
    n_pos = 64
    inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    fr = torch.outer(torch.arange(n_pos).float(), inv)
    cos, sin = fr.cos().to(DEV), fr.sin().to(DEV)
    tok_row = torch.tensor([r for r, n in enumerate(new) for _ in range(n)], dtype=torch.int32)
    tok_pos = torch.tensor([c + i for c, n in zip(ctx, new) for i in range(n)], dtype=torch.int32)
    kp = torch.zeros(total, n_kv, bs, d, dtype=dt, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.empty(T, n_q * d, dtype=dt, device=DEV)
    st = status()
    K.rope_append(qkv.to(DEV), q_out, cos, sin, tok_row.to(DEV), tok_pos.to(DEV),
                  torch.tensor(slots, dtype=torch.int32, device=DEV), kp, vp, table.to(DEV),
                  n_q, n_kv, d, True, st)
    assert int(st.item()) == 0
    x = qkv.double().view(T, n_q + 2 * n_kv, d)
    c2, s2 = P.rope_tables(d, n_pos, theta)
    rot = P.apply_rope(x[:, :n_q + n_kv], c2[tok_pos.long()], s2[tok_pos.long()])
    tol = 1e-6 if dtype == "float32" else 5e-3
    assert rel(q_out.view(T, n_q, d), rot[:, :n_q]) < tol
    for t in range(T):
        s, pos = slots[int(tok_row[t])], int(tok_pos[t])
        b = int(table[s, pos // bs])
        assert rel(kp[b, :, pos % bs], rot[t, n_q:]) < tol
        assert torch.equal(vp[b, :, pos % bs].cpu(), qkv.view(T, n_q + 2 * n_kv, d)[t, n_q + n_kv:])
    # the projection given as float partial sums of a split product, bias still to add
    g2 = torch.Generator().manual_seed(60)
    bias = torch.randn((n_q + 2 * n_kv) * d, generator=g2).to(dt)
    parts = torch.randn(3, T, (n_q + 2 * n_kv) * d, generator=g2)
    kp2, vp2, q2 = torch.zeros_like(kp), torch.zeros_like(vp), torch.empty_like(q_out)
    K.rope_append(parts.to(DEV), q2, cos, sin, tok_row.to(DEV), tok_pos.to(DEV),
                  torch.tensor(slots, dtype=torch.int32, device=DEV), kp2, vp2, table.to(DEV),
                  n_q, n_kv, d, True, st, bias=bias.to(DEV))
    x2 = (parts.double().sum(0) + bias.double()).view(T, n_q + 2 * n_kv, d)
    rot2 = P.apply_rope(x2[:, :n_q + n_kv], c2[tok_pos.long()], s2[tok_pos.long()])
    assert rel(q2.view(T, n_q, d), rot2[:, :n_q]) < tol
    t_last = T - 1
    s_, pos_ = slots[int(tok_row[t_last])], int(tok_pos[t_last])
    b_ = int(table[s_, pos_ // bs])
    assert rel(kp2[b_, :, pos_ % bs], rot2[t_last, n_q:]) < tol
    assert rel(vp2[b_, :, pos_ % bs], x2[t_last, n_q + n_kv:]) < tol
    # nothing else in the pools was touched
    written = sum(new) * n_kv * d
    assert int((kp != 0).sum().item()) <= written
    # a padding row (slot -1) writes nothing and reports nothing
    kp.zero_()
    K.rope_append(qkv.to(DEV), q_out, cos, sin, tok_row.to(DEV), tok_pos.to(DEV),
                  torch.tensor([-1, -1, -1], dtype=torch.int32, device=DEV), kp, vp, table.to(DEV),
                  n_q, n_kv, d, True, st)
    assert int(st.item()) == 0 and float(kp.abs().max()) == 0.0


def paired_order(n_q, n_kv, d):
    """Rows of a packed q/k/v matrix as the decode projection kernel wants them: in each q and
    k head, dims 8t..8t+7 followed by d/2+8t..d/2+8t+7; v heads in natural order."""
    rows = []
    for h in range(n_q + n_kv):
        for t in range(d // 16):
            rows += [h * d + 8 * t + i for i in range(8)] + [h * d + d // 2 + 8 * t + i for i in range(8)]
    return torch.tensor(rows + list(range((n_q + n_kv) * d, (n_q + 2 * n_kv) * d)))


@pytest.mark.parametrize("n_q,n_kv,d,bs,Kd", [(12, 2, 128, 16, 1536), (6, 2, 48, 4, 96), (3, 1, 32, 16, 96),
                                              (7, 7, 16, 8, 64), (28, 4, 128, 32, 224)])
@pytest.mark.parametrize("M", [1, 5, 8, 16])
def test_projection_with_rotary_epilogue(n_q, n_kv, d, bs, Kd, M):
    """q/k/v product + bias + rotation + cache append in one kernel (and the
    separate rotary kernel on the same paired column order) against the plain
    functions applied to the natural-order weights."""
    g = torch.Generator().manual_seed(n_q * 100 + M)
    bf = torch.bfloat16
    N = (n_q + 2 * n_kv) * d
    x = torch.randn(M, Kd, generator=g).to(bf)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(bf)
    b = (0.5 * torch.randn(N, generator=g)).to(bf)
    ctx = [int(v) for v in torch.randint(0, 50, (M,), generator=g)]
    table, slots, total = scrambled_table([c + 1 for c in ctx], bs, M + 2, g)
    theta, n_pos = 9999.0, 64
    inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    fr = torch.outer(torch.arange(n_pos).float(), inv)
    cos, sin = fr.cos().to(DEV), fr.sin().to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tok_row, tok_pos, row_slot = i32(list(range(M))), i32(ctx), i32(slots)
    order = paired_order(n_q, n_kv, d)
    wp, bp = w[order].contiguous().to(DEV), b[order].contiguous().to(DEV)

    qkv = (P.linear(x.double(), w.double(), b.double())).view(M, n_q + 2 * n_kv, d)
    c2, s2 = P.rope_tables(d, n_pos, theta)
    rot = P.apply_rope(qkv[:, :n_q + n_kv], c2[torch.tensor(ctx)], s2[torch.tensor(ctx)])

    def check(q_out, kp, vp, tol):
        assert rel(q_out.view(M, n_q, d), rot[:, :n_q]) < tol
        for m in range(M):
            blk = int(table[slots[m], ctx[m] // bs])
            assert rel(kp[blk, :, ctx[m] % bs], rot[m, n_q:]) < tol
            assert rel(vp[blk, :, ctx[m] % bs], qkv[m, n_q + n_kv:]) < tol

    for splits in sorted({1, K.gemv_splits(M, N, Kd, 592)}):
        kp = torch.zeros(total, n_kv, bs, d, dtype=bf, device=DEV)
        vp = torch.zeros_like(kp)
        q_out = torch.zeros(M, n_q * d, dtype=bf, device=DEV)
        st = status()
        K.gemv_qkv_rope(x.to(DEV), wp, bp, q_out, cos, sin, tok_row, tok_pos, row_slot, kp, vp, table.to(DEV),
                        n_q, n_kv, d, True, st, splits)
        assert int(st.item()) == 0
        check(q_out, kp, vp, 6e-3)
        assert int((kp != 0).sum().item()) <= M * n_kv * d            # only this step's positions were written
        # asked to fetch some other memory into L2 on the way (whole, and a size that is no multiple of a line or of
        # the CTAs' shares): the same bits, and that memory untouched
        for n_other in (5000, 8 + 13 * 1024):
            other = torch.full((n_other,), 3.0, dtype=bf, device=DEV)
            q2, kp2, vp2 = torch.zeros_like(q_out), torch.zeros_like(kp), torch.zeros_like(vp)
            K.gemv_qkv_rope(x.to(DEV), wp, bp, q2, cos, sin, tok_row, tok_pos, row_slot, kp2, vp2, table.to(DEV),
                            n_q, n_kv, d, True, st, splits, prefetch=other)
            assert int(st.item()) == 0
            assert torch.equal(q2, q_out) and torch.equal(kp2, kp) and torch.equal(vp2, vp)
            assert bool((other == 3.0).all())
    # a hint the kernel cannot take (not 16-byte aligned) is passed over, not an error
    K.gemv_qkv_rope(x.to(DEV), wp, bp, q_out, cos, sin, tok_row, tok_pos, row_slot, kp, vp, table.to(DEV),
                    n_q, n_kv, d, True, st, 1, prefetch=torch.zeros(64, dtype=bf, device=DEV)[1:])
    assert int(st.item()) == 0
    # the same fusion in the tcgen05 kernel that prompt steps use
    kp = torch.zeros(total, n_kv, bs, d, dtype=bf, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.zeros(M, n_q * d, dtype=bf, device=DEV)
    st = status()
    K.gemm_tc_qkv_rope(x.to(DEV), wp, bp, q_out, cos, sin, tok_row, tok_pos, row_slot, kp, vp, table.to(DEV),
                       n_q, n_kv, d, True, st)
    assert int(st.item()) == 0
    check(q_out, kp, vp, 6e-3)
    assert int((kp != 0).sum().item()) <= M * n_kv * d
    # the separate kernel on a projection whose columns are in the paired order
    proj = (x.double() @ wp.double().cpu().T + bp.double().cpu()).to(bf).to(DEV)
    kp = torch.zeros(total, n_kv, bs, d, dtype=bf, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.zeros(M, n_q * d, dtype=bf, device=DEV)
    K.rope_append(proj, q_out, cos, sin, tok_row, tok_pos, row_slot, kp, vp, table.to(DEV), n_q, n_kv, d, True,
                  status(), paired=True)
    check(q_out, kp, vp, 1e-2)
    # a padding row writes nothing
    kp.zero_()
    K.gemv_qkv_rope(x.to(DEV), wp, bp, q_out, cos, sin, tok_row, tok_pos, i32([-1] * M), kp, vp, table.to(DEV),
                    n_q, n_kv, d, True, status(), 1)
    assert float(kp.abs().max()) == 0.0


@pytest.mark.parametrize("n_q,n_kv,d,bs,Kd", [(12, 2, 128, 16, 1536), (6, 2, 48, 4, 96), (3, 1, 32, 16, 96),
                                              (7, 7, 16, 8, 64), (28, 4, 128, 32, 224)])
@pytest.mark.parametrize("M", [3, 17, 33, 64, 100])
def test_stream_projection_with_rotary_epilogue(n_q, n_kv, d, bs, Kd, M):
    """q/k/v product + bias + rotation + cache append in the streaming tcgen05 kernel, unsplit and with K
    split over clusters, against the plain functions applied to the natural-order weights; some rows
    of the step are padding (slot -1) and must write nothing."""
    g = torch.Generator().manual_seed(n_q * 100 + M)
    bf = torch.bfloat16
    N = (n_q + 2 * n_kv) * d
    x = torch.randn(M, Kd, generator=g).to(bf)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(bf)
    b = (0.5 * torch.randn(N, generator=g)).to(bf)
    ctx = [int(v) for v in torch.randint(0, 50, (M,), generator=g)]
    table, slots, total = scrambled_table([c + 1 for c in ctx], bs, M + 2, g)
    padding = [m for m in range(M) if m % 5 == 4]
    slots_in = [(-1 if m in padding else s) for m, s in enumerate(slots)]
    theta, n_pos = 9999.0, 64
    inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    fr = torch.outer(torch.arange(n_pos).float(), inv)
    cos, sin = fr.cos().to(DEV), fr.sin().to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tok_row, tok_pos, row_slot = i32(list(range(M))), i32(ctx), i32(slots_in)
    order = paired_order(n_q, n_kv, d)
    wp, bp = w[order].contiguous().to(DEV), b[order].contiguous().to(DEV)
    qkv = (P.linear(x.double(), w.double(), b.double())).view(M, n_q + 2 * n_kv, d)
    c2, s2 = P.rope_tables(d, n_pos, theta)
    rot = P.apply_rope(qkv[:, :n_q + n_kv], c2[torch.tensor(ctx)], s2[torch.tensor(ctx)])
    live = [m for m in range(M) if m not in padding]
    for splits in (0, 1, 2, 8):
        for bias in (bp, bp.float()):
            kp = torch.zeros(total, n_kv, bs, d, dtype=bf, device=DEV)
            vp = torch.zeros_like(kp)
            q_out = torch.zeros(M, n_q * d, dtype=bf, device=DEV)
            st = status()
            K.gemm_stream_qkv_rope(x.to(DEV), wp, bias, q_out, cos, sin, tok_row, tok_pos, row_slot, kp, vp,
                                   table.to(DEV), n_q, n_kv, d, True, st, splits)
            assert int(st.item()) == 0
            assert rel(q_out.view(M, n_q, d)[live], rot[live, :n_q]) < 6e-3
            assert float(q_out.view(M, n_q, d)[padding].abs().max() if padding else 0.0) == 0.0
            for m in live:
                blk = int(table[slots[m], ctx[m] // bs])
                assert rel(kp[blk, :, ctx[m] % bs], rot[m, n_q:]) < 6e-3
                assert rel(vp[blk, :, ctx[m] % bs], qkv[m, n_q + n_kv:]) < 6e-3
            assert int((kp != 0).sum().item()) <= len(live) * n_kv * d        # only this step's positions were written
    # an entry that reads another entry's cache writes no keys
    kp.zero_()
    K.gemm_stream_qkv_rope(x.to(DEV), wp, bp, q_out, cos, sin, tok_row, tok_pos, row_slot, kp, vp, table.to(DEV),
                           n_q, n_kv, d, False, status())
    assert float(kp.abs().max()) == 0.0


@pytest.mark.parametrize("n_q,n_kv,d,bs,Kd", [(12, 2, 128, 16, 1536), (6, 2, 48, 4, 96), (5, 1, 64, 32, 72)])
def test_prompt_projection_with_rotary_epilogue(n_q, n_kv, d, bs, Kd, tc_tiling):
    """The tcgen05 q/k/v projection over two prompts (several 128-row tiles, a
    ragged last one), one of them continuing a cached prefix, plus a padding row."""
    g = torch.Generator().manual_seed(n_q)
    bf = torch.bfloat16
    N = (n_q + 2 * n_kv) * d
    ctx, new = [0, 37], [170, 131]
    T = sum(new) + 1                                  # one extra token belongs to a padding row
    x = torch.randn(T, Kd, generator=g).to(bf)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(bf)
    b = (0.5 * torch.randn(N, generator=g)).to(bf)
    table, slots, total = scrambled_table([c + n for c, n in zip(ctx, new)], bs, 4, g)
    theta, n_pos = 7777.0, 256
    inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    fr = torch.outer(torch.arange(n_pos).float(), inv)
    cos, sin = fr.cos().to(DEV), fr.sin().to(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    rows = [r for r, n in enumerate(new) for _ in range(n)] + [2]
    pos = [c + i for c, n in zip(ctx, new) for i in range(n)] + [0]
    order = paired_order(n_q, n_kv, d)
    kp = torch.zeros(total, n_kv, bs, d, dtype=bf, device=DEV)
    vp = torch.zeros_like(kp)
    q_out = torch.zeros(T, n_q * d, dtype=bf, device=DEV)
    st = status()
    K.gemm_tc_qkv_rope(x.to(DEV), w[order].contiguous().to(DEV), b[order].contiguous().to(DEV), q_out, cos, sin,
                       i32(rows), i32(pos), i32(slots + [-1]), kp, vp, table.to(DEV), n_q, n_kv, d, True, st)
    assert int(st.item()) == 0
    qkv = P.linear(x.double(), w.double(), b.double()).view(T, n_q + 2 * n_kv, d)
    c2, s2 = P.rope_tables(d, n_pos, theta)
    rot = P.apply_rope(qkv[:, :n_q + n_kv], c2[torch.tensor(pos)], s2[torch.tensor(pos)])
    assert rel(q_out.view(T, n_q, d)[:-1], rot[:-1, :n_q]) < 6e-3
    assert float(q_out[-1].float().abs().max()) == 0.0            # the padding row's token is left alone
    for t in list(range(0, T - 1, 17)) + [T - 2]:
        blk = int(table[slots[rows[t]], pos[t] // bs])
        assert rel(kp[blk, :, pos[t] % bs], rot[t, n_q:]) < 6e-3
        assert rel(vp[blk, :, pos[t] % bs], qkv[t, n_q + n_kv:]) < 6e-3
    assert int((kp != 0).sum().item()) <= sum(new) * n_kv * d


def attention_reference(q, k_seqs, v_seqs, ctx, new, n_q, n_kv, d, scale, window):
    """Plain causal GQA attention of the new tokens of every row (float64)."""
    G = n_q // n_kv
    outs = []
    o = 0
    for ks, vs, c, n in zip(k_seqs, v_seqs, ctx, new):
        qq = q[o:o + n].double().view(n, n_q, d)
        o += n
        out = torch.zeros(n, n_q, d, dtype=torch.float64)
        for i in range(n):
            pos = c + i
            lo = max(0, pos - window + 1) if window else 0
            for h in range(n_q):
                sc = (ks[lo:pos + 1, h // G].double() @ qq[i, h]) * scale
                out[i, h] = torch.softmax(sc, 0) @ vs[lo:pos + 1, h // G].double()
        outs.append(out.view(n, n_q * d))
    return torch.cat(outs)


def run_attention(dtype, n_q, n_kv, d, bs, ctx, new, window=0, n_splits=1, split_len=0, seed=7,
                  spike=None, pad_rows=0, fn=None, qk_scale=1.0, ramp=0.0, expect_status=0):
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    lens = [c + n for c, n in zip(ctx, new)]
    table, slots, total = scrambled_table(lens, bs, len(lens) + 2, g)
    k_seqs = [torch.randn(n, n_kv, d, generator=g).to(dt) for n in lens]
    v_seqs = [torch.randn(n, n_kv, d, generator=g).to(dt) for n in lens]
    T = sum(new)
    q = (torch.randn(T, n_q * d, generator=g) * qk_scale).to(dt)
    if ramp:
        # scores that rise along the keys by `ramp` (in units of the softmax's exponent) per key
        u = torch.zeros(d)
        u[0] = 1.0
        k_seqs = [(k.float() * (1 - u) + u * ramp * math.sqrt(d) * torch.arange(len(k)).view(-1, 1, 1)).to(dt) for k in k_seqs]
        q = (q.float().view(T, n_q, d) * (1 - u) + u).view(T, n_q * d).to(dt)
    if spike is not None:
        # one far key and one query made to match: its score stands out, so a
        # kernel that drops that key (a split boundary, a window edge) shows
        row, key_pos = spike
        k_seqs[row][key_pos] *= 6.0
        q.view(T, n_q, d)[sum(new[:row + 1]) - 1] = k_seqs[row][key_pos].repeat_interleave(n_q // n_kv, 0) * 0.8
    kp, vp = fill_pools(k_seqs, v_seqs, table, slots, bs, total, dt)
    rows = len(new) + pad_rows
    new_p, ctx_p, slots_p = new + [1] * pad_rows, ctx + [0] * pad_rows, slots + [-1] * pad_rows
    Tp = T + pad_rows
    qp = torch.cat([q, torch.zeros(pad_rows, n_q * d, dtype=dt)]).to(DEV)
    starts = [sum(new_p[:i]) for i in range(rows)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tok_row = i32([r for r, n in enumerate(new_p) for _ in range(n)])
    out = torch.full((Tp, n_q * d), float("nan"), dtype=dt, device=DEV)
    scratch = None
    if n_splits > 1:
        scratch = torch.full((K.attention_scratch_floats(Tp, n_q, d, n_splits),), float("nan"), device=DEV)
    st = status()
    scale = 1.0 / math.sqrt(d)
    (fn or K.attention_simt)(qp, kp, vp, out, table.to(DEV), tok_row, i32(slots_p), i32(starts), i32(new_p), i32(ctx_p),
                     rows, max(new_p), n_q, n_kv, d, scale, window, n_splits, split_len, scratch, st)
    assert int(st.item()) == expect_status
    want = attention_reference(q, k_seqs, v_seqs, ctx, new, n_q, n_kv, d, scale, window)
    return out[:T], want, out[T:]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_q,n_kv,d,bs", [(6, 2, 48, 4), (5, 1, 16, 16), (12, 2, 128, 16), (7, 7, 80, 32),
                                           (4, 2, 256, 8), (28, 4, 128, 16)])
def test_attention_prompts(dtype, n_q, n_kv, d, bs):
    """Whole prompts of unequal lengths, some continuing a cached prefix."""
    got, want, _ = run_attention(dtype, n_q, n_kv, d, bs, ctx=[0, 0, 13, 0], new=[1, 37, 22, 70])
    assert rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 5, 32, 33])
def test_attention_window(dtype, window):
    got, want, _ = run_attention(dtype, 6, 2, 32, 8, ctx=[0, 40, 7], new=[50, 9, 1], window=window)
    assert rel(got, want) < TOL[dtype]
    got, want, _ = run_attention(dtype, 6, 2, 32, 8, ctx=[64, 40, 7], new=[1, 1, 1], window=window,
                                 n_splits=3, split_len=32)
    assert rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_splits,split_len", [(1, 0), (2, 160), (4, 96), (10, 32), (16, 64)])
def test_attention_decode_splits(dtype, n_splits, split_len):
    """One new token per row over cached lengths 0..300; more splits than some
    rows have keys for (empty partial results), and a padding row."""
    got, want, pad = run_attention(dtype, 12, 2, 64, 16, ctx=[0, 15, 16, 299, 100], new=[1] * 5,
                                   n_splits=n_splits, split_len=split_len, pad_rows=2)
    assert rel(got, want) < TOL[dtype]
    if n_splits > 1:
        assert float(pad.float().abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_decode_splits_odd_counts(dtype):
    """One row, three heads, an odd number of splits: every sub-array of the
    scratch memory starts at an odd multiple of something."""
    for n_q, n_kv, n_splits, split_len in ((3, 1, 3, 64), (5, 5, 7, 32), (1, 1, 5, 32)):
        got, want, _ = run_attention(dtype, n_q, n_kv, 32, 16, ctx=[150], new=[1], n_splits=n_splits,
                                     split_len=split_len)
        assert rel(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_far_key_stands_out(dtype):
    """Among 700 keys one early key carries nearly all the weight of the last
    query; it lies in the first split and in a block far from the others."""
    for key_pos in (0, 31, 32, 255, 256, 698):
        got, want, _ = run_attention(dtype, 6, 2, 64, 16, ctx=[699, 40], new=[1, 1], n_splits=6, split_len=128,
                                     spike=(0, key_pos))
        assert rel(got, want) < TOL[dtype], key_pos
        got, want, _ = run_attention(dtype, 6, 2, 64, 16, ctx=[0, 0], new=[700, 3], spike=(0, key_pos))
        assert rel(got, want) < TOL[dtype], key_pos


@pytest.fixture(params=[0, 1, 2, 4, 5], ids=["auto", "heads_as_rows", "four_warps", "eight_warps", "heads_as_rows_eight_warps"])
def decode_form(request):
    """The forms of the tensor-core decode attention: keys or heads as the rows of the MMAs (the first for
    groups of up to 8 heads only), CTAs of four or eight warps."""
    K.attn_decode_set_form(request.param)
    yield request.param
    K.attn_decode_set_form(0)


@pytest.mark.parametrize("n_q,n_kv,d,bs", [(12, 2, 128, 16), (7, 1, 128, 4), (5, 5, 64, 32), (16, 1, 64, 16),
                                           (28, 4, 128, 16), (40, 8, 128, 8), (3, 3, 128, 1)])
@pytest.mark.parametrize("n_splits,split_len", [(1, 0), (2, 160), (3, 128), (11, 32), (16, 32), (33, 32)])
def test_attention_decode_tensor_cores(n_q, n_kv, d, bs, n_splits, split_len, decode_form):
    """The dispatcher's tensor-core kernel for bfloat16 decode steps: groups that
    are no power of two, cached lengths at tile and split edges, a padding row.
    The CTA that finishes last merges the splits and leaves zeros in padding rows."""
    ctx = [0, 15, 16, 17, 127, 128, 300, 63]
    got, want, pad = run_attention("bfloat16", n_q, n_kv, d, bs, ctx=ctx, new=[1] * len(ctx),
                                   n_splits=n_splits, split_len=split_len, pad_rows=1, fn=K.attention)
    assert rel(got, want) < TOL["bfloat16"]
    if n_splits > 1:
        assert float(pad.float().abs().max()) == 0.0


# head size 128: K.attention takes the tcgen05 kernel, K.attention_mma_sync the mma.sync one
def _attention_in_form(form):
    def fn(*args, **kwargs):
        K.attn_prefill_set_form(form)
        try:
            return K.attention(*args, **kwargs)
        finally:
            K.attn_prefill_set_form(0)
    return fn


# the dispatcher's own choice; the tcgen05 kernel with two query tiles per CTA; the same with one query tile whose
# key tiles are dealt to the two softmax groups; the mma.sync kernel
PROMPT_KERNELS = [K.attention, _attention_in_form(1), _attention_in_form(2), K.attention_mma_sync]
PROMPT_IDS = ["auto", "two_tiles", "dealt_keys", "mma_sync"]


@pytest.mark.parametrize("fn", PROMPT_KERNELS, ids=PROMPT_IDS)
@pytest.mark.parametrize("n_q,n_kv,d,bs", [(12, 2, 128, 16), (7, 1, 128, 4), (5, 5, 64, 32), (6, 2, 64, 16), (28, 4, 128, 8)])
def test_attention_prompts_tensor_cores(n_q, n_kv, d, bs, fn):
    """The dispatcher's tensor-core kernels for bfloat16 prompt steps: unequal
    lengths around the 64-token tile edges, some continuing a cached prefix."""
    got, want, _ = run_attention("bfloat16", n_q, n_kv, d, bs, ctx=[0, 0, 13, 0, 100, 64], new=[1, 64, 65, 130, 30, 63],
                                 fn=fn)
    assert rel(got, want) < TOL["bfloat16"]


@pytest.mark.parametrize("fn", PROMPT_KERNELS, ids=PROMPT_IDS)
@pytest.mark.parametrize("window", [1, 5, 63, 64, 65, 200])
def test_attention_prompts_tensor_cores_window_and_far_key(window, fn):
    got, want, _ = run_attention("bfloat16", 6, 2, 64, 16, ctx=[0, 90, 7], new=[150, 70, 1], window=window, fn=fn)
    assert rel(got, want) < TOL["bfloat16"]
    if window == 200:
        for key_pos in (0, 63, 64, 400, 639, 698):
            got, want, _ = run_attention("bfloat16", 12, 2, 128, 16, ctx=[0, 0], new=[700, 3], spike=(0, key_pos),
                                         fn=fn)
            assert rel(got, want) < TOL["bfloat16"], key_pos
            got, want, _ = run_attention("bfloat16", 12, 2, 128, 16, ctx=[640, 0], new=[60, 3], spike=(0, key_pos),
                                         fn=fn)
            assert rel(got, want) < TOL["bfloat16"], key_pos


@pytest.mark.parametrize("form", [1, 2], ids=["two_tiles", "dealt_keys"])
def test_attention_prompts_tcgen05_large_scores(form):
    """The tcgen05 kernel moves a row's running maximum only when it grows by more than 2^8:
    scores that rise steadily along the keys (each tile a little above the last), scores that
    jump far, and a long prompt over several hundred keys must all come out the same."""
    for qk_scale, ramp in ((1.0, 0.0), (6.0, 0.0), (30.0, 0.0), (1.0, 0.05), (1.0, 0.125), (1.0, 1.0), (0.0, 0.03)):
        got, want, _ = run_attention("bfloat16", 4, 2, 128, 16, ctx=[0, 300], new=[520, 200], fn=_attention_in_form(form),
                                     qk_scale=qk_scale, ramp=ramp)
        assert rel(got, want) < TOL["bfloat16"], (qk_scale, ramp)


@pytest.mark.parametrize("window", [1, 40, 127, 128, 129, 300])
@pytest.mark.parametrize("bs", [8, 16, 64, 128])
@pytest.mark.parametrize("form", [1, 2], ids=["two_tiles", "dealt_keys"])
def test_attention_prompts_tcgen05_window(window, bs, form):
    """Head size 128 goes to the tcgen05 kernel: windows around its tiles of 64 keys and 128
    queries, every block size it takes, prompts that continue a cached prefix."""
    got, want, _ = run_attention("bfloat16", 6, 2, 128, bs, ctx=[0, 150, 7, 256], new=[260, 130, 1, 128], window=window,
                                 fn=_attention_in_form(form))
    assert rel(got, want) < TOL["bfloat16"]


@pytest.mark.parametrize("window", [1, 16, 17, 100])
def test_attention_decode_tensor_cores_window_and_far_key(window, decode_form):
    got, want, _ = run_attention("bfloat16", 6, 2, 128, 16, ctx=[200, 40, 7], new=[1, 1, 1], window=window,
                                 n_splits=4, split_len=64, fn=K.attention)
    assert rel(got, want) < TOL["bfloat16"]
    for key_pos in (0, 15, 16, 255, 256, 511, 698):
        got, want, _ = run_attention("bfloat16", 12, 2, 128, 16, ctx=[699, 40], new=[1, 1], n_splits=6,
                                     split_len=128, spike=(0, key_pos), fn=K.attention)
        assert rel(got, want) < TOL["bfloat16"], key_pos


def test_attention_refuses_what_it_cannot_do():
    with pytest.raises(K.KernelError, match="head size"):
        run_attention("float32", 4, 2, 24, 4, ctx=[0], new=[3])
    with pytest.raises(K.KernelError, match="multiple"):
        run_attention("float32", 5, 2, 32, 4, ctx=[0], new=[3])


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("V", [7, 256, 333, 151936])
def test_sample_greedy_and_temperature(V):
    g = torch.Generator().manual_seed(9)
    n = 5
    logits = torch.randn(n, V, generator=g)
    logits[1, V // 2] = logits[1].max() + 1          # a clear winner
    logits[2, :] = 0.25                              # all tied: the lowest index wins
    logits[3, V - 1] = logits[3, 0] = 9.0            # two tied winners
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    K.sample(logits.to(DEV), out)
    want = [P.sample(logits[i], 0.0, 0, 0, 0) for i in range(n)]
    assert out.tolist() == want
    assert out[2].item() == 0 and out[3].item() == 0 and out[1].item() == V // 2
    if V > 1000:
        n = 2
    temps = [0.8, 0.0, 1.3, 0.5, 2.0][:n]
    reqs = [3, 1, 2 ** 40 + 5, 0, 7][:n]
    steps = [0, 5, 1, 2, 9][:n]
    K.sample(logits[:n].to(DEV), out[:n], torch.tensor(temps, device=DEV),
             torch.tensor(reqs, dtype=torch.int64, device=DEV), torch.tensor(steps, dtype=torch.int32, device=DEV),
             seed=2 ** 33 + 17)
    want = [P.sample(logits[i], temps[i], 2 ** 33 + 17, reqs[i], steps[i]) for i in range(n)]
    assert out[:n].tolist() == want


def test_sample_temperature_follows_the_distribution():
    """Over many (request, step) keys the draws follow softmax(logits / T)."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]])
    n = 4000
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    K.sample(logits.expand(n, 5).contiguous().to(DEV), out, torch.full((n,), 0.7, device=DEV),
             torch.arange(n, dtype=torch.int64, device=DEV), torch.zeros(n, dtype=torch.int32, device=DEV), seed=1)
    freq = torch.bincount(out.cpu().long(), minlength=5).double() / n
    want = torch.softmax(logits[0].double() / 0.7, 0)
    assert float((freq - want).abs().max()) < 0.03


# ---------------------------------------------------------------------------
# drawn shapes: what the hand-picked cases above may have missed
# ---------------------------------------------------------------------------
def test_attention_prompts_drawn_shapes():
    """Prompt steps at head size 128 with drawn group sizes, block sizes, cached prefixes, prompt lengths
    around the 128- and 256-row tiles and windows (both forms of the tcgen05 kernel in turn, and the decode
    kernel where every sequence brings one token)."""
    import random
    rnd = random.Random(11)
    for case in range(40):
        n_kv = rnd.choice([1, 2, 3])
        n_q = n_kv * rnd.choice([1, 2, 3, 6])
        bs = rnd.choice([8, 16, 32, 64, 128])
        n_seq = rnd.randint(1, 4)
        ctx = [rnd.choice([0, 0, rnd.randint(1, 300)]) for _ in range(n_seq)]
        new = [rnd.choice([1, rnd.randint(2, 127), 128, 129, 255, 256, 257, rnd.randint(130, 600)]) for _ in range(n_seq)]
        window = rnd.choice([0, 0, 1, rnd.randint(2, 700), 64, 128, 256])
        got, want, _ = run_attention("bfloat16", n_q, n_kv, 128, bs, ctx=ctx, new=new, window=window,
                                     fn=_attention_in_form(1 + case % 2), seed=case)
        assert rel(got, want) < TOL["bfloat16"], dict(n_q=n_q, n_kv=n_kv, bs=bs, ctx=ctx, new=new, window=window,
                                                      form=1 + case % 2)


def test_attention_decode_drawn_shapes():
    """Decode steps on the tensor-core kernel with drawn head sizes, groups, block sizes (also below a
    16-key tile and no power of two), lengths, windows and splits of the keys."""
    import random
    rnd = random.Random(12)
    for case in range(60):
        d = rnd.choice([64, 128])
        n_kv = rnd.choice([1, 2, 4])
        n_q = n_kv * rnd.choice([1, 2, 3, 6, 7, 16])
        bs = rnd.choice([1, 4, 8, 16, 32, 64, 48])
        n_seq = rnd.randint(1, 6)
        ctx = [rnd.choice([0, rnd.randint(1, 40), rnd.randint(41, 900)]) for _ in range(n_seq)]
        window = rnd.choice([0, 0, 1, rnd.randint(2, 900), 16, 128])
        n_splits = rnd.choice([1, 2, 3, 5, 8, 16, 17, 32])
        split_len = 0
        if n_splits > 1:
            split_len = -(-(-(-(max(ctx) + 1) // n_splits)) // 32) * 32 + rnd.choice([0, 32])
        got, want, _ = run_attention("bfloat16", n_q, n_kv, d, bs, ctx=ctx, new=[1] * n_seq, window=window,
                                     n_splits=n_splits, split_len=split_len, pad_rows=rnd.choice([0, 2]),
                                     fn=K.attention, seed=case)
        assert rel(got, want) < TOL["bfloat16"], dict(d=d, n_q=n_q, n_kv=n_kv, bs=bs, ctx=ctx, window=window,
                                                      n_splits=n_splits, split_len=split_len)


def test_gemm_tcgen05_drawn_shapes():
    """The four tilings of the tcgen05 product at drawn M, N, K: around the tile edges, fewer rows than one
    CTA of a pair holds, N between one and two wide tiles, K that is no multiple of the 64-wide stage."""
    import random
    rnd = random.Random(13)
    st = status()
    try:
        for case in range(60):
            M = rnd.choice([1, 17, 127, 128, 129, 255, 256, 257, 300, 512, 1000, rnd.randint(1, 2500)])
            N = rnd.choice([16, 256, 272, 384, 511, 512, 528, 1536, 2048, rnd.randint(1, 300) * 16])
            K_ = rnd.choice([8, 64, 72, 128, 200, 1536, rnd.randint(1, 200) * 8])
            tiling = case % 4
            K.gemm_tc_set_wide(tiling)
            g = torch.Generator().manual_seed(case)
            x = torch.randn(M, K_, generator=g).to(torch.bfloat16).to(DEV)
            w = (torch.randn(N, K_, generator=g) / math.sqrt(K_)).to(torch.bfloat16).to(DEV)
            b = torch.randn(N, generator=g).to(torch.bfloat16).to(DEV)
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
            K.gemm_tc(x, w, b, out, status=st)
            assert rel(out, P.linear(x.double(), w.double()) + b.double()) < 5e-3, (M, N, K_, tiling)
        assert int(st.item()) == 0
    finally:
        K.gemm_tc_set_wide(TC_DEFAULT_TILING)


# ---------------------------------------------------------------------------
# the status word: an index that a kernel had to skip, and a bounded wait that ran out

def _rotary_case(M, n_q, n_kv, d, bs, Kd, n_pos, seed):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    N = (n_q + 2 * n_kv) * d
    x = torch.randn(M, Kd, generator=g).to(bf).to(DEV)
    order = paired_order(n_q, n_kv, d)
    w = (torch.randn(N, Kd, generator=g) / math.sqrt(Kd)).to(bf)[order].contiguous().to(DEV)
    ctx = [int(v) for v in torch.randint(0, n_pos - 1, (M,), generator=g)]
    table, slots, total = scrambled_table([c + 1 for c in ctx], bs, M + 2, g)
    inv = 1.0 / (1e4 ** (torch.arange(0, d, 2).float() / d))
    fr = torch.outer(torch.arange(n_pos).float(), inv)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    kp = torch.zeros(total, n_kv, bs, d, dtype=bf, device=DEV)
    return dict(x=x, w=w, cos=fr.cos().to(DEV), sin=fr.sin().to(DEV), tok_row=i32(list(range(M))), tok_pos=i32(ctx),
                row_slot=i32(slots), kp=kp, vp=torch.zeros_like(kp), table=table.to(DEV), slots=slots, ctx=ctx,
                q=torch.zeros(M, n_q * d, dtype=bf, device=DEV))


ROTARY_KERNELS = {
    "gemv": lambda c, dims, st: K.gemv_qkv_rope(c["x"], c["w"], None, c["q"], c["cos"], c["sin"], c["tok_row"], c["tok_pos"],
                                                c["row_slot"], c["kp"], c["vp"], c["table"], *dims, True, st, 1),
    "stream": lambda c, dims, st: K.gemm_stream_qkv_rope(c["x"], c["w"], None, c["q"], c["cos"], c["sin"], c["tok_row"],
                                                         c["tok_pos"], c["row_slot"], c["kp"], c["vp"], c["table"], *dims,
                                                         True, st),
    "prompt": lambda c, dims, st: K.gemm_tc_qkv_rope(c["x"], c["w"], None, c["q"], c["cos"], c["sin"], c["tok_row"],
                                                     c["tok_pos"], c["row_slot"], c["kp"], c["vp"], c["table"], *dims, True, st),
    "separate": lambda c, dims, st: K.rope_append((c["x"] @ c["w"].T).contiguous(), c["q"], c["cos"], c["sin"], c["tok_row"],
                                                  c["tok_pos"], c["row_slot"], c["kp"], c["vp"], c["table"], *dims, True, st,
                                                  paired=True),
}


def test_launch_count_counts_kernels_where_they_are_launched():
    """``launch_count`` rises by one for a product, by one for a decode attention that merges its own splits, by
    two for the float32 attention with splits (its merge is a kernel of its own), and by nothing for a call that
    the launcher refuses."""
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(4, 32, dtype=torch.bfloat16, device=DEV)
    n0 = K.launch_count()
    K.gemv(x, w, None, out, K.GEMV_BF16)
    assert K.launch_count() == n0 + 1
    run_attention("bfloat16", 6, 2, 128, 16, ctx=[300, 40], new=[1, 1], n_splits=3, split_len=128, fn=K.attention)
    assert K.launch_count() == n0 + 2
    run_attention("float32", 6, 2, 128, 16, ctx=[300, 40], new=[1, 1], n_splits=3, split_len=128, fn=K.attention)
    assert K.launch_count() == n0 + 4
    with pytest.raises(K.KernelError):
        K.gemm_stream(torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV), torch.zeros(16, 12, dtype=torch.bfloat16, device=DEV),
                      None, torch.zeros(4, 16, dtype=torch.bfloat16, device=DEV))
    assert K.launch_count() == n0 + 4
    torch.cuda.synchronize()


@pytest.mark.parametrize("kernel", list(ROTARY_KERNELS))
def test_status_bits_of_the_rotary_kernels(kernel):
    """A token whose place in the cache maps to no block (a -1 in the table under a live length), and a
    position beyond the rotation table: the kernel skips the access, says so in the status word, writes
    nothing for that token and everything for the others.  Nothing faults."""
    dims = (6, 2, 64)
    M, bs = 12, 16
    # a missing block
    c = _rotary_case(M, *dims, bs, 128, 200, seed=1)
    bad = 5
    good_blk = int(c["table"][c["slots"][bad], c["ctx"][bad] // bs])
    c["table"][c["slots"][bad], c["ctx"][bad] // bs] = -1
    st = status()
    ROTARY_KERNELS[kernel](c, dims, st)
    assert int(st.item()) == K.STATUS_BAD_BLOCK
    assert float(c["kp"][good_blk].float().abs().max()) == 0.0               # nothing written for that token
    other = 0 if bad else 1
    blk = int(c["table"][c["slots"][other], c["ctx"][other] // bs])
    assert float(c["kp"][blk, :, c["ctx"][other] % bs].float().abs().max()) > 0.0
    # a block number beyond the pool
    c = _rotary_case(M, *dims, bs, 128, 200, seed=2)
    c["table"][c["slots"][bad], c["ctx"][bad] // bs] = c["kp"].shape[0] + 7
    st = status()
    ROTARY_KERNELS[kernel](c, dims, st)
    assert int(st.item()) == K.STATUS_BAD_BLOCK
    # a rotation table shorter than a position
    c = _rotary_case(M, *dims, bs, 128, 200, seed=3)
    short = max(c["ctx"])                                                     # the table ends just before the farthest position
    c["cos"], c["sin"] = c["cos"][:short].contiguous(), c["sin"][:short].contiguous()
    st = status()
    ROTARY_KERNELS[kernel](c, dims, st)
    assert int(st.item()) & K.STATUS_BAD_POSITION
    assert "rotation table" in K.status_message(int(st.item()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_status_bit_of_attention_over_a_missing_block(dtype):
    """A -1 in the block table inside a sequence's length: prompt and decode attention (CUDA cores in float32,
    tensor cores in bfloat16) skip the block, set the status bit and return."""
    g = torch.Generator().manual_seed(3)
    dt = DT[dtype]
    n_q, n_kv, d, bs = 6, 2, 64, 16
    for new, n_splits, split_len in (([1, 1], 1, 0), ([1, 1], 3, 64), ([40, 9], 1, 0)):
        ctx = [150, 33]
        lens = [c + n for c, n in zip(ctx, new)]
        table, slots, total = scrambled_table(lens, bs, 4, g)
        table[slots[0], 2] = -1                                               # keys 32..47 of the first sequence
        kp = torch.randn(total, n_kv, bs, d, generator=g).to(dt).to(DEV)
        vp = torch.randn(total, n_kv, bs, d, generator=g).to(dt).to(DEV)
        T = sum(new)
        q = torch.randn(T, n_q * d, generator=g).to(dt).to(DEV)
        out = torch.zeros(T, n_q * d, dtype=dt, device=DEV)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        starts = [0, new[0]]
        tok_row = i32([0] * new[0] + [1] * new[1])
        scratch = torch.zeros(max(1, K.attention_scratch_floats(T, n_q, d, n_splits)), device=DEV)
        st = status()
        K.attention(q, kp, vp, out, table.to(DEV), tok_row, i32(slots), i32(starts), i32(new), i32(ctx), 2, max(new),
                    n_q, n_kv, d, 0.125, 0, n_splits, split_len, scratch, st)
        assert int(st.item()) == K.STATUS_BAD_BLOCK, (new, n_splits)
        assert bool(torch.isfinite(out.float()).all())


def test_bounded_waits_report_and_return(tc_tiling):
    """The TMA + tcgen05 kernels with their wait limit set to a millisecond and their producers told to leave
    out their very last copy: the consumer's wait runs out, the kernel sets STATUS_WAIT_TIMEOUT, frees its
    tensor memory and returns; the next launch, with the hook off, is correct.  Nothing hangs or faults."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(200, 256, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(512, 256, generator=g) / 16).to(torch.bfloat16).to(DEV)
    want = P.linear(x.double(), w.double())
    out = torch.zeros(200, 512, dtype=torch.bfloat16, device=DEV)
    xs = x[:40].contiguous()
    outs = torch.zeros(40, 512, dtype=torch.bfloat16, device=DEV)
    try:
        K.tc_test_hook(wait_ns=1_000_000, skip_last=True)
        st = status()
        K.gemm_tc(x, w, None, out, status=st)
        torch.cuda.synchronize()
        assert int(st.item()) == K.STATUS_WAIT_TIMEOUT
        for splits in (1, 2):
            st = status()
            K.gemm_stream(xs, w, None, outs, splits=splits, status=st)
            torch.cuda.synchronize()
            assert int(st.item()) == K.STATUS_WAIT_TIMEOUT, splits
    finally:
        K.tc_test_hook()
    st = status()
    K.gemm_tc(x, w, None, out, status=st)
    K.gemm_stream(xs, w, None, outs, status=st)
    assert int(st.item()) == 0
    assert rel(out, want) < 5e-3 and rel(outs, want[:40]) < 5e-3


@pytest.mark.parametrize("form", [1, 2], ids=["two_tiles", "dealt_keys"])
def test_bounded_waits_of_the_prompt_attention(form):
    """The same for the tcgen05 prompt attention: one copy of a CTA's last key tile never leaves, the waits run
    out one after another, the status bit is set, and the next launch is correct."""
    run = _attention_in_form(form)
    try:
        K.tc_test_hook(wait_ns=1_000_000, skip_last=True)
        run_attention("bfloat16", 4, 2, 128, 16, ctx=[0], new=[200], fn=run, expect_status=K.STATUS_WAIT_TIMEOUT)
    finally:
        K.tc_test_hook()
    got, want, _ = run_attention("bfloat16", 4, 2, 128, 16, ctx=[0], new=[200], fn=run)
    assert rel(got, want) < TOL["bfloat16"]
