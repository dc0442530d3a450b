"""Each kernel alone against a plain float32 PyTorch statement of the same operation, at
sizes other than the engine's (odd widths, partial tiles, partial pages, poisoned slots)."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (1, 4096, 4096), (5, 311, 96), (16, 256, 128), (17, 384, 200),
                                   (33, 130, 72), (64, 1000, 512), (100, 128, 8), (129, 2048, 1024), (300, 520, 264),
                                   (2048, 1536, 512), (8, 12288, 4096), (7, 4096, 12288), (200, 512, 1024), (256, 384, 4096)])
@pytest.mark.parametrize("mode", ["bf16", "f32", "acc"])
def test_gemm_tensor_core(T, N, K, mode):
    from reinfer_b200 import ops
    a, w = rnd(T, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    ref = a.float() @ w.float().t()
    if mode == "bf16":
        c = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_bf16(a, w, c)
        want = ref
    elif mode == "f32":
        c = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
        ops.gemm_bf16(a, w, c)
        want = ref
    else:
        base = rnd(T, N, seed=3)
        c = base.clone()
        ops.gemm_bf16(a, w, c, accumulate=True)
        want = base + ref
    assert ops.kernel_error() == 0
    tol = 4e-3 if mode == "bf16" else 2e-5 * math.sqrt(K) + 1e-6          # bfloat16: one rounding of the result
    err = (c.float() - want).abs().max().item() / max(want.abs().max().item(), 1e-6)
    assert err <= tol, f"relative error {err:.3e}"


@pytest.mark.parametrize("T,F,K", [(1, 128, 64), (1, 12288, 4096), (8, 12288, 4096), (5, 160, 96), (17, 300, 200), (40, 1000, 512),
                                   (64, 2048, 1024), (100, 130, 72), (65, 1000, 520), (128, 9728, 2560), (129, 640, 264), (300, 520, 520), (2048, 1024, 512),
                                   (200, 512, 512), (130, 1024, 2048), (256, 256, 4096)])
def test_gemm_swiglu_epilogue(T, F, K):
    from reinfer_b200 import ops
    a = rnd(T, K, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * F, K, dtype=torch.bfloat16, scale=0.08, seed=2)
    out = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.gemm_bf16_swiglu(a, w, out)
    assert ops.kernel_error() == 0
    g, u = a.float() @ w[:F].float().t(), a.float() @ w[F:].float().t()
    ref = g / (1 + torch.exp(-g)) * u
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()


@pytest.mark.parametrize("T,N,K", [(257, 256, 64), (300, 700, 320), (1000, 130, 520), (2048, 4096, 1024), (777, 1000, 4104),
                                   (513, 384, 8192)])
@pytest.mark.parametrize("token_lanes", [0, 1, 224, 256])
def test_gemm_over_many_token_tiles_to_the_roundings_own_width(T, N, K, token_lanes):
    """Prompt portions run persistent CTAs over the output tiles.  Sizes with ragged edges in every direction, every
    output mode and the SwiGLU epilogue, in both forms of the kernel (a feature or a token per accumulator lane), held to what the arithmetic allows: a float32 result to the
    accumulation's rounding, a bfloat16 result to one rounding to bfloat16 (4e-3 of the scale) - a wrong 16-column
    step of K, one of K / 16, moves a result by about sqrt(16 / K) of the scale (6 % at K = 4,096) and would show."""
    from reinfer_b200 import ops
    # (values above 1: the token-lane forms with tiles of that many weight rows instead of the width the launcher picks)
    old = ops.set_gemm_token_lanes(1 if token_lanes else 0)
    old_feats = ops.set_gemm_tile_features(token_lanes if token_lanes > 1 else 0)
    try:
        _many_token_tiles(ops, T, N, K)
    finally:
        ops.set_gemm_token_lanes(old)
        ops.set_gemm_tile_features(old_feats)


def _many_token_tiles(ops, T, N, K):
    a = rnd(T, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    ref = a.float() @ w.float().t()
    base = rnd(T, N, seed=3)
    F = N // 2
    g, u = ref[:, :F], ref[:, F:2 * F]
    ref_act = g / (1 + torch.exp(-g)) * u
    c16 = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16(a, w, c16)
    c32 = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_bf16(a, w, c32)
    acc = base.clone()
    ops.gemm_bf16(a, w, acc, accumulate=True)
    act = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.gemm_bf16_swiglu(a, w[:2 * F].contiguous(), act)
    assert ops.kernel_error() == 0
    scale = ref.abs().max().item()
    assert (c32 - ref).abs().max().item() <= (2e-5 * math.sqrt(K) + 1e-6) * scale
    assert (c16.float() - ref).abs().max().item() <= 4e-3 * scale
    assert (acc - base - ref).abs().max().item() <= (2e-5 * math.sqrt(K) + 1e-6) * scale + 1e-5
    assert (act.float() - ref_act).abs().max().item() <= 1e-2 * ref_act.abs().max().item()


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 8, -2, -5, -11])    # > 0: one cluster; < 0: through the workspace
def test_gemm_split_k_is_deterministic(splits):
    from reinfer_b200 import ops
    a, w = rnd(4, 1000, dtype=torch.bfloat16, seed=5), rnd(200, 1000, dtype=torch.bfloat16, seed=6)
    c1 = torch.empty(4, 200, dtype=torch.float32, device=DEV)
    c2 = torch.empty_like(c1)
    ops.gemm_bf16(a, w, c1, splits=splits)
    ops.gemm_bf16(a, w, c2, splits=splits)
    assert torch.equal(c1, c2)
    ref = a.float() @ w.float().t()
    assert (c1 - ref).abs().max().item() <= 1e-3 * ref.abs().max().item()


@pytest.mark.parametrize("T,N,K", [(1, 128, 256), (8, 4096, 4096), (5, 311, 1000), (33, 130, 520), (64, 1000, 2048), (7, 384, 12288)])
def test_gemm_partial_sums_and_the_norm_that_adds_them(T, N, K):
    """A split product may leave its partial sums [S, T, N]; add_rmsnorm adds a stack of them to the residual in
    ascending order before it normalises - twice the same bits, and the sum is the product."""
    from reinfer_b200 import ops
    a, w = rnd(T, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    p1 = ops.gemm_bf16_partials(a, w)
    p2 = ops.gemm_bf16_partials(a, w)
    assert ops.kernel_error() == 0
    assert p1 is not None and p1.dim() == 3 and p1.shape[1:] == (T, N) and p1.dtype == torch.float32
    assert torch.equal(p1, p2)
    ref = a.float() @ w.float().t()
    assert (p1.sum(0) - ref).abs().max().item() <= (2e-5 * math.sqrt(K) + 1e-6) * ref.abs().max().item()
    if p1.shape[0] > 1:                                     # the ranges of K are disjoint: no partial sum is the whole
        assert (p1[0] - ref).abs().max().item() > 1e-3 * ref.abs().max().item()
    # the norm over the residual plus the stack, against the plain statement
    base = rnd(T, N, seed=3)
    gamma = rnd(N, seed=4).abs() + 0.5
    for out_dtype in (torch.bfloat16, torch.float32):
        x = base.clone()
        out = torch.empty(T, N, dtype=out_dtype, device=DEV)
        ops.add_rmsnorm(x, p1, gamma, out, 1e-6)
        want_x = base.clone()
        for k in range(p1.shape[0]):
            want_x += p1[k]
        assert torch.equal(x, want_x)                       # ascending order, float32: the same bits
        want = want_x * torch.rsqrt((want_x * want_x).mean(-1, keepdim=True) + 1e-6) * gamma
        tol = 1e-2 if out_dtype == torch.bfloat16 else 1e-5
        assert (out.float() - want).abs().max().item() <= tol * want.abs().max().item()
    # gathered rows: the sums are formed for those rows only and x stays as it was
    idx = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    x = base.clone()
    out = torch.empty(2, N, dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(x, p1, gamma, out, 1e-6, row_idx=idx)
    assert torch.equal(x, base)
    assert (out.float() - want[idx.long()]).abs().max().item() <= 1e-2 * want.abs().max().item()


@pytest.mark.parametrize("T,h,N", [(1, 128, 256), (8, 4096, 6144), (5, 1000, 311), (33, 520, 130), (64, 2048, 1000), (100, 1040, 260),
                                   (300, 1040, 520), (700, 512, 1000)])
@pytest.mark.parametrize("n_delta", [0, 1, 7])
def test_norm_whose_division_is_left_to_the_product(T, h, N, n_delta):
    """residual_rowscale leaves x*w and the parts of sum(x^2); a product that is told of them multiplies its
    results by the row's factor - together the same as normalising first (plain, cluster-split, gated, partial)."""
    from reinfer_b200 import ops
    eps = 1e-6
    base = rnd(T, h, seed=1, scale=3.0)
    gamma = rnd(h, seed=2).abs() + 0.5
    delta = rnd(n_delta, T, h, seed=3) if n_delta else None
    x = base.clone()
    y, sumsq = ops.residual_rowscale(x, delta if n_delta != 1 else delta[0], gamma)
    want_x = base.clone()
    for k in range(n_delta):
        want_x += delta[k]
    assert torch.equal(x, want_x)
    assert y.dtype == torch.bfloat16 and sumsq.shape[0] == T
    ss = (want_x.double() ** 2).sum(-1)
    assert (sumsq.double().sum(-1) - ss).abs().max().item() <= 1e-5 * ss.max().item()
    assert (y.float() - want_x * gamma).abs().max().item() <= 4e-3 * (want_x * gamma).abs().max().item()
    xn = y.float() * torch.rsqrt(ss / h + eps).float()[:, None]          # what the rows stand for
    w = rnd(N, h, dtype=torch.bfloat16, scale=0.05, seed=4)
    ref = xn @ w.float().t()
    scale = (sumsq, h, eps)
    for splits in ((0, 1, 3) if T <= 256 else (0,)):          # several token tiles: the persistent product only
        c = torch.empty(T, N, dtype=torch.float32, device=DEV)
        ops.gemm_bf16(y, w, c, splits=splits, row_scale=scale)
        assert (c - ref).abs().max().item() <= 2e-4 * ref.abs().max().item(), f"splits {splits}"
    p = ops.gemm_bf16_partials(y, w, row_scale=scale)
    assert (p is None) == (T > ops.STREAMING_TOKENS)          # partial sums are for streaming products only
    if p is not None:
        assert (p.sum(0) - ref).abs().max().item() <= 2e-4 * ref.abs().max().item()
    if N % 2 == 0:
        F = N // 2
        act = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
        for splits in ((0, 1, 2) if T <= 256 else (0,)):
            assert ops.gemm_bf16_swiglu(y, w, act, splits=splits, row_scale=scale)
            g, u = ref[:, :F], ref[:, F:]
            want = g / (1 + torch.exp(-g)) * u
            assert (act.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item(), f"gated, splits {splits}"
    assert ops.kernel_error() == 0


@pytest.mark.parametrize("T,K,N", [(1, 256, 128), (8, 4096, 4096), (8, 12288, 4096), (5, 1000 - 8, 384), (33, 520, 1280), (64, 2048, 2560), (100, 1040, 256), (300, 520, 1040)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
def test_product_that_prepares_the_next_norm(T, K, N, wdt):
    """A decode step's product into the residual whose cluster also makes the next norm's rows: the residual gets the
    product, the rows are the new residual times the norm's weight, and the parts add up to its sum of squares, so
    that a product told of them gives what normalising first gives.  One token tile only."""
    from reinfer_b200 import ops
    eps = 1e-6
    a = rnd(T, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    base = rnd(T, N, seed=3, scale=2.0)
    gamma = (rnd(N, seed=4).abs() + 0.5).to(wdt)
    x = base.clone()
    made = ops.gemm_bf16_residual_norm(a, w, x, gamma)
    assert (made is None) == (T > ops.STREAMING_TOKENS)
    if made is None:
        assert torch.equal(x, base)
        return
    rows, sumsq = made
    want_x = base + a.float() @ w.float().t()
    assert (x - want_x).abs().max().item() <= 2e-4 * want_x.abs().max().item()
    assert rows.dtype == torch.bfloat16 and tuple(sumsq.shape) == (T, N // 128)
    assert (rows.float() - x * gamma.float()).abs().max().item() <= 4e-3 * (x * gamma.float()).abs().max().item()
    ss = (x.double() ** 2).sum(-1)
    assert (sumsq.double().sum(-1) - ss).abs().max().item() <= 1e-5 * ss.max().item()
    xn = rows.float() * torch.rsqrt(ss / N + eps).float()[:, None]
    w2 = rnd(200, N, dtype=torch.bfloat16, scale=0.05, seed=5)
    c = torch.empty(T, 200, dtype=torch.float32, device=DEV)
    ops.gemm_bf16(rows, w2, c, row_scale=(sumsq, N, eps))
    ref = xn @ w2.float().t()
    assert (c - ref).abs().max().item() <= 2e-4 * ref.abs().max().item()
    # a second product in a row, with rows that lack their factor as its own input
    x2 = base.clone()
    w3 = rnd(N, N, dtype=torch.bfloat16, scale=0.05, seed=6)
    made2 = ops.gemm_bf16_residual_norm(rows, w3, x2, gamma, row_scale=(sumsq, N, eps))
    want2 = base + xn @ w3.float().t()
    assert (x2 - want2).abs().max().item() <= 3e-4 * want2.abs().max().item()
    assert (made2[0].float() - x2 * gamma.float()).abs().max().item() <= 4e-3 * (x2 * gamma.float()).abs().max().item()
    assert ops.kernel_error() == 0


def test_gemm_plan_and_prefetch_hint():
    """What the decode product chooses can be asked for; a range to call into L2 changes no result."""
    import ctypes
    from reinfer_b200 import ops
    lib = ops.lib()
    torch.zeros(1, device=DEV)
    for N, K, dual in ((6144, 4096, 0), (4096, 12288, 0), (12288, 4096, 1), (151936, 4096, 0), (128, 64, 0)):
        out = (ctypes.c_int * 9)()
        assert lib.rb_gemm_plan(N, K, dual, out) == 0
        assert 1 <= out[0] <= 8
        tiles = -(-N // 128)
        assert tiles * out[0] <= max(out[out[0]], tiles), "the chosen split fits the resident CTAs (or is no split)"
    a, w = rnd(8, 1024, dtype=torch.bfloat16, seed=1), rnd(512, 1024, dtype=torch.bfloat16, scale=0.05, seed=2)
    nxt = rnd(300, 1000, dtype=torch.bfloat16, seed=3)
    c0 = torch.empty(8, 512, dtype=torch.float32, device=DEV)
    c1 = torch.empty_like(c0)
    ops.gemm_bf16(a, w, c0)
    chain = ops.StreamChain()
    old = ops.set_chain(chain)
    try:
        for _ in range(2):                                  # the second pass knows what follows each product
            chain.begin()
            ops.gemm_bf16(a, w, c1)
            ops.gemm_bf16(a[:, :1000].contiguous(), nxt, torch.empty(8, 300, dtype=torch.float32, device=DEV))
            chain.end()
        assert chain.known == [(w.data_ptr(), w.numel() * 2), (nxt.data_ptr(), nxt.numel() * 2)]
    finally:
        ops.set_chain(old)
    assert ops.kernel_error() == 0
    assert torch.equal(c0, c1)


@pytest.mark.parametrize("ta,tw,tc", [(torch.float32, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.float32, torch.bfloat16),
                                      (torch.float32, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("T,N,K", [(1, 7, 5), (65, 130, 33), (70, 64, 257)])
def test_gemm_plain(ta, tw, tc, T, N, K):
    from reinfer_b200 import ops
    a, w = rnd(T, K, dtype=ta, seed=1), rnd(N, K, dtype=tw, seed=2)
    c = torch.empty(T, N, dtype=tc, device=DEV)
    ops.gemm_ref(a, w, c)
    ref = a.double() @ w.double().t()
    tol = 1e-2 if tc == torch.bfloat16 else 1e-5
    assert (c.double() - ref).abs().max().item() <= tol * ref.abs().max().item()
    if tc == torch.float32:
        base = rnd(T, N, seed=9)
        c2 = base.clone()
        ops.gemm_ref(a, w, c2, accumulate=True)
        assert (c2.double() - (base.double() + ref)).abs().max().item() <= 1e-5 * ref.abs().max().item()
    # a token's row does not depend on the rest of the batch (same bits alone and in the batch)
    c1 = torch.empty(1, N, dtype=tc, device=DEV)
    ops.gemm_ref(a[T // 2:T // 2 + 1], w, c1)
    assert torch.equal(c1[0], c[T // 2])


@pytest.mark.parametrize("h,rows", [(64, 1), (96, 5), (1000, 3), (4096, 2), (5120, 4)])
@pytest.mark.parametrize("out_dtype,w_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                               (torch.bfloat16, torch.float32)])
def test_rmsnorm_and_residual(h, rows, out_dtype, w_dtype):
    from reinfer_b200 import ops
    eps = 3e-5
    x, w = rnd(rows, h, scale=3.0, seed=1), (1 + rnd(h, scale=0.1, seed=2)).to(w_dtype)

    def ref(xx):
        return xx * torch.rsqrt((xx * xx).mean(-1, keepdim=True) + eps) * w.float()
    out = torch.empty(rows, h, dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x, None, w, out, eps)
    tol = 1e-2 if out_dtype == torch.bfloat16 else 2e-6
    assert (out.float() - ref(x)).abs().max().item() <= tol * ref(x).abs().max().item()
    delta = rnd(rows, h, dtype=out_dtype, seed=3)
    x2 = x.clone()
    ops.add_rmsnorm(x2, delta, w, out, eps)
    assert torch.allclose(x2, x + delta.float(), atol=1e-6)
    assert (out.float() - ref(x + delta.float())).abs().max().item() <= tol * ref(x).abs().max().item()
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, h, dtype=out_dtype, device=DEV)
    ops.add_rmsnorm(x, None, w, out2, eps, row_idx=idx)
    assert (out2.float() - ref(x)[[rows - 1, 0]]).abs().max().item() <= tol * ref(x).abs().max().item()
    x3 = x.clone()
    ops.residual_add(x3, delta)
    assert torch.allclose(x3, x + delta.float(), atol=1e-6)


@pytest.mark.parametrize("h,rows", [(64, 65), (1000, 70), (4096, 100), (5120, 65), (8192, 66), (12288, 65)])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_delta", [0, 1, 3])
def test_rmsnorm_many_rows(h, rows, w_dtype, n_delta):
    """A prompt portion's rows of 16-bit activations (the vectorised kernel up to 8192 columns, the scalar one beyond)."""
    from reinfer_b200 import ops
    eps = 1e-6
    base, w = rnd(rows, h, scale=3.0, seed=1), (1 + rnd(h, scale=0.1, seed=2)).to(w_dtype)
    delta = rnd(n_delta, rows, h, seed=3) if n_delta else None
    x = base.clone()
    out = torch.empty(rows, h, dtype=torch.bfloat16, device=DEV)
    ops.add_rmsnorm(x, delta if n_delta != 1 else delta[0], w, out, eps)
    want_x = base.clone()
    for k in range(n_delta):
        want_x += delta[k]
    assert torch.equal(x, want_x)
    want = want_x * torch.rsqrt((want_x * want_x).mean(-1, keepdim=True) + eps) * w.float()
    assert (out.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item()


def test_embedding_gather():
    from reinfer_b200 import ops
    for dtype in (torch.float32, torch.bfloat16):
        table = rnd(77, 50, dtype=dtype)
        ids = torch.tensor([0, 76, 5, 5, 31], dtype=torch.int32, device=DEV)
        out = torch.empty(5, 50, dtype=torch.float32, device=DEV)
        ops.embed_gather(table, ids, out)
        assert torch.equal(out, table[ids.long()].float())


def _rope_ref(x, pos, theta, rot):
    half = rot // 2
    p = torch.arange(half, dtype=torch.float64)
    inv = (torch.tensor(theta, dtype=torch.float64) ** (-(2 * p) / rot)).to(torch.float32).double().to(x.device)
    ang = pos.double()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half].double(), x[..., half:rot].double()
    return torch.cat([a * c - b * s, a * s + b * c, x[..., rot:].double()], dim=-1)


@pytest.mark.parametrize("QH,KH,d,rot,page", [(4, 2, 16, 16, 16), (6, 2, 32, 32, 8), (3, 1, 80, 48, 4), (8, 8, 128, 128, 16),
                                              (5, 5, 256, 256, 32), (4, 2, 64, 64, 16), (3, 3, 192, 192, 8), (2, 1, 384, 384, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("norm", [True, False])
def test_qknorm_rope_append(QH, KH, d, rot, page, dtype, norm):
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import RotaryEncoding
    T, eps, theta, pages = 9, 1e-5, 5e4, 7
    qkv = rnd(T, (QH + 2 * KH) * d, dtype=dtype, seed=4)
    qw = (1 + rnd(d, scale=0.1, seed=5)).to(dtype) if norm else None
    kw = (1 + rnd(d, scale=0.1, seed=6)).to(dtype) if norm else None
    pos = torch.tensor([0, 1, 2, 40, 41, 1000, 7, 8, 9], dtype=torch.int32, device=DEV)
    slots = torch.tensor([3, 0, page * pages - 1, 2 * page + 2, -1, page, page + 2, page + 1, 2 * page - 1], dtype=torch.int32, device=DEV)
    cache = torch.full((pages, 2, KH, page, d), 7.0, dtype=dtype, device=DEV)
    q_out = torch.empty(T, QH, d, dtype=dtype, device=DEV)
    rope = RotaryEncoding(d, theta, rot)
    rope.prepare(DEV)
    ops.qknorm_rope_append(qkv, qw, kw, rope.inv_freq, pos, slots, q_out, cache, QH, KH, d, rot, page, eps)
    x = qkv.float().view(T, QH + 2 * KH, d)
    q, k, v = x[:, :QH], x[:, QH:QH + KH], x[:, QH + KH:]
    if norm:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * qw.float()
        k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * kw.float()
    q, k = _rope_ref(q, pos, theta, rot), _rope_ref(k, pos, theta, rot)
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    assert (q_out.double() - q).abs().max().item() <= tol * q.abs().max().item()
    flat = cache.permute(0, 3, 1, 2, 4).reshape(pages * page, 2, KH, d)     # [slot, kv, head, d]
    untouched = torch.ones(pages * page, dtype=torch.bool)
    for t in range(T):
        sl = int(slots[t])
        if sl < 0:
            continue
        untouched[sl] = False
        assert (flat[sl, 0].double() - k[t]).abs().max().item() <= tol * k.abs().max().item()
        assert torch.equal(flat[sl, 1], qkv.view(T, QH + 2 * KH, d)[t, QH + KH:])
    assert bool((flat[untouched.to(DEV)] == 7.0).all())                      # nothing else was written
    if dtype == torch.bfloat16 and rot == d and d % 128 == 0:
        # the same with the step's table of cosines and sines: identical bits
        cache2 = torch.full_like(cache, 7.0)
        q2 = torch.empty_like(q_out)
        ops.qknorm_rope_append(qkv, qw, kw, rope.inv_freq, pos, slots, q2, cache2, QH, KH, d, rot, page, eps,
                               cs_table=ops.rope_table(pos, rope.inv_freq))
        assert torch.equal(q2, q_out) and torch.equal(cache2, cache)


@pytest.mark.parametrize("T,QH,KH,K,page,wdt", [(300, 4, 2, 264, 16, torch.float32), (700, 5, 1, 520, 64, torch.bfloat16),
                                                (1027, 32, 8, 1024, 16, torch.bfloat16), (513, 3, 3, 72, 8, torch.float32)])
@pytest.mark.parametrize("scaled", [False, True])
def test_qkv_projection_with_the_heads_work_in_its_epilogue(T, QH, KH, K, page, wdt, scaled):
    """The q/k/v projection of a prompt portion that normalises, rotates and stores its heads itself, against the
    product followed by the kernel that does the same on the rounded projection: the same queries, and the same
    keys and values in the same slots (slots in a random order, some tokens not stored, ragged last token tile,
    an odd number of heads so that the last tile holds one head only); nothing else in the cache is touched."""
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import RotaryEncoding
    d, eps, theta = 128, 1e-6, 1e6
    N = (QH + 2 * KH) * d
    x = rnd(T, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.06, seed=2)
    qw = (1 + rnd(d, scale=0.1, seed=5)).to(wdt)
    kw = (1 + rnd(d, scale=0.1, seed=6)).to(wdt)
    pos = (torch.arange(T, dtype=torch.int32) * 7 % 3000).to(DEV)
    pages = -(-T // page) + 3
    perm = torch.randperm(pages * page, generator=torch.Generator().manual_seed(1))[:T].to(torch.int32)
    perm[5] = -1
    perm[T - 1] = -1
    slots = perm.to(DEV)
    rope = RotaryEncoding(d, theta, d)
    rope.prepare(DEV)
    cs = ops.rope_table(pos, rope.inv_freq)
    scale = ((rnd(T, 5, seed=9).abs() * K).contiguous(), K, eps) if scaled else None      # rows that lack their factor
    # the two-kernel way
    qkv = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16(x, w, qkv, row_scale=scale)
    cache_ref = torch.full((pages, 2, KH, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_ref = torch.empty(T, QH, d, dtype=torch.bfloat16, device=DEV)
    ops.qknorm_rope_append(qkv, qw, kw, rope.inv_freq, pos, slots, q_ref, cache_ref, QH, KH, d, d, page, eps, cs_table=cs)
    # the one-kernel way
    cache = torch.full((pages, 2, KH, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.full((T, QH, d), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.gemm_qkv_heads(x, w, q_out, cache, slots, cs, qw, kw, QH, KH, page, eps, row_scale=scale)
    assert ops.kernel_error() == 0
    assert not torch.isnan(q_out.float()).any()
    # the same arithmetic on the same rounded projection, but for the order of the sum of squares: a unit of bfloat16
    qs = q_ref.float().abs().max().item()
    assert (q_out.float() - q_ref.float()).abs().max().item() <= 8e-3 * qs
    assert (q_out != q_ref).float().mean().item() < 0.02
    ks = cache_ref[:, 0].float().abs().max().item()
    assert (cache[:, 0].float() - cache_ref[:, 0].float()).abs().max().item() <= 8e-3 * ks
    assert torch.equal(cache[:, 1], cache_ref[:, 1])                        # values are copied as they are
    assert not ops.gemm_qkv_heads(x[:200], w, q_out[:200], cache, slots, cs[:200], qw, kw, QH, KH, page, eps)   # one token tile: the other way


@pytest.mark.parametrize("T,QH,KH,K,page", [(1, 32, 8, 4096, 16), (8, 32, 8, 4096, 16), (7, 3, 1, 520, 8), (33, 8, 2, 1024, 64), (64, 5, 5, 256, 16)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16, None])
@pytest.mark.parametrize("scaled", [False, True])
def test_decode_qkv_projection_whose_cluster_does_the_heads_work(T, QH, KH, K, page, wdt, scaled):
    """The q/k/v projection of a decode step's rows whose cluster normalises, rotates and stores the heads, against
    the product followed by the kernel that does the same on the stored projection: the same queries, keys and values
    in the same slots (with and without norm weights, rows with and without their factor, one token that is not
    stored, no slots at all); nothing else in the cache is touched."""
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import RotaryEncoding
    d, eps, theta = 128, 1e-6, 1e6
    N = (QH + 2 * KH) * d
    x = rnd(T, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.06, seed=2)
    qw = (1 + rnd(d, scale=0.1, seed=5)).to(wdt) if wdt is not None else None
    kw = (1 + rnd(d, scale=0.1, seed=6)).to(wdt) if wdt is not None else None
    pos = (torch.arange(T, dtype=torch.int32) * 977 % 30000).to(DEV)
    pages = -(-T // page) + 3
    perm = torch.randperm(pages * page, generator=torch.Generator().manual_seed(1))[:T].to(torch.int32)
    if T > 2:
        perm[1] = -1
    slots = perm.to(DEV)
    rope = RotaryEncoding(d, theta, d)
    rope.prepare(DEV)
    scale = None
    if scaled:
        sumsq = (rnd(T, 3, seed=9).abs() * K).contiguous()
        scale = (sumsq, K, eps)
    for use_slots in (slots, None):
        qkv = torch.empty(T, N, dtype=torch.bfloat16, device=DEV)
        ops.gemm_bf16(x, w, qkv, row_scale=scale)
        cache_ref = torch.full((pages, 2, KH, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
        q_ref = torch.empty(T, QH, d, dtype=torch.bfloat16, device=DEV)
        ops.qknorm_rope_append(qkv, qw, kw, rope.inv_freq, pos, use_slots, q_ref, cache_ref, QH, KH, d, d, page, eps)
        cache = torch.full((pages, 2, KH, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
        q_out = torch.full((T, QH, d), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert ops.gemm_qkv_heads_stream(x, w, q_out, cache, use_slots, pos, rope.inv_freq, qw, kw, QH, KH, page, eps, row_scale=scale)
        assert ops.kernel_error() == 0
        assert not torch.isnan(q_out.float()).any()
        qs = q_ref.float().abs().max().item()
        assert (q_out.float() - q_ref.float()).abs().max().item() <= 8e-3 * qs
        assert (q_out != q_ref).float().mean().item() < 0.02
        ks = cache_ref[:, 0].float().abs().max().item()
        assert (cache[:, 0].float() - cache_ref[:, 0].float()).abs().max().item() <= 8e-3 * ks
        # values are the rounded sums as they are; the two ways may split K differently, so a sum may round the other way
        vs = cache_ref[:, 1].float().abs().max().item()
        assert (cache[:, 1].float() - cache_ref[:, 1].float()).abs().max().item() <= 8e-3 * vs
        assert (cache[:, 1] != cache_ref[:, 1]).float().mean().item() < 0.02
        untouched = cache_ref == 7.0
        assert torch.equal(cache[untouched], cache_ref[untouched])
    assert not ops.gemm_qkv_heads_stream(x.repeat(70, 1)[:70], w, torch.empty(70, QH, d, dtype=torch.bfloat16, device=DEV), cache, None,
                                         pos.repeat(70)[:70].contiguous(), rope.inv_freq, qw, kw, QH, KH, page, eps)   # over the streaming size: the other way


@pytest.mark.parametrize("QH,KH,d,page", [(8, 8, 128, 16), (32, 8, 128, 64), (5, 5, 256, 32), (12, 3, 64, 16), (9, 1, 128, 8), (6, 2, 128, 16)])
@pytest.mark.parametrize("norm", [True, False])
@pytest.mark.parametrize("table", [True, False])
def test_qknorm_rope_append_many_tokens(QH, KH, d, page, norm, table):
    """A prompt portion (more than 64 tokens; heads of 128 go through the kernel that takes a token's heads in
    groups) against the plain statement, with slots in a random order and one token that is not stored."""
    from reinfer_b200 import ops
    from reinfer_b200.parts.rope import RotaryEncoding
    T, eps, theta = 150, 1e-6, 1e6
    pages = -(-T // page) + 2
    qkv = rnd(T, (QH + 2 * KH) * d, dtype=torch.bfloat16, seed=4)
    qw = (1 + rnd(d, scale=0.1, seed=5)) if norm else None
    kw = (1 + rnd(d, scale=0.1, seed=6)) if norm else None
    pos = (torch.arange(T, dtype=torch.int32) * 7 % 3000).to(DEV)
    perm = torch.randperm(pages * page, generator=torch.Generator().manual_seed(1))[:T].to(torch.int32)
    perm[5] = -1
    slots = perm.to(DEV)
    rope = RotaryEncoding(d, theta, d)
    rope.prepare(DEV)
    cs = ops.rope_table(pos, rope.inv_freq) if table else None
    cache = torch.full((pages, 2, KH, page, d), 7.0, dtype=torch.bfloat16, device=DEV)
    q_out = torch.empty(T, QH, d, dtype=torch.bfloat16, device=DEV)
    ops.qknorm_rope_append(qkv, qw, kw, rope.inv_freq, pos, slots, q_out, cache, QH, KH, d, d, page, eps, cs_table=cs)
    x = qkv.float().view(T, QH + 2 * KH, d)
    q, k = x[:, :QH], x[:, QH:QH + KH]
    if norm:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * qw
        k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * kw
    q, k = _rope_ref(q, pos, theta, d), _rope_ref(k, pos, theta, d)
    assert (q_out.double() - q).abs().max().item() <= 2e-2 * q.abs().max().item()
    flat = cache.permute(0, 3, 1, 2, 4).reshape(pages * page, 2, KH, d)     # [slot, kv, head, d]
    stored = slots >= 0
    sl = slots[stored].long()
    assert (flat[sl, 0].double() - k[stored]).abs().max().item() <= 2e-2 * k.abs().max().item()
    assert torch.equal(flat[sl, 1], qkv.view(T, QH + 2 * KH, d)[stored][:, QH + KH:])
    untouched = torch.ones(pages * page, dtype=torch.bool, device=DEV)
    untouched[sl] = False
    assert bool((flat[untouched] == 7.0).all())                              # nothing else was written


def test_kv_append_and_k_out_path():
    from reinfer_b200 import ops
    T, QH, KH, d, page = 5, 4, 2, 32, 8
    qkv = rnd(T, (QH + 2 * KH) * d, dtype=torch.bfloat16)
    q_out = torch.empty(T, QH, d, dtype=torch.bfloat16, device=DEV)
    k_out = torch.empty(T, KH, d, dtype=torch.bfloat16, device=DEV)
    ops.qknorm_rope_append(qkv, None, None, None, None, None, q_out, None, QH, KH, d, 0, page, 1e-6, k_out=k_out)
    assert torch.equal(q_out.view(T, -1), qkv[:, :QH * d]) and torch.equal(k_out.view(T, -1), qkv[:, QH * d:(QH + KH) * d])
    cache = torch.zeros(3, 2, KH, page, d, dtype=torch.bfloat16, device=DEV)
    slots = torch.tensor([0, 9, 23, -1, 8], dtype=torch.int32, device=DEV)
    ops.kv_append(k_out.view(T, KH * d), qkv[:, (QH + KH) * d:], slots, cache, KH, d, page)
    flat = cache.permute(0, 3, 1, 2, 4).reshape(3 * page, 2, KH, d)
    for t, sl in enumerate(slots.tolist()):
        if sl >= 0:
            assert torch.equal(flat[sl, 0], k_out[t]) and torch.equal(flat[sl, 1].reshape(-1), qkv[t, (QH + KH) * d:])
    assert flat.abs().sum(dim=(1, 2, 3)).ne(0).sum().item() == 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    from reinfer_b200 import ops
    gu = rnd(7, 2 * 150, dtype=dtype, scale=3.0)
    out = torch.empty(7, 150, dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    g, u = gu[:, :150].float(), gu[:, 150:].float()
    ref = g / (1 + torch.exp(-g)) * u
    assert (out.float() - ref).abs().max().item() <= (1e-2 if dtype == torch.bfloat16 else 1e-6) * ref.abs().max().item()


def paged_setup(lens, q_lens, QH, KH, d, page, dtype, seed=0, poison=True):
    """Random requests in a shuffled, sparse pool; unwritten slots hold NaN."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lens) + 5
    perm = torch.randperm(n_pages, generator=g).tolist()
    cache = torch.full((n_pages, 2, KH, page, d), float("nan") if poison else 0.0, dtype=dtype)
    max_pages = max(-(-n // page) for n in lens) + 1
    bt = torch.full((len(lens), max_pages), -1, dtype=torch.int32)
    ks, vs = [], []
    for r, n in enumerate(lens):
        k, v = torch.randn(n, KH, d, generator=g).to(dtype), torch.randn(n, KH, d, generator=g).to(dtype)
        ks.append(k); vs.append(v)
        for i in range(-(-n // page)):
            pg = perm.pop()
            bt[r, i] = pg
            m = min(page, n - i * page)
            cache[pg, 0, :, :m] = k[i * page:i * page + m].transpose(0, 1)
            cache[pg, 1, :, :m] = v[i * page:i * page + m].transpose(0, 1)
    tok_row, positions = [], []
    for r, (n, ql) in enumerate(zip(lens, q_lens)):
        tok_row += [r] * ql
        positions += list(range(n - ql, n))
    T = len(tok_row)
    q = torch.randn(T, QH, d, generator=g).to(dtype)
    return dict(q=q.to(DEV), cache=cache.to(DEV), bt=bt.to(DEV), tok_row=torch.tensor(tok_row, dtype=torch.int32, device=DEV),
                positions=torch.tensor(positions, dtype=torch.int32, device=DEV), ks=ks, vs=vs, rows=tok_row, pos=positions)


def attention_truth(s, QH, KH, window, scale):
    out = torch.zeros(s["q"].shape, dtype=torch.float64)
    q = s["q"].double().cpu()
    for t, (r, p) in enumerate(zip(s["rows"], s["pos"])):
        lo = max(0, p - window + 1) if window > 0 else 0
        k, v = s["ks"][r][lo:p + 1].double(), s["vs"][r][lo:p + 1].double()
        for h in range(QH):
            kh = h // (QH // KH)
            pr = torch.softmax((k[:, kh] @ q[t, h]) * scale, 0)
            out[t, h] = pr @ v[:, kh]
    return out


@pytest.mark.parametrize("QH,KH,d,page", [(4, 2, 16, 16), (6, 2, 32, 8), (14, 2, 64, 4), (5, 5, 80, 32), (8, 1, 128, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 13])
def test_paged_attention_plain(QH, KH, d, page, dtype, window):
    from reinfer_b200 import ops
    lens, q_lens = [1, 37, 64, 131], [1, 5, 1, 131]
    s = paged_setup(lens, q_lens, QH, KH, d, page, dtype)
    out = torch.empty_like(s["q"])
    scale = 0.7 / math.sqrt(d)
    ops.paged_attention_ref(s["q"], s["cache"], s["bt"], s["tok_row"], s["positions"], out, QH, KH, d, page, window, scale)
    ref = attention_truth(s, QH, KH, window, scale)
    assert not torch.isnan(out).any()
    tol = 1.5e-2 if dtype == torch.bfloat16 else 1e-5
    assert (out.double().cpu() - ref).abs().max().item() <= tol * ref.abs().max().item()


def test_attention_finds_one_far_key():
    """One key among hundreds gets a score that stands out; the output must be its value."""
    from reinfer_b200 import ops
    QH, KH, d, page = 4, 2, 32, 8
    s = paged_setup([700], [1], QH, KH, d, page, torch.float32, seed=3)
    far = 5
    pg, off = int(s["bt"][0, far // page]), far % page
    s["q"][0, :, :] = 0.0
    s["q"][0, :, 0] = 50.0
    s["cache"][pg, 0, :, off, 0] = 50.0
    out = torch.empty_like(s["q"])
    ops.paged_attention_ref(s["q"], s["cache"], s["bt"], s["tok_row"], s["positions"], out, QH, KH, d, page, 0, 1.0)
    want = s["cache"][pg, 1, :, off]                                   # [KH, d]
    for h in range(QH):
        assert torch.allclose(out[0, h], want[h // 2], atol=1e-4)
    # with a window that ends before the far key it must NOT be seen
    ops.paged_attention_ref(s["q"], s["cache"], s["bt"], s["tok_row"], s["positions"], out, QH, KH, d, page, 699 - far, 1.0)
    assert not torch.allclose(out[0, 0], want[0], atol=1e-2)
    ops.paged_attention_ref(s["q"], s["cache"], s["bt"], s["tok_row"], s["positions"], out, QH, KH, d, page, 700 - far, 1.0)
    assert torch.allclose(out[0, 0], want[0], atol=1e-4)


@pytest.mark.parametrize("QH,KH,d,page", [(4, 2, 16, 16), (6, 2, 32, 8), (14, 2, 64, 4), (5, 5, 80, 32), (8, 1, 128, 16),
                                          (32, 8, 128, 16), (32, 1, 64, 16), (3, 1, 256, 64), (6, 3, 24, 8), (8, 2, 128, 128),
                                          (4, 4, 192, 16), (6, 1, 128, 64), (7, 7, 128, 8), (32, 2, 128, 32)])
@pytest.mark.parametrize("window", [0, 37])
def test_flash_prefill_and_decode_against_plain(QH, KH, d, page, window):
    """The tensor-core kernels on a batch that mixes decode entries and prompt portions which
    continue from cached pages; shuffled pages, partial last pages, NaN in every unwritten slot."""
    from reinfer_b200 import ops
    lens = [1, 37, 64, 300, 5, 131, 1000]
    q_lens = [1, 1, 1, 1, 5, 70, 130]
    s = paged_setup(lens, q_lens, QH, KH, d, page, torch.bfloat16, seed=11)
    scale = 0.9 / math.sqrt(d)
    ref = attention_truth(s, QH, KH, window, scale)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    cu_q = torch.tensor(cu, dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    gc = ops.fa_group_chunk(QH // KH)
    kernels = [(ops.fa_decode, ops.fa_prefill)] + ([(ops.fa_decode_tma, ops.fa_prefill_tma)] if ops.tma_pages(page) else [])
    if d == 128 and ops.tma_pages(page):
        kernels.append((ops.fa_decode_tma, "tcgen05"))                      # scores and weighted sums in tensor memory
    for n_splits, (decode, prefill) in [(n, f) for n in (1, 3, 8) for f in kernels]:
        out = torch.full_like(s["q"], float("nan"))
        decode(s["q"], s["cache"], s["bt"], cu_q, kv_len, out, 0, 4, 0, n_splits, QH, KH, d, page, window, scale)
        assert ops.kernel_error() == 0
        tpt = 64 // gc
        n_tiles = sum(-(-n // tpt) for n in q_lens[4:])
        if prefill == "tcgen05":
            ops.fa_prefill_tc(s["q"], s["cache"], s["bt"], cu_q, kv_len, out, 4, 3, q_lens[4:], QH, KH, d, page, window, scale)
            assert ops.kernel_error() == 0
        else:
            prefill(s["q"], s["cache"], s["bt"], cu_q, kv_len, out, 4, 3, n_tiles, QH, KH, d, page, window, scale)
        assert not torch.isnan(out.float()).any()
        err = (out.double().cpu() - ref).abs().max().item() / ref.abs().max().item()
        assert err <= 1.5e-2, f"splits {n_splits}: error {err:.3e}"


@pytest.mark.parametrize("QH,KH,d,page", [(32, 8, 128, 64), (8, 1, 128, 16), (14, 2, 64, 8), (3, 1, 256, 64), (5, 5, 80, 32)])
@pytest.mark.parametrize("n_splits", [2, 3, 4, 7, 8, 11, 16])
def test_flash_decode_merge_inside_the_cluster_and_by_kernel_agree(QH, KH, d, page, n_splits, monkeypatch):
    """Up to 16 splits merge inside a cluster of CTAs (more than 8: where the device can place such clusters and
    all of them at once), or go through scratch and the merge kernel: both add the parts in ascending order with
    the same formulas, so the results have the same bits (requests shorter than the splits, and one of a single
    key, included)."""
    from reinfer_b200 import ops
    lens = [1, 37, 64, 300, 2000, 131]
    s = paged_setup(lens, [1] * len(lens), QH, KH, d, page, torch.bfloat16, seed=5)
    cu_q = torch.arange(len(lens) + 1, dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    outs = []
    for in_kernel in (True, False):
        monkeypatch.setattr(ops, "ATTN_CLUSTER_MERGE", in_kernel)
        out = torch.full_like(s["q"], float("nan"))
        ops.fa_decode_tma(s["q"], s["cache"], s["bt"], cu_q, kv_len, out, 0, len(lens), 0, n_splits, QH, KH, d, page, 0, 0.9 / math.sqrt(d))
        assert ops.kernel_error() == 0
        outs.append(out)
    assert not torch.isnan(outs[0].float()).any()
    assert torch.equal(outs[0], outs[1])
    ref = attention_truth(s, QH, KH, 0, 0.9 / math.sqrt(d))
    assert (outs[0].double().cpu() - ref).abs().max().item() <= 1.5e-2 * ref.abs().max().item()


@pytest.mark.parametrize("direction", ["rising", "falling", "spikes"])
def test_flash_prefill_tcgen05_when_the_maximum_keeps_moving(direction):
    """The tcgen05 prefill kernel keeps O in tensor memory, scaled to a maximum that follows the true one only in
    large steps.  Scores that rise from tile to tile (every tile brings a new maximum far above the last), fall,
    or spike now and then make it rescale often, seldom, or in the middle of a row's keys - always the plain result."""
    from reinfer_b200 import ops
    QH, KH, d, page = 8, 2, 128, 64
    T = 700
    s = paged_setup([T], [T], QH, KH, d, page, torch.bfloat16, seed=21)
    # keys along one direction with a strength that depends on the position; queries all look that way
    gen = torch.Generator().manual_seed(5)
    u = torch.zeros(d); u[3] = 1.0
    pos = torch.arange(T, dtype=torch.float32)
    strength = {"rising": 0.12 * pos, "falling": 0.12 * (T - pos), "spikes": torch.where(pos.long() % 97 == 5, 60.0, 0.0)}[direction]
    k_new = (torch.randn(T, KH, d, generator=gen) * 0.3 + strength[:, None, None] * u).to(torch.bfloat16)
    s["ks"][0] = k_new
    for i in range(-(-T // page)):
        m = min(page, T - i * page)
        s["cache"][int(s["bt"][0, i]), 0, :, :m] = k_new[i * page:i * page + m].transpose(0, 1).to(DEV)
    q_new = (torch.randn(T, QH, d, generator=gen) * 0.3 + 4.0 * u).to(torch.bfloat16)
    s["q"] = q_new.to(DEV)
    scale = 1.0 / math.sqrt(d)
    ref = attention_truth(s, QH, KH, 0, scale)
    cu_q = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([T], dtype=torch.int32, device=DEV)
    out = torch.full_like(s["q"], float("nan"))
    ops.fa_prefill_tc(s["q"], s["cache"], s["bt"], cu_q, kv_len, out, 0, 1, [T], QH, KH, d, page, 0, scale)
    assert ops.kernel_error() == 0
    assert not torch.isnan(out.float()).any()
    err = (out.double().cpu() - ref).abs().max().item() / ref.abs().max().item()
    assert err <= 1.5e-2, f"{direction}: error {err:.3e}"


def test_flash_decode_finds_one_far_key_across_splits():
    from reinfer_b200 import ops
    QH, KH, d, page = 8, 2, 64, 16
    s = paged_setup([3000], [1], QH, KH, d, page, torch.bfloat16, seed=5)
    cu_q = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([3000], dtype=torch.int32, device=DEV)
    for far in (0, 63, 64, 1537, 2999):
        q, cache = s["q"].clone(), s["cache"].clone()
        pg, off = int(s["bt"][0, far // page]), far % page
        q[0] = 0.0; q[0, :, 3] = 40.0
        cache[pg, 0, :, off, 3] = 40.0
        for n_splits, decode in [(n, f) for n in (1, 5, 47) for f in (ops.fa_decode, ops.fa_decode_tma)]:
            out = torch.empty_like(q)
            decode(q, cache, s["bt"], cu_q, kv_len, out, 0, 1, 0, n_splits, QH, KH, d, page, 0, 1.0)
            want = cache[pg, 1, :, off].float()
            for h in range(QH):
                assert torch.allclose(out[0, h].float(), want[h // 4], atol=2e-2), (far, n_splits, h)
