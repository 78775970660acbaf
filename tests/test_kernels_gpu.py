"""Each kernel alone against a plain fp32 statement of the same operation, at sizes other
than the engine's."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)


@pytest.fixture(scope="module")
def ops():
    from pyre_b200.kernels import ops
    return ops


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [40, 101, 3584])
def test_embedding(ops, dtype, H):
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randn(300, H, device="cuda", generator=g).to(dtype)
    ids = torch.tensor([0, 299, 5, 5, 17], dtype=torch.int32, device="cuda")
    x = ops.embedding(table, ids)
    assert x.dtype == torch.float32
    assert torch.equal(x, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,eps", [(40, 1e-5), (101, 1e-6), (3584, 1e-6), (5120, 3e-6), (9000, 1e-6), (2051, 1e-5)])
def test_add_rmsnorm(ops, dtype, H, eps):
    g = torch.Generator(device="cuda").manual_seed(1)
    T = 7
    x = torch.randn(T, H, device="cuda", generator=g) * 3
    delta = torch.randn(T, H, device="cuda", generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(H, device="cuda", generator=g)
    x0 = x.clone()
    v = x0 + delta.float()
    want = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)) * w
    out = ops.add_rmsnorm(x, delta, w, eps, dtype)
    torch.testing.assert_close(x, v, rtol=0, atol=0)          # the sum went back to the stream
    torch.testing.assert_close(out.float(), want, **tol(dtype))
    # without delta, x untouched
    x1 = x0.clone()
    out = ops.add_rmsnorm(x1, None, w, eps, dtype)
    assert torch.equal(x1, x0)
    want0 = (x0 * torch.rsqrt(x0.pow(2).mean(-1, keepdim=True) + eps)) * w
    torch.testing.assert_close(out.float(), want0, **tol(dtype))
    # gathered rows: x untouched, delta still counted
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device="cuda")
    x2 = x0.clone()
    out = ops.add_rmsnorm(x2, delta, w, eps, dtype, rows=rows)
    assert torch.equal(x2, x0)
    torch.testing.assert_close(out.float(), want[rows.long()], **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 40), (7, 101), (300, 3584)])
def test_add_residual(ops, dtype, shape):
    """The plain residual sum for a branch that no norm follows: fp32 stream += delta, summed in fp32."""
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(*shape, device="cuda", generator=g)
    delta = torch.randn(*shape, device="cuda", generator=g).to(dtype)
    want = x + delta.float()
    assert ops.add_residual(x, delta) is x
    assert torch.equal(x, want)                       # one fp32 addition per element: exact


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I", [176, 99, 1000])
def test_silu_mul(ops, dtype, I):
    g = torch.Generator(device="cuda").manual_seed(2)
    gu = (torch.randn(5, 2 * I, device="cuda", generator=g) * 4).to(dtype)
    want = torch.nn.functional.silu(gu[:, :I].float()) * gu[:, I:].float()
    torch.testing.assert_close(ops.silu_mul(gu).float(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I,block", [(176, 8), (384, 64), (1000, 40)])
def test_silu_mul_interleaved(ops, dtype, I, block):
    """Gates and ups alternating in blocks: the same result as the stacked layout."""
    g = torch.Generator(device="cuda").manual_seed(2)
    gu = (torch.randn(5, 2 * I, device="cuda", generator=g) * 4).to(dtype)
    mixed = torch.stack([gu[:, :I].reshape(5, I // block, block), gu[:, I:].reshape(5, I // block, block)], dim=2).reshape(5, 2 * I).contiguous()
    assert torch.equal(ops.silu_mul(mixed, block=block), ops.silu_mul(gu))
    with pytest.raises(ops.UnsupportedSize):
        ops.silu_mul(gu, block=12)


@pytest.mark.parametrize("M,I,K", [(300, 384, 136), (129, 128, 64), (2048, 1024, 512), (8, 256, 200), (100, 640, 96), (1, 18944, 256),
                                   (8, 18944, 520), (37, 1024, 64), (128, 2048, 192), (300, 192, 64)])
def test_gated_product(ops, M, I, K):
    """silu(x gate^T) * (x up^T) with the activation in the product's epilogue (tokens on the row
    side) or after it (few tokens): both equal the separate kernels on the stacked weight bit for
    bit, and agree with an fp32 evaluation."""
    g = torch.Generator(device="cuda").manual_seed(M + I)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    wg = (torch.randn(I, K, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    wu = (torch.randn(I, K, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    mixed = ops.interleave_gate_up(wg, wu)
    got = ops.gated_linear(x, mixed, True)
    ops.check_device_errors()
    stacked = torch.cat([wg, wu]).contiguous()
    plan = ops.tc_gemm_plan(M, 2 * I, K)
    # the same tiles and the same order of the sums: force the plan of the interleaved call on the stacked weight
    separate = ops.silu_mul(ops.gemm_tc(x, stacked, torch.bfloat16, plan=(plan[0], plan[1], 1)))
    if plan[2] == 1:
        assert torch.equal(got, separate)
    if M > 128 and (2 * I) % 256 == 0:      # one CTA per tile and a pair of CTAs per 256-row tile: the same bits
        assert torch.equal(ops.gemm_tc(x, mixed, gated=True, pair=False), ops.gemm_tc(x, mixed, gated=True, pair=True))
    gate = (x.float() @ wg.float().t()).to(torch.bfloat16).float()
    up = (x.float() @ wu.float().t()).to(torch.bfloat16).float()
    want = torch.nn.functional.silu(gate) * up
    scale = float(want.abs().max())
    assert float((got.float() - want).abs().max()) <= 2.0 ** -6 * scale
    assert float((separate.float() - want).abs().max()) <= 2.0 ** -6 * scale
    assert got.shape == (M, I)


@pytest.mark.parametrize("M,N,K", [(1, 130, 70), (5, 64, 64), (33, 257, 100), (200, 300, 131), (64, 1000, 96)])
def test_sgemm_is_true_fp32(ops, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g)
    bias = torch.randn(N, device="cuda", generator=g)
    want = (a.double() @ w.double().t()).float()
    got = ops.sgemm_nt(a, w)
    # fp32 products and sums: error of a K-term sum, far below what TF32 (10-bit mantissa) gives
    assert (got - want).abs().max().item() <= 2e-6 * K * 4
    torch.testing.assert_close(ops.sgemm_nt(a, w, bias), got + bias, rtol=1e-6, atol=1e-6)
    # a row's result does not depend on how many rows are in the product
    if M > 1:
        assert torch.equal(ops.sgemm_nt(a[:1].contiguous(), w), got[:1])


def test_sgemm_sums_in_two_levels(ops):
    """Positive operands and a long K are the worst case of a single chain of additions (its
    relative error passes 3e-6 at K = 8192); runs of 32 summed on their own stay under 1e-6."""
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.rand(40, 8192, device="cuda", generator=g)
    w = torch.rand(96, 8192, device="cuda", generator=g)
    want = a.double() @ w.double().t()
    got = ops.sgemm_nt(a, w).double()
    assert ((got - want).abs() / want).max().item() <= 2e-6


@pytest.mark.parametrize("M,N,K", [(1, 4608, 3584), (8, 3584, 3584), (8, 3584, 18944), (8, 37888, 3584), (5, 130, 72),
                                   (16, 256, 64), (17, 1000, 96), (64, 777, 200), (100, 640, 1024), (128, 152064 // 8, 512),
                                   (129, 512, 256), (300, 1000, 96), (300, 777, 200), (2048, 4608, 3584), (1000, 3584, 1888)])
def test_gemm_tc_matches_fp32_product(ops, M, N, K):
    """The tcgen05 kernel against an fp32 product of the same bf16 operands: fp32
    accumulation, so only the order of the sum and the final rounding differ."""
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    want = a.float() @ w.float().t()
    got32 = ops.gemm_tc(a, w, torch.float32)
    ops.check_device_errors()
    scale = float(want.abs().max())
    assert float((got32 - want).abs().max()) <= 2e-5 * scale * max(1.0, (K / 64) ** 0.5)
    got16 = ops.gemm_tc(a, w, torch.bfloat16)
    assert float((got16.float() - want).abs().max()) <= 2.0 ** -8 * scale
    # every plan gives the same product: both orientations, every tile width, split K
    for plan in [(True, 16, 1), (True, 32, 3), (True, 64, 2), (True, 128, 1), (True, 256, 4), (False, 128, 1), (False, 256, 2),
                 (False, 160, 1), (False, 192, 2), (False, 208, 1), (False, 224, 1)]:
        if not plan[0] and N % 8:
            continue
        if plan[0] and M > 4 * plan[1]:
            continue
        other = ops.gemm_tc(a, w, torch.float32, plan=plan, pair=False)
        assert float((other - want).abs().max()) <= 2e-5 * scale * max(1.0, (K / 64) ** 0.5), f"plan {plan}"
        # two CTAs of a cluster on each 256-row tile: the same sums in the same order
        if not plan[0] and M > 128:
            paired = ops.gemm_tc(a, w, torch.float32, plan=plan, pair=True)
            assert torch.equal(paired, other), f"plan {plan} with CTA pairs"
    ops.check_device_errors()
    # strided activations (a slice of a wider buffer)
    if K % 16 == 0:
        wide = torch.randn(M, 2 * K, device="cuda", generator=g).to(torch.bfloat16)
        part = wide[:, K:]
        got = ops.gemm_tc(part, w, torch.float32)
        assert float((got - part.float() @ w.float().t()).abs().max()) <= 2e-5 * scale * max(1.0, (K / 64) ** 0.5) * 2


@pytest.mark.parametrize("M", [1, 8, 64, 300])
def test_output_head_at_the_full_vocabulary(ops, M):
    """The product that gives the logits at the benchmark model's sizes (152,064 x 3,584): fp32 logits
    from the accumulator, for decode batches (weights on the MMA's rows, many CTAs in several rounds)
    and for a prompt portion (tokens on the rows, CTA pairs)."""
    V, K = 152064, 3584
    g = torch.Generator(device="cuda").manual_seed(M)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.empty(V, K, device="cuda", dtype=torch.bfloat16)
    for lo in range(0, V, 16384):      # drawn in pieces: an fp32 copy of the whole matrix is 2 GB
        w[lo:lo + 16384] = (torch.randn(min(16384, V - lo), K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    got = ops.linear(a, w, out_dtype=torch.float32)
    ops.check_device_errors()
    assert got.dtype == torch.float32 and got.shape == (M, V)
    worst, scale = 0.0, 0.0
    for lo in range(0, V, 16384):
        want = a.float() @ w[lo:lo + 16384].float().t()
        worst = max(worst, float((got[:, lo:lo + 16384] - want).abs().max()))
        scale = max(scale, float(want.abs().max()))
    assert worst <= 2e-5 * scale * (K / 64) ** 0.5, f"max error {worst:.3e} at scale {scale:.3f}"
    # the first and the last vocabulary entries come from the first and the last tile
    assert torch.isfinite(got[:, 0]).all() and torch.isfinite(got[:, -1]).all()


def test_sampling_at_the_full_vocabulary(ops):
    """Greedy and temperature sampling over 152,064 entries (the two-stage kernel, a last slice that is
    not full) against the plain sampler; ties across slices go to the lowest index."""
    from plain import qwen2_plain
    V = 152064
    g = torch.Generator(device="cuda").manual_seed(21)
    logits = torch.randn(8, V, device="cuda", generator=g) * 2
    logits[3, 152063] = 40.0                          # the very last entry
    logits[4, 70000] = logits[4, 151000] = 41.0       # a tie far apart
    want = [int(logits[r].argmax()) for r in range(8)]
    want[3], want[4] = 152063, 70000
    assert ops.sample(logits).tolist() == want
    temps = torch.tensor([0.7, 0.0, 1.0, 0.0, 1.9, 0.3, 1.0, 0.7], device="cuda")
    seeds = torch.tensor([1, 2, 3, 4, 5, 6, 3, 1], dtype=torch.int64, device="cuda")
    tix = torch.tensor([0, 1, 2, 3, 4, 5, 3, 0], dtype=torch.int32, device="cuda")
    got = ops.sample(logits, temps, seeds, tix).tolist()
    cpu = logits.cpu()
    assert got == [qwen2_plain.sample(cpu[r], float(temps[r]), int(seeds[r]), int(tix[r])) for r in range(8)]
    # a padded row stride (logits as a slice of a wider buffer), as a captured step hands them over
    wide = torch.zeros(8, V + 64, device="cuda")
    wide[:, :V] = logits
    assert ops.sample(wide[:, :V], temps, seeds, tix).tolist() == got


def plain_rope(x, pos, inv, rot):
    # x [T, n, hd]; half-split pairs over the first rot dims (pyre/model.py:41-63);
    # inv = theta^(-2j/rot) is computed once on the CPU and shared with the kernel under
    # test: at position 30000 one ulp of inv_freq already moves the angle by 3e-3
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :rot // 2], x[..., rot // 2:rot]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, x[..., rot:]], dim=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot,page,theta", [(4, 2, 16, 16, 16, 1e4), (3, 1, 32, 32, 8, 1e6),
                                                     (5, 5, 48, 32, 4, 5e4), (28, 4, 128, 128, 16, 1e6)])
@pytest.mark.parametrize("T", [13, 300])      # few tokens and many tokens take different kernels when the rotary covers the head
def test_qkv_rope_write(ops, dtype, nh, nkv, hd, rot, page, theta, T):
    g = torch.Generator(device="cuda").manual_seed(4)
    pages = -(-T // page) + 8
    width = (nh + 2 * nkv) * hd
    qkv = torch.randn(T, width, device="cuda", generator=g).to(dtype)
    bias = torch.randn(width, device="cuda", generator=g) * 0.5
    base = [0, 1, 2, 3, 40, 41, 1000, 7, 8, 9, 30000, 5, 6]
    pos = torch.tensor([base[t] if t < 13 else (t * 37) % 9001 for t in range(T)], dtype=torch.int32, device="cuda")
    slots = torch.randperm(pages * page, device="cuda", generator=g)[:T].to(torch.int32)
    slots[3] = -1  # this token stores nothing
    inv = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).cuda()
    cos, sin = ops.rope_table(pos, inv)
    ang = pos.float()[:, None] * inv[None, :]
    torch.testing.assert_close(cos, ang.cos(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(sin, ang.sin(), rtol=1e-5, atol=1e-6)
    cache = torch.full((pages, 2, nkv, page, hd), 7.0, device="cuda").to(dtype)
    q = ops.qkv_rope_write(qkv, bias, cos, sin, cache, slots, nh, nkv, hd, rot, page)

    full = qkv.float() + bias
    qw = plain_rope(full[:, :nh * hd].view(T, nh, hd), pos, inv, rot)
    kw = plain_rope(full[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), pos, inv, rot)
    vw = full[:, (nh + nkv) * hd:].view(T, nkv, hd)
    torch.testing.assert_close(q.float().view(T, nh, hd), qw, **tol(dtype))
    want_cache = torch.full((pages, 2, nkv, page, hd), 7.0, device="cuda")
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        want_cache[s // page, 0, :, s % page] = kw[t]
        want_cache[s // page, 1, :, s % page] = vw[t]
    torch.testing.assert_close(cache.float(), want_cache, **tol(dtype))


def plain_paged_attention(q, cache, table, seq_of_token, positions, nh, nkv, hd, scale, window):
    T = q.shape[0]
    page = cache.shape[3]
    out = torch.zeros(T, nh, hd, dtype=torch.float64, device=q.device)
    qf = q.double().view(T, nh, hd)
    for t in range(T):
        s, p = int(seq_of_token[t]), int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        idx = torch.arange(lo, p + 1, device=q.device)
        pages = table[s, idx // page].long()
        k = cache[pages, 0, :, idx % page].double()   # [n, nkv, hd]
        v = cache[pages, 1, :, idx % page].double()
        for h in range(nh):
            kvh = h // (nh // nkv)
            sc = (k[:, kvh] @ qf[t, h]) * scale
            pr = torch.softmax(sc, dim=0)
            out[t, h] = pr @ v[:, kvh]
    return out.view(T, nh * hd).float()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,page,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, 37),
                                                   (8, 2, 64, 32, None), (7, 1, 128, 16, 50), (2, 2, 256, 16, None)])
def test_paged_attention_generic(ops, dtype, nh, nkv, hd, page, window):
    g = torch.Generator(device="cuda").manual_seed(5)
    # three sequences: a decode token far into a long context, a prompt portion that
    # starts mid-page, and a short whole prompt
    ctx_lens = [301, 77, 9]
    new = [1, 20, 9]
    n_pages = sum(-(-c // page) for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(6)).tolist()
    W = max(-(-c // page) for c in ctx_lens)
    table = torch.full((3, W), -1, dtype=torch.int32)
    for s, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s, lp] = perm.pop()
    table = table.cuda()
    cache = torch.randn(n_pages, 2, nkv, page, hd, device="cuda", generator=g)
    # positions never written hold NaN: a kernel that reads past a sequence's end shows it
    for s, c in enumerate(ctx_lens):
        last = int(table[s, (c - 1) // page])
        if c % page:
            cache[last, :, :, c % page:] = float("nan")
    for p in perm:
        cache[p] = float("nan")
    seq_of_token = torch.tensor(sum(([s] * n for s, n in enumerate(new)), []), dtype=torch.int32, device="cuda")
    positions = torch.tensor(sum((list(range(c - n, c)) for c, n in zip(ctx_lens, new)), []), dtype=torch.int32, device="cuda")
    T = int(seq_of_token.shape[0])
    q = torch.randn(T, nh * hd, device="cuda", generator=g)
    # make one far key decide the first (decode) token: a key near the start of the long
    # context gets a large score for head 0 (if it is inside the window)
    far = 3 if not window else ctx_lens[0] - window + 1
    kvh0 = 0
    pg, off = int(table[0, far // page]), far % page
    cache[pg, 0, kvh0, off] = q[0, :hd] * 3.0
    cache = cache.to(dtype)
    q = q.to(dtype)
    scale = hd ** -0.5
    want = plain_paged_attention(q.float(), cache.float(), table, seq_of_token, positions, nh, nkv, hd, scale, window)
    got = ops.paged_attention_generic(q, cache, table, seq_of_token, positions, nh, nkv, hd, scale, window)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got.float(), want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else tol(dtype)))
    # the far key really decides: head 0 of token 0 is close to that key's value
    v_far = cache[pg, 1, kvh0, off].float()
    assert (got[0, :hd].float() - v_far).abs().max() < 0.2 * v_far.abs().max() + 0.1


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, 37),
                                                   (8, 2, 64, 32, None), (28, 4, 128, 16, None), (7, 1, 128, 16, 50),
                                                   (40, 2, 80, 16, None), (5, 5, 112, 8, 19), (16, 16, 96, 16, None)])
@pytest.mark.parametrize("n_splits", [1, 3, 16, -5])
def test_paged_attention_mma(ops, nh, nkv, hd, page, window, n_splits):
    """The tensor-core kernel on a mixed batch (a decode token deep in a long context, a
    prompt portion that starts in the middle of a page, a short whole prompt, a second decode
    token) with scrambled pages, unowned slots full of NaN and one far key that decides."""
    g = torch.Generator(device="cuda").manual_seed(15)
    ctx_lens = [301, 77, 9, 160]
    new = [1, 20, 9, 1]
    n_pages = sum(-(-c // page) for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(16)).tolist()
    W = max(-(-c // page) for c in ctx_lens)
    table = torch.full((4, W), -1, dtype=torch.int32)
    for s_, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s_, lp] = perm.pop()
    table = table.cuda()
    cache = torch.randn(n_pages, 2, nkv, page, hd, device="cuda", generator=g)
    for s_, c in enumerate(ctx_lens):
        if c % page:
            cache[int(table[s_, (c - 1) // page]), :, :, c % page:] = float("nan")
    for pg in perm:
        cache[pg] = float("nan")
    seq_of_token = torch.tensor(sum(([s_] * n for s_, n in enumerate(new)), []), dtype=torch.int32, device="cuda")
    positions = torch.tensor(sum((list(range(c - n, c)) for c, n in zip(ctx_lens, new)), []), dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 1, 21, 30, 31], dtype=torch.int32, device="cuda")
    T = int(seq_of_token.shape[0])
    q = torch.randn(T, nh * hd, device="cuda", generator=g)
    far = 3 if not window else ctx_lens[0] - window + 1
    pg, off = int(table[0, far // page]), far % page
    cache[pg, 0, 0, off] = q[0, :hd] * 3.0
    cache, q = cache.to(torch.bfloat16), q.to(torch.bfloat16)
    scale = hd ** -0.5
    want = plain_paged_attention(q.float(), cache.float(), table, seq_of_token, positions, nh, nkv, hd, scale, window)
    # splits merge through a thread-block cluster (up to 16 CTAs); a negative count here asks
    # for the other way: partial results in scratch memory and a combining kernel
    if n_splits > 0:
        got = ops.paged_attention_mma(q, cache, table, cu, positions, 4, nh, nkv, hd, scale, window, n_splits)
    else:
        scratch = torch.empty(T * nh * -n_splits * (hd + 2), dtype=torch.float32, device="cuda")
        got = ops.paged_attention_mma(q, cache, table, cu, positions, 4, nh, nkv, hd, scale, window, -n_splits, scratch=scratch)
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got.float(), want, rtol=1.6e-2, atol=1.2e-2)
    exact = ops.paged_attention_generic(q, cache, table, seq_of_token, positions, nh, nkv, hd, scale, window)
    assert (got.float() - exact.float()).abs().max().item() < 0.03
    v_far = cache[pg, 1, 0, off].float()
    assert (got[0, :hd].float() - v_far).abs().max() < 0.2 * v_far.abs().max() + 0.1


@pytest.mark.parametrize("dtype", DTYPES)
def test_consumers_add_partial_sums(ops, dtype):
    """A product whose K was split arrives as fp32 partial sums; the norm and the rotary
    kernel add them themselves and give what they give on the summed tensor."""
    g = torch.Generator(device="cuda").manual_seed(21)
    T, H, n = 6, 136, 3
    parts = torch.randn(n, T, H, device="cuda", generator=g)
    x = torch.randn(T, H, device="cuda", generator=g)
    w = 1 + 0.1 * torch.randn(H, device="cuda", generator=g)
    total = parts[0] + parts[1] + parts[2]
    x1, x2 = x.clone(), x.clone()
    a = ops.add_rmsnorm(x1, ops.PartialSums(parts, dtype), w, 1e-6, dtype)
    v = x + total
    want = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6)) * w
    torch.testing.assert_close(x1, v, rtol=0, atol=0)
    torch.testing.assert_close(a.float(), want, **tol(dtype))
    rows = torch.tensor([4, 1], dtype=torch.int32, device="cuda")
    b = ops.add_rmsnorm(x2, ops.PartialSums(parts, dtype), w, 1e-6, dtype, rows=rows)
    assert torch.equal(x2, x)
    torch.testing.assert_close(b.float(), want[rows.long()], **tol(dtype))
    torch.testing.assert_close(ops.materialize(ops.PartialSums(parts, dtype)).float(), total, **tol(dtype))
    # rotary: partial sums in, same result as the summed tensor in the activation dtype (fp32: exactly)
    nh, nkv, hd, page = 3, 1, 32, 8
    width = (nh + 2 * nkv) * hd
    parts = torch.randn(n, T, width, device="cuda", generator=g)
    bias = torch.randn(width, device="cuda", generator=g)
    pos = torch.arange(10, 10 + T, dtype=torch.int32, device="cuda")
    inv = (1.0 / (1e4 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).cuda()
    cos, sin = ops.rope_table(pos, inv)
    slots = torch.arange(T, dtype=torch.int32, device="cuda")
    c1 = torch.zeros(2, 2, nkv, page, hd, device="cuda", dtype=dtype)
    c2 = torch.zeros(2, 2, nkv, page, hd, device="cuda")
    q1 = ops.qkv_rope_write(ops.PartialSums(parts, dtype), bias, cos, sin, c1, slots, nh, nkv, hd, hd, page)
    q2 = ops.qkv_rope_write(parts[0] + parts[1] + parts[2], bias, cos, sin, c2, slots, nh, nkv, hd, hd, page)
    torch.testing.assert_close(c1.float(), c2, **tol(dtype))
    torch.testing.assert_close(q1.float(), q2, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(4, 2, 64, 16, None), (7, 1, 128, 16, None), (6, 3, 128, 8, 70),
                                                   (8, 8, 64, 32, 33), (28, 4, 128, 16, None)])
def test_attention_prefill_and_mixed_dispatch(ops, nh, nkv, hd, page, window):
    """Prompt portions (one that starts mid-page deep in a context, one whole prompt, one of
    exactly 64 tokens) beside decode tokens in ONE step: the long entries go to the tiled
    kernel, the short ones to the split-KV kernel, both write the same output tensor."""
    import numpy as np
    from pyre_b200.engine.context import StepContext
    g = torch.Generator(device="cuda").manual_seed(31)
    ctx_lens = [450, 100, 64, 333, 77, 40]
    new = [150, 100, 64, 1, 1, 20]
    B = len(new)
    n_pages = sum(-(-c // page) for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(32)).tolist()
    W = max(-(-c // page) for c in ctx_lens)
    table = torch.full((B, W), -1, dtype=torch.int32)
    for s_, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s_, lp] = perm.pop()
    table = table.cuda()
    cache = torch.randn(n_pages, 2, nkv, page, hd, device="cuda", generator=g)
    for s_, c in enumerate(ctx_lens):
        if c % page:
            cache[int(table[s_, (c - 1) // page]), :, :, c % page:] = float("nan")
    for pg in perm:
        cache[pg] = float("nan")
    seq_of_token = torch.tensor(sum(([s_] * n for s_, n in enumerate(new)), []), dtype=torch.int32, device="cuda")
    positions = torch.tensor(sum((list(range(c - n, c)) for c, n in zip(ctx_lens, new)), []), dtype=torch.int32, device="cuda")
    cu_host = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    cu = torch.from_numpy(cu_host).cuda()
    T = int(seq_of_token.shape[0])
    q = torch.randn(T, nh * hd, device="cuda", generator=g) * 1.5
    # one far key decides a row in the middle of the first portion (if its window reaches it)
    row = 77
    far = 5 if not window else int(positions[row]) - window + 1
    pg, off = int(table[0, far // page]), far % page
    cache[pg, 0, 0, off] = q[row, :hd] * 2.0
    cache, q = cache.to(torch.bfloat16), q.to(torch.bfloat16)
    scale = hd ** -0.5
    want = plain_paged_attention(q.float(), cache.float(), table, seq_of_token, positions, nh, nkv, hd, scale, window)
    z = torch.zeros(T, dtype=torch.int32, device="cuda")
    ctx = StepContext(dtype=torch.bfloat16, device=torch.device("cuda"), num_tokens=T, num_seqs=B, num_logit_rows=0,
                      token_ids=z, positions=positions, seq_of_token=seq_of_token, cu_seqlens=cu, logit_rows=z[:0],
                      cu_seqlens_host=cu_host, start_pos_host=np.asarray([c - n for c, n in zip(ctx_lens, new)]))
    got = ops.paged_attention_bf16(ctx, q, cache, table, nh, nkv, hd, scale, window)
    assert torch.isfinite(got).all()
    err = (got.float() - want).abs()
    bad = (err > 1.2e-2 + 1.6e-2 * want.abs()).any(dim=1)
    assert not bad.any(), f"first wrong token row {int(torch.where(bad)[0][0])} of {T}, max error {float(err.max()):.3e}"
    v_far = cache[pg, 1, 0, off].float()
    assert (got[row, :hd].float() - v_far).abs().max() < 0.25 * v_far.abs().max() + 0.1
    ops.check_device_errors()
    # both prompt-portion kernels alone (the tcgen05 one and the mma.sync one) agree with the plain statement
    for kernel, min_len in ((ops.attention_prefill_tc, 64), (ops.attention_prefill, 32)):
        if kernel is ops.attention_prefill_tc and page & (page - 1):
            continue
        alone = torch.full_like(q, 7.0)
        n_long = sum(n for n in new if n >= min_len)
        if kernel is ops.attention_prefill_tc:
            kernel(q, cache, table, cu, positions, B, n_long, nh, nkv, hd, scale, window, alone, min_len)
        else:
            kernel(q, cache, table, cu, positions, B, n_long, nh, nkv, hd, scale, window, alone)
        ops.check_device_errors()
        e2 = (alone[:314].float() - want[:314]).abs()
        bad2 = (e2 > 1.2e-2 + 1.6e-2 * want[:314].abs()).any(dim=1)
        assert not bad2.any(), f"{kernel.__name__}: first wrong row {int(torch.where(bad2)[0][0])}, max error {float(e2.max()):.3e}"
        assert float((alone[314:316].float() - 7.0).abs().max()) == 0.0
    # the tiled kernel alone leaves the short entries' rows untouched
    out = torch.full_like(q, 7.0)
    ops.attention_prefill(q, cache, table, cu, positions, B, 150 + 100 + 64, nh, nkv, hd, scale, window, out)
    assert float((out[314:316].float() - 7.0).abs().max()) == 0.0 and float((out[316:].float() - 7.0).abs().max()) == 0.0
    assert (out[:314].float() - want[:314]).abs().max() < 0.05


def plain_attention_portions(q, cache, table, cu, starts, nh, nkv, hd, scale, window):
    """Causal (windowed) attention of whole portions over the paged cache, in float64: pyre/model.py:104-124."""
    page = cache.shape[3]
    out = torch.zeros(q.shape[0], nh, hd, dtype=torch.float64, device=q.device)
    for s in range(len(starts)):
        b, e = int(cu[s]), int(cu[s + 1])
        n, ctx = e - b, int(starts[s]) + e - b
        idx = torch.arange(ctx, device=q.device)
        pages = table[s, idx // page].long()
        k = cache[pages, 0, :, idx % page].double().repeat_interleave(nh // nkv, dim=1)     # [ctx, nh, hd]
        v = cache[pages, 1, :, idx % page].double().repeat_interleave(nh // nkv, dim=1)
        pos = int(starts[s]) + torch.arange(n, device=q.device)
        mask = idx[None, :] <= pos[:, None]
        if window:
            mask &= idx[None, :] >= pos[:, None] - window + 1
        sc = torch.einsum("qhd,khd->hqk", q[b:e].double().view(n, nh, hd), k) * scale
        pr = torch.softmax(sc.masked_fill(~mask[None], float("-inf")), dim=-1)
        out[b:e] = torch.einsum("hqk,khd->qhd", pr, v)
    return out.view(q.shape[0], nh * hd).float()


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(4, 2, 128, 16, None), (3, 1, 64, 4, None), (2, 2, 128, 64, 100),
                                                   (4, 1, 64, 256, 300), (2, 1, 128, 8, 129), (7, 1, 128, 16, 1000)])
def test_attention_prefill_tc_long_portions(ops, nh, nkv, hd, page, window):
    """Portions of several 256-token pieces that start anywhere in their contexts (two query tiles per CTA share the
    key tiles; the last piece has one tile, or a second one of a single row), windows shorter and longer than a
    tile, pages from 4 tokens to more than a key tile; unwritten cache positions hold NaN, and one far key decides
    a row deep in the first portion."""
    g = torch.Generator(device="cuda").manual_seed(41)
    ctx_lens = [1000, 300, 2000, 500, 70]
    new = [700, 300, 257, 129, 64]
    starts = [c - n for c, n in zip(ctx_lens, new)]
    B = len(new)
    n_pages = sum(-(-c // page) for c in ctx_lens) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(42)).tolist()
    W = max(-(-c // page) for c in ctx_lens)
    table = torch.full((B, W), -1, dtype=torch.int32)
    for s_, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s_, lp] = perm.pop()
    table = table.cuda()
    cache = torch.randn(n_pages, 2, nkv, page, hd, device="cuda", generator=g)
    for s_, c in enumerate(ctx_lens):
        if c % page:
            cache[int(table[s_, (c - 1) // page]), :, :, c % page:] = float("nan")
    for pg in perm:
        cache[pg] = float("nan")
    cu = torch.tensor([0] + [sum(new[:k + 1]) for k in range(B)], dtype=torch.int32, device="cuda")
    positions = torch.tensor(sum((list(range(c - n, c)) for c, n in zip(ctx_lens, new)), []), dtype=torch.int32, device="cuda")
    T = int(positions.shape[0])
    q = torch.randn(T, nh * hd, device="cuda", generator=g) * 1.5
    row = 600                                           # of the first portion: position 900
    far = 5 if not window else max(int(positions[row]) - window + 1, 3)
    pg, off = int(table[0, far // page]), far % page
    cache[pg, 0, 0, off] = q[row, :hd] * 2.0
    cache, q = cache.to(torch.bfloat16), q.to(torch.bfloat16)
    scale = hd ** -0.5
    want = plain_attention_portions(q.float(), cache.float(), table, cu, starts, nh, nkv, hd, scale, window)
    # whole, and with the keys of every (query tile, head) shared by 2, 3 and 8 CTAs (some shares are empty, some hold
    # only masked keys for their first rows): the second launch of each also shows that nothing is left behind
    for key_splits in (1, 1, 2, 3, 8, 8):
        got = torch.full_like(q, 7.0)
        ops.attention_prefill_tc(q, cache, table, cu, positions, B, T, nh, nkv, hd, scale, window, got, 64, key_splits)
        ops.check_device_errors()
        assert torch.isfinite(got).all(), f"{key_splits} shares"
        err = (got.float() - want).abs()
        bad = (err > 1.2e-2 + 1.6e-2 * want.abs()).any(dim=1)
        assert not bad.any(), f"{key_splits} shares: first wrong token row {int(torch.where(bad)[0][0])} of {T}, max error {float(err.max()):.3e}"
        v_far = cache[pg, 1, 0, off].float()
        assert (got[row, :hd].float() - v_far).abs().max() < 0.25 * v_far.abs().max() + 0.1


def test_sampling_large_vocabulary_two_stages(ops):
    from plain import qwen2_plain
    g = torch.Generator(device="cuda").manual_seed(8)
    V = 40001                                  # above the one-block limit, not a multiple of the slice
    logits = torch.randn(3, V, device="cuda", generator=g)
    logits[1, 4095] = logits[1, 4096] = logits[1, 39999] = 30.0     # ties across slices: the lowest index wins
    assert ops.sample(logits).tolist() == [int(logits[0].argmax()), 4095, int(logits[2].argmax())]
    temps = torch.tensor([0.9, 0.0, 1.3], device="cuda")
    seeds = torch.tensor([5, 6, 7], dtype=torch.int64, device="cuda")
    tix = torch.tensor([2, 0, 11], dtype=torch.int32, device="cuda")
    got = ops.sample(logits, temps, seeds, tix).tolist()
    want = [qwen2_plain.sample(logits[r].cpu(), float(temps[r]), int(seeds[r]), int(tix[r])) for r in range(3)]
    assert got == want


def test_sampling(ops):
    from plain import qwen2_plain
    g = torch.Generator(device="cuda").manual_seed(7)
    V = 1531
    logits = torch.randn(6, V, device="cuda", generator=g)
    logits[2, 100] = logits[2, 900] = 50.0      # a tie: the lower index wins
    got = ops.sample(logits)
    want = [int(logits[r].argmax()) for r in range(6)]
    want[2] = 100
    assert got.tolist() == want
    temps = torch.tensor([0.0, 0.8, 0.8, 1.5, 0.3, 0.8], device="cuda")
    seeds = torch.tensor([1, 1, 2, 3, 4, 1], dtype=torch.int64, device="cuda")
    tix = torch.tensor([0, 0, 0, 5, 9, 1], dtype=torch.int32, device="cuda")
    got = ops.sample(logits, temps, seeds, tix).tolist()
    want = [qwen2_plain.sample(logits[r].cpu(), float(temps[r]), int(seeds[r]), int(tix[r])) for r in range(6)]
    assert got == want
    # the draw depends on (seed, token index) only, not on the row or the batch
    alone = ops.sample(logits[1:2].contiguous(), temps[1:2].contiguous(), seeds[1:2].contiguous(), tix[1:2].contiguous())
    assert alone.tolist() == [got[1]]
    # large vocabulary, many draws: frequencies follow softmax(logits / T)
    V2 = 50
    lg = torch.randn(1, V2, device="cuda", generator=g).repeat(4000, 1)
    draws = ops.sample(lg, torch.full((4000,), 0.7, device="cuda"), torch.arange(4000, dtype=torch.int64, device="cuda"),
                       torch.zeros(4000, dtype=torch.int32, device="cuda"))
    freq = torch.bincount(draws.long(), minlength=V2).float() / 4000
    p = torch.softmax(lg[0] / 0.7, dim=0)
    assert (freq - p).abs().max().item() < 0.03


def plain_attention_one_sequence(q, cache, table_row, positions, nh, nkv, hd, scale, window):
    """The queries of ONE sequence at ``positions`` over its cached keys 0..max position, all at once (fp64)."""
    page = cache.shape[3]
    n_ctx = int(positions.max()) + 1
    idx = torch.arange(n_ctx, device=q.device)
    pages = table_row[idx // page].long()
    k = cache[pages, 0, :, idx % page].double()            # [n_ctx, nkv, hd]
    v = cache[pages, 1, :, idx % page].double()
    T = q.shape[0]
    qf = q.double().view(T, nh, hd)
    pos = positions.long()[:, None]
    seen = idx[None, :] <= pos
    if window:
        seen &= idx[None, :] > pos - window
    out = torch.empty(T, nh, hd, dtype=torch.float64, device=q.device)
    for h in range(nh):
        kvh = h // (nh // nkv)
        sc = (qf[:, h] @ k[:, kvh].t()) * scale
        sc = sc.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(sc, dim=-1) @ v[:, kvh]
    return out.view(T, nh * hd).float()


@pytest.mark.parametrize("nh,nkv,hd,page,window", [(8, 2, 128, 16, None), (4, 1, 64, 64, 3000), (7, 1, 128, 32, None),
                                                   (6, 2, 128, 8, 5000)])
def test_attention_long_context(ops, nh, nkv, hd, page, window):
    """Thousands of keys: a 700-token portion at the end of a 9,000-token context (the tcgen05 kernel walks
    140 key tiles: its rings, its barrier phases and its lazy rescale wrap many times) and a decode token
    over 7,000 keys with 1, 4 and 16 splits (with one split a warp walks over a hundred tiles and re-reads
    its page numbers every 32), on scrambled pages, with one far key that decides a row."""
    import numpy as np
    from pyre_b200.engine.context import StepContext
    g = torch.Generator(device="cuda").manual_seed(41)
    ctx_lens, new = [9000, 7000], [700, 1]
    n_pages = sum(-(-c // page) for c in ctx_lens) + 5
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(42)).tolist()
    W = max(-(-c // page) for c in ctx_lens)
    table = torch.full((2, W), -1, dtype=torch.int32)
    for s_, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s_, lp] = perm.pop()
    table = table.cuda()
    cache = torch.randn(n_pages, 2, nkv, page, hd, device="cuda", generator=g)
    for pg in perm:
        cache[pg] = float("nan")                                   # pages nobody owns
    for s_, c in enumerate(ctx_lens):
        if c % page:
            cache[int(table[s_, (c - 1) // page]), :, :, c % page:] = float("nan")
    positions = torch.tensor(list(range(8300, 9000)) + [6999], dtype=torch.int32, device="cuda")
    seq_of_token = torch.tensor([0] * 700 + [1], dtype=torch.int32, device="cuda")
    cu_host = np.asarray([0, 700, 701], dtype=np.int32)
    cu = torch.from_numpy(cu_host).cuda()
    T = 701
    q = torch.randn(T, nh * hd, device="cuda", generator=g) * 1.5
    # a far key decides row 300 of the portion and the decode token: position 3, or the first inside the window
    marks = []
    for row, s_ in ((300, 0), (700, 1)):
        far = 3 if not window else int(positions[row]) - window + 1
        pg, off = int(table[s_, far // page]), far % page
        cache[pg, 0, 0, off] = q[row, :hd] * 2.5
        marks.append((row, pg, off))
    cache, q = cache.to(torch.bfloat16), q.to(torch.bfloat16)
    scale = hd ** -0.5
    want = torch.cat([plain_attention_one_sequence(q[:700].float(), cache.float(), table[0], positions[:700], nh, nkv, hd, scale, window),
                      plain_attention_one_sequence(q[700:].float(), cache.float(), table[1], positions[700:], nh, nkv, hd, scale, window)])
    z = torch.zeros(T, dtype=torch.int32, device="cuda")
    ctx = StepContext(dtype=torch.bfloat16, device=torch.device("cuda"), num_tokens=T, num_seqs=2, num_logit_rows=0,
                      token_ids=z, positions=positions, seq_of_token=seq_of_token, cu_seqlens=cu, logit_rows=z[:0],
                      cu_seqlens_host=cu_host, start_pos_host=np.asarray([8300, 6999]))

    def check(got, rows, what):
        assert torch.isfinite(got[rows]).all(), what
        err = (got[rows].float() - want[rows]).abs()
        bad = (err > 1.2e-2 + 1.6e-2 * want[rows].abs()).any(dim=1)
        assert not bad.any(), f"{what}: first wrong row {int(torch.where(bad)[0][0])}, max error {float(err.max()):.3e}"

    got = ops.paged_attention_bf16(ctx, q, cache, table, nh, nkv, hd, scale, window)
    ops.check_device_errors()
    check(got, slice(0, T), "dispatch")
    for row, pg, off in marks:
        v_far = cache[pg, 1, 0, off].float()
        assert (got[row, :hd].float() - v_far).abs().max() < 0.25 * v_far.abs().max() + 0.1
    # the decode token alone through the split-KV kernel: one split (long walks per warp), clusters of 4 and 16,
    # and 32 splits, which go through scratch memory and the combining kernel
    dec_cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    for n_splits in (1, 4, 16, 32, 64):
        alone = ops.paged_attention_mma(q[700:].contiguous(), cache, table[1:2].contiguous(), dec_cu, positions[700:].contiguous(),
                                        1, nh, nkv, hd, scale, window, n_splits, uniform_len=1)
        ops.check_device_errors()
        err = (alone.float() - want[700:]).abs()
        assert float((err - 1.2e-2 - 1.6e-2 * want[700:].abs()).max()) <= 0, f"{n_splits} splits: max error {float(err.max()):.3e}"
    # the portion through the mma.sync prompt kernel as well
    other = torch.full_like(q, 7.0)
    ops.attention_prefill(q, cache, table, cu, positions, 2, 700, nh, nkv, hd, scale, window, other)
    ops.check_device_errors()
    check(other, slice(0, 700), "mma.sync prompt kernel")


@pytest.mark.parametrize("M", [3, 100, 165, 256, 358])
@pytest.mark.parametrize("N", [148, 256, 20])
def test_rows_without_their_rms_into_any_product(ops, M, N):
    """Activations that still lack their 1/rms (``ScaledRows``) go into products of every plan: widths that are no
    multiple of 8 put the weights on the MMA's rows whatever the token count, and more than 128 tokens there are
    served by materialising the rows first."""
    g = torch.Generator(device="cuda").manual_seed(M + N)
    H, eps = 112, 1e-5
    v = torch.randn(M, H, device="cuda", generator=g) * 3.0
    gain = 1 + 0.1 * torch.randn(H, device="cuda", generator=g)
    w = (torch.randn(N, H, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    rows = (v * gain).to(torch.bfloat16)
    ssq = v.pow(2).sum(-1)[None].contiguous()                     # one tile of up to 128 features
    h = ops.ScaledRows(rows, ssq, eps)
    want = (rows.float() * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)) @ w.float().t()
    got = ops.linear(h, w)
    ops.check_device_errors()
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))
    torch.testing.assert_close(ops.materialize(h).float(), rows.float() * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps),
                               rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K", [(1, 3584, 3584), (8, 3584, 18944), (64, 896, 4864), (100, 200, 136), (128, 3584, 512), (5, 1160, 72),
                                   (2048, 3584, 3584), (300, 3584, 3584), (1000, 896, 4864), (2048, 3584, 18944), (700, 1160, 136)])
def test_product_with_residual_and_norm_folded_in(ops, M, N, K):
    """A product of few tokens launched by the norm that consumes it: the CTA that finishes a tile last adds the
    splits' partial sums to the residual stream and leaves the next norm's activations without their 1/rms
    (``ScaledRows``); the product that takes those applies the factor in its epilogue.  Against the same steps
    in fp32, for several launches in a row (the arrival counters return to zero)."""
    g = torch.Generator(device="cuda").manual_seed(3 * M + N)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.03).to(torch.bfloat16)
    gain = 1 + 0.1 * torch.randn(N, device="cuda", generator=g)
    w_next = (torch.randn(256, N, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    x0 = torch.randn(M, N, device="cuda", generator=g)
    eps = 1e-5
    for rep in range(3):
        x = x0.clone()
        prod = ops.linear(a, w, partials_ok=True, deferred_ok="residual")
        assert isinstance(prod, ops.DeferredProduct) == ops.folds_residual(M, N, K)     # offered only where it pays
        prod = ops.DeferredProduct(a, w, torch.bfloat16)
        assert tuple(prod.shape) == (M, N)
        if M > 128 and not ops.folds_residual(M, N, K):
            pytest.skip(f"the plan for {M} x {N} x {K} splits K: nothing to fold")
        h = ops.gemm_residual_norm(prod, x, gain, eps) if M <= 128 else ops.add_rmsnorm(x, prod, gain, eps, torch.bfloat16, scaled_ok=True)
        ops.check_device_errors()
        assert isinstance(h, ops.ScaledRows)
        v = x0 + a.float() @ w.float().t()
        scale = float(v.abs().max())
        assert float((x - v).abs().max()) <= 2e-5 * scale * max(1.0, (K / 64) ** 0.5), f"launch {rep}: residual stream"
        want = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * gain
        torch.testing.assert_close(ops.materialize(h).float(), want, rtol=1.6e-2, atol=2e-3)
        # the consumer applies the factor itself: plain product, split product, gated product
        y = ops.linear(h, w_next)
        torch.testing.assert_close(y.float(), want @ w_next.float().t(), rtol=2e-2, atol=2e-2 * float(want.abs().max()))
        y_parts = ops.materialize(ops.linear(h, w_next, partials_ok=True))
        torch.testing.assert_close(y_parts.float(), y.float(), rtol=1.6e-2, atol=1e-2)
        if N % 8 == 0:
            gu = ops.interleave_gate_up(w_next[:128], w_next[128:])
            act = ops.gated_linear(h, gu, interleaved=True)
            yy = want.to(torch.bfloat16).float() @ w_next.float().t()
            ref = torch.nn.functional.silu(yy[:, :128]) * yy[:, 128:]
            torch.testing.assert_close(act.float(), ref, rtol=3e-2, atol=3e-2 * float(ref.abs().max()))
    # the same norm without the permission to fold gives plain tensors
    x = x0.clone()
    plain = ops.add_rmsnorm(x, ops.DeferredProduct(a, w, torch.bfloat16), gain, eps, torch.bfloat16)
    assert isinstance(plain, torch.Tensor)
    torch.testing.assert_close(plain.float(), want, rtol=1.6e-2, atol=2e-3)
    ops.check_device_errors()


@pytest.mark.parametrize("nh,nkv,hd,rot,page", [(28, 4, 128, 128, 16), (14, 2, 64, 64, 16), (3, 1, 32, 32, 8), (5, 2, 16, 16, 4),
                                                (6, 3, 64, 0, 32), (7, 1, 128, 128, 64)])
@pytest.mark.parametrize("T", [1, 8, 77])
def test_product_with_rotary_and_cache_write_folded_in(ops, nh, nkv, hd, rot, page, T):
    """The stacked q/k/v projection launched by ``qkv_rope_write``: bias, rotation and the paged write of keys and
    values as the product's fix-up give bit for bit what the separate kernel gives on the same partial sums."""
    g = torch.Generator(device="cuda").manual_seed(nh * 13 + T)
    K = 264
    width = (nh + 2 * nkv) * hd
    a = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(width, K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(width, device="cuda", generator=g)
    pos = torch.randint(0, 5000, (T,), device="cuda", generator=g, dtype=torch.int32)
    inv = 1.0 / (1e4 ** (torch.arange(0, max(rot, 2), 2, device="cuda", dtype=torch.float32) / max(rot, 2)))
    cos, sin = ops.rope_table(pos, inv) if rot else (None, None)
    n_pages = -(-T // page) + 3
    slots = torch.randperm(n_pages * page, device="cuda", generator=g)[:T].to(torch.int32).contiguous()
    caches, qs = [], []
    for fold in (True, False):
        cache = torch.zeros(n_pages, 2, nkv, page, hd, device="cuda", dtype=torch.bfloat16)
        prod = ops.DeferredProduct(a, w, torch.bfloat16)
        qs.append(ops.qkv_rope_write(prod if fold else prod.partials(), bias, cos, sin, cache, slots, nh, nkv, hd, rot, page))
        caches.append(cache)
    ops.check_device_errors()
    assert torch.equal(qs[0], qs[1]) and torch.equal(caches[0], caches[1])
    assert float(caches[0].float().abs().sum()) > 0
    # a layer that reads another layer's cache stores nothing
    q_only = ops.qkv_rope_write(ops.DeferredProduct(a, w, torch.bfloat16), bias, cos, sin, None, None, nh, nkv, hd, rot, page)
    assert torch.equal(q_only, qs[0])


@pytest.mark.parametrize("nh,nkv,hd,rot,page", [(28, 4, 128, 128, 16), (14, 2, 64, 64, 16), (6, 3, 64, 0, 32), (3, 1, 32, 32, 8),
                                                (7, 1, 128, 128, 64), (5, 2, 48, 48, 16)])
@pytest.mark.parametrize("T", [129, 300, 2048])
def test_rotary_and_cache_write_in_the_epilogue_of_a_prompt_portion(ops, nh, nkv, hd, rot, page, T):
    """More than 128 tokens: the stacked q/k/v product has the tokens on the MMA's rows, and where its tiles hold whole
    heads the epilogue thread that owns a token row adds the bias, rotates and stores queries, keys and values itself
    (no rotary kernel, no q/k/v matrix in memory).  Against the formula in fp64; the folded result rounds once and is
    at least as close as the separate kernel's; shapes whose heads do not fill tiles take the separate kernel."""
    g = torch.Generator(device="cuda").manual_seed(nh * 17 + T)
    K = 264
    width = (nh + 2 * nkv) * hd
    a = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(width, K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    bias = torch.randn(width, device="cuda", generator=g)
    pos = torch.randint(0, 5000, (T,), device="cuda", generator=g, dtype=torch.int32)
    inv = 1.0 / (1e4 ** (torch.arange(0, max(rot, 2), 2, device="cuda", dtype=torch.float32) / max(rot, 2)))
    cos, sin = ops.rope_table(pos, inv) if rot else (None, None)
    n_pages = -(-T // page) + 3
    slots = torch.randperm(n_pages * page, device="cuda", generator=g)[:T].to(torch.int32).contiguous()
    y = (a.double() @ w.double().t() + bias.double()).view(T, nh + 2 * nkv, hd)
    if rot:
        c, s_ = cos.double()[:, None, :], sin.double()[:, None, :]
        y1, y2 = y[:, :nh + nkv, :hd // 2], y[:, :nh + nkv, hd // 2:]
        y = torch.cat([torch.cat([y1 * c - y2 * s_, y2 * c + y1 * s_], dim=-1), y[:, nh + nkv:]], dim=1)
    want_q = y[:, :nh].reshape(T, nh * hd)
    want_k, want_v = y[:, nh:nh + nkv], y[:, nh + nkv:]
    assert ops.folds_rope(T, width, K, hd) == (ops.rope_fold_width(width, hd) > 0)
    errs = []
    for fold in (True, False):
        cache = torch.full((n_pages, 2, nkv, page, hd), 9.0, device="cuda", dtype=torch.bfloat16)
        prod = ops.DeferredProduct(a, w, torch.bfloat16)
        q = ops.qkv_rope_write(prod if fold else prod.partials(), bias, cos, sin, cache, slots, nh, nkv, hd, rot, page)
        ops.check_device_errors()
        pg, off = (slots // page).long(), (slots % page).long()
        got_k, got_v = cache[pg, 0, :, off], cache[pg, 1, :, off]             # [T, nkv, hd]
        scale = float(y.abs().max())
        for got, want in ((q, want_q), (got_k, want_k), (got_v, want_v)):
            assert float((got.double() - want).abs().max()) <= 1.2e-2 * scale
        errs.append(float((q.double() - want_q).abs().mean() + (got_k.double() - want_k).abs().mean()))
        untouched = torch.ones(n_pages * page, dtype=torch.bool, device="cuda")
        untouched[slots.long()] = False
        assert bool((cache.permute(0, 3, 1, 2, 4).reshape(n_pages * page, -1)[untouched] == 9.0).all()), "a slot of no token was written"
    assert errs[0] <= errs[1] * 1.02, f"folded {errs[0]:.3e} against separate {errs[1]:.3e}"


@pytest.mark.parametrize("kernel,dtype,nh,nkv,hd,page,window", [
    ("generic", torch.float32, 6, 3, 48, 4, 37), ("generic", torch.bfloat16, 3, 1, 32, 8, 19), ("generic", torch.float32, 4, 2, 16, 16, 64),
    ("mma", torch.bfloat16, 6, 3, 48, 4, 37), ("mma", torch.bfloat16, 7, 1, 128, 8, 50), ("mma", torch.bfloat16, 28, 4, 128, 16, 64),
    ("prefill", torch.bfloat16, 6, 3, 128, 8, 50), ("prefill", torch.bfloat16, 4, 2, 64, 12, 37),
    ("tc", torch.bfloat16, 6, 3, 128, 8, 50), ("tc", torch.bfloat16, 4, 1, 64, 4, 37), ("tc", torch.bfloat16, 28, 4, 128, 16, 64)])
def test_window_edges_are_exact(ops, kernel, dtype, nh, nkv, hd, page, window):
    """Both edges of a window, for a decode row and for a row in the middle of a prompt portion.  The first key inside
    the window (position p - window + 1) carries a large score and a distinctive value: the output is that value.  The
    key just outside (p - window) carries a larger score still, and so does a key one page further out: the output
    must not move by a bit when those keys' values are exchanged (+40 against -40), which an off-by-one at the edge,
    in the mask or in the tiles' range, could not survive."""
    g = torch.Generator(device="cuda").manual_seed(nh * 7 + page)
    ctx_lens, new = [301, 200], [1, 70]
    n_pages = sum(-(-c // page) for c in ctx_lens) + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(9)).tolist()
    table = torch.full((2, max(-(-c // page) for c in ctx_lens)), -1, dtype=torch.int32)
    for s_, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s_, lp] = perm.pop()
    table = table.cuda()
    seq_of_token = torch.tensor([0] + [1] * 70, dtype=torch.int32, device="cuda")
    positions = torch.tensor([300] + list(range(130, 200)), dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, 1, 71], dtype=torch.int32, device="cuda")
    T = 71
    q = torch.randn(T, nh * hd, device="cuda", generator=g)
    master = torch.randn(n_pages, 2, nkv, page, hd, device="cuda", generator=g)
    rows = [0, 1 + 35]                                   # the decode row; row 35 of the portion
    inside_value = torch.linspace(-3, 3, hd, device="cuda")

    def slot(s_, pos):
        return int(table[s_, pos // page]), pos % page

    def build(sign):
        cache = master.clone()
        for r in rows:
            s_, p = int(seq_of_token[r]), int(positions[r])
            qh = q[r, :hd] / q[r, :hd].norm() * hd ** 0.5      # head 0 of the row, which reads key/value head 0
            pg, off = slot(s_, p - window + 1)
            cache[pg, 0, 0, off], cache[pg, 1, 0, off] = qh * 6.0, inside_value
            for outside in (p - window, p - window - page):      # just outside, and a page further out
                pg, off = slot(s_, outside)
                cache[pg, 0, 0, off], cache[pg, 1, 0, off] = qh * 9.0, sign * 40.0
        return cache.to(dtype)

    qd = q.clone()
    for r in rows:
        qd[r, :hd] = q[r, :hd] / q[r, :hd].norm() * hd ** 0.5
    qd = qd.to(dtype)
    scale = hd ** -0.5

    def run(cache):
        if kernel == "generic":
            return ops.paged_attention_generic(qd, cache, table, seq_of_token, positions, nh, nkv, hd, scale, window)
        out = torch.zeros_like(qd)
        if kernel == "mma":
            return ops.paged_attention_mma(qd, cache, table, cu, positions, 2, nh, nkv, hd, scale, window, 3, out=out)
        if kernel == "prefill":
            return ops.attention_prefill(qd, cache, table, cu, positions, 2, 70, nh, nkv, hd, scale, window, out, min_len=32)
        return ops.attention_prefill_tc(qd, cache, table, cu, positions, 2, 70, nh, nkv, hd, scale, window, out, min_len=64)

    a, b = run(build(+1.0)), run(build(-1.0))
    ops.check_device_errors()
    for r in rows if kernel in ("generic", "mma") else rows[1:]:      # the prompt-portion kernels take the long entry only
        head0 = a[r, :hd].float()
        assert torch.equal(a[r], b[r]), f"row {r}: a key outside the window reaches the output"
        assert (head0 - inside_value).abs().max() < 0.05 * 3 + (0.02 if dtype == torch.float32 else 0.06), \
            f"row {r}: the first key inside the window does not decide (max diff {(head0 - inside_value).abs().max():.3f})"
