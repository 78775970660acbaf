"""The allocation-free attention entry point, called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory where they call
attention (in a serving loop with a fixed memory budget, under a host runtime that owns
all device memory, from a C host without an allocator); ``pyre_paged_attention_mma_noalloc`` keeps the
split-KV scratch in a device array inside its own library for them.  This test loads
that library with ctypes, calls the symbol twice in a row on different inputs (the
array keeps the first call's contents) and checks each result against the ordinary entry
point, which gets its scratch from the caller.  It also checks that a request beyond the
array's capacity is refused.  The file sorts last so that a run that stops at the first
failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_SCRATCH_TOO_LARGE = 100003


def _load():
    from pyre_b200.kernels import build
    build.ensure_built(["attention_mma_noalloc"])
    lib = ctypes.CDLL(str(build.library_path("attention_mma_noalloc")))
    fn = lib.pyre_paged_attention_mma_noalloc
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, P]
    fn.restype = I
    lib.pyre_paged_attention_mma_noalloc_capacity.restype = ctypes.c_longlong
    return lib, fn


def _case(seed, nh, nkv, hd, page, ctx_lens, new):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_seqs = len(ctx_lens)
    n_pages = sum(-(-c // page) for c in ctx_lens) + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(-(-c // page) for c in ctx_lens)
    table = torch.full((n_seqs, width), -1, dtype=torch.int32)
    for s, c in enumerate(ctx_lens):
        for lp in range(-(-c // page)):
            table[s, lp] = perm.pop()
    cache = torch.randn(n_pages, 2, nkv, page, hd, device="cuda", generator=g).to(torch.bfloat16)
    positions = torch.tensor(sum((list(range(c - n, c)) for c, n in zip(ctx_lens, new)), []), dtype=torch.int32, device="cuda")
    cu = torch.tensor([0] + list(torch.tensor(new).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(int(positions.shape[0]), nh * hd, device="cuda", generator=g).to(torch.bfloat16)
    return q, cache, table.cuda(), cu, positions, n_seqs


def test_noalloc_entry_matches_the_ordinary_one_twice_in_a_row():
    from pyre_b200.kernels import ops
    lib, fn = _load()
    assert lib.pyre_paged_attention_mma_noalloc_capacity() == 4 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    cases = [
        (dict(nh=28, nkv=4, hd=128, page=16, ctx_lens=[700, 33, 512, 90], new=[1, 1, 1, 1]), 5),   # decode, 5 splits
        (dict(nh=6, nkv=3, hd=48, page=8, ctx_lens=[301, 77, 9], new=[1, 20, 9]), 3),               # mixed, 3 splits
        (dict(nh=8, nkv=2, hd=64, page=32, ctx_lens=[400, 160], new=[1, 1]), 1),                    # no scratch at all
    ]
    for n, (shape, n_splits) in enumerate(cases):
        q, cache, table, cu, positions, n_seqs = _case(40 + n, **shape)
        nh, nkv, hd = shape["nh"], shape["nkv"], shape["hd"]
        scale = hd ** -0.5
        # the ordinary entry point with scratch from the caller (torch's allocator here)
        scratch = torch.empty(max(1, q.shape[0] * nh * n_splits * (hd + 2)), dtype=torch.float32, device="cuda")
        want = ops.paged_attention_mma(q, cache, table, cu, positions, n_seqs, nh, nkv, hd, scale, None, n_splits,
                                       scratch=scratch)
        got = torch.full_like(q, float("nan"))
        rc = fn(q.data_ptr(), cache.data_ptr(), got.data_ptr(), table.data_ptr(), table.stride(0), cu.data_ptr(),
                positions.data_ptr(), q.shape[0], n_seqs, nh, nkv, hd, shape["page"], 0, scale, n_splits, stream)
        assert rc == 0, f"case {n}: the entry point returned {rc}"
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # the same kernel code on the same inputs: the tolerance of the kernel tests is far from needed
        torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1.2e-2)
        assert torch.equal(got, want)


def test_noalloc_entry_refuses_what_does_not_fit():
    lib, fn = _load()
    q, cache, table, cu, positions, n_seqs = _case(7, nh=28, nkv=4, hd=128, page=16, ctx_lens=[64] * 40, new=[32] * 40)
    out = torch.zeros_like(q)
    # 1280 tokens x 28 heads x 64 splits x 130 floats is far beyond 4 Mi floats
    rc = fn(q.data_ptr(), cache.data_ptr(), out.data_ptr(), table.data_ptr(), table.stride(0), cu.data_ptr(),
            positions.data_ptr(), q.shape[0], n_seqs, 28, 4, 128, 16, 0, 0.1, 64, torch.cuda.current_stream().cuda_stream)
    assert rc == ERR_SCRATCH_TOO_LARGE
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0          # nothing was launched
