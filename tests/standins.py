"""Plain torch stand-ins for the CUDA kernels, for tests without a GPU.

They state each kernel's contract (arguments, layouts, what is written where) in the simplest
terms and share no code with the kernels.  With them in place of ``pyre_b200.kernels.ops`` the
package's own parts, model, cache manager, step function and replay loop run on the CPU, so the
host side of the engine (the batch's layout, the block tables, the order of the schedule, the
bookkeeping of lengths and pages) is tested against the plain implementation where no GPU is."""

from __future__ import annotations

import torch


def embedding(table, ids, out=None, err_flag=None):
    return table[ids.long()].float()


def add_rmsnorm(x, delta, weight, eps, out_dtype, rows=None, update_x=True, out=None, scaled_ok=False):
    v = x if delta is None else x + delta.float()
    if rows is None and update_x and delta is not None:
        x.copy_(v)
    if rows is not None:
        v = v[rows.long()]
    h = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight
    return h.to(out_dtype)


def add_residual(x, delta):
    x.add_(delta.float())
    return x


def rope_table(positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def qkv_rope_write(qkv, bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads, head_dim, rotary_dim,
                   page_size, q_out=None):
    T = qkv.shape[0]
    x = qkv.float()
    if bias is not None:
        x = x + bias
    q, k, v = x.split([n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim], dim=1)
    q, k, v = q.reshape(T, n_heads, head_dim), k.reshape(T, n_kv_heads, head_dim), v.reshape(T, n_kv_heads, head_dim)

    def rotate(t):
        if not rotary_dim:
            return t
        half = rotary_dim // 2
        a, b, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
        c, s = cos[:, None, :], sin[:, None, :]
        return torch.cat([a * c - b * s, b * c + a * s, rest], dim=-1)

    q, k = rotate(q), rotate(k)
    if cache_layer is not None:
        for t in range(T):
            page, off = divmod(int(slot_mapping[t]), page_size)
            cache_layer[page, 0, :, off, :] = k[t].to(cache_layer.dtype)
            cache_layer[page, 1, :, off, :] = v[t].to(cache_layer.dtype)
    return q.reshape(T, n_heads * head_dim).to(qkv.dtype)


def paged_attention_generic(q, cache_layer, block_table, seq_of_token, positions, n_heads, n_kv_heads, head_dim, scale,
                            window=None, out=None):
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    n_rep = n_heads // n_kv_heads
    result = torch.empty_like(q)
    for t in range(T):
        b, p = int(seq_of_token[t]), int(positions[t])
        lo = 0 if not window else max(0, p - window + 1)
        pos = torch.arange(lo, p + 1)
        pages = block_table[b].long()[pos // page_size]
        assert (pages >= 0).all(), f"token {t}: a key in its window lies on a page that was given back"
        keys = cache_layer[pages, 0, :, pos % page_size, :].float()          # [keys, kv heads, head_dim]
        vals = cache_layer[pages, 1, :, pos % page_size, :].float()
        qt = q[t].float().reshape(n_kv_heads, n_rep, head_dim)
        scores = torch.einsum("grd,kgd->grk", qt, keys) * scale
        probs = torch.softmax(scores, dim=-1)
        result[t] = torch.einsum("grk,kgd->grd", probs, vals).reshape(-1).to(q.dtype)
    return result


def sgemm_nt(a, w, bias=None, out=None):
    y = a @ w.t()
    return y if bias is None else y + bias


def silu_mul(gate_up, out=None, block=0):
    assert block == 0, "the float32 path stacks all gates before all ups"
    inter = gate_up.shape[1] // 2
    return torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]


def sample(logits, temperature=None, seeds=None, token_index=None, out=None):
    assert temperature is None, "the stand-in samples greedily only"
    return logits.argmax(dim=-1).to(torch.int32)


def feed_tokens(token_ids, dst, src, prev):
    for d, s in zip(dst.tolist(), src.tolist()):
        if d >= 0:
            token_ids[d] = prev[s]


def install(monkeypatch) -> None:
    """Put the stand-ins in place of the kernels for one test (float32 models on the CPU)."""
    from pyre_b200.engine import step
    from pyre_b200.kernels import build, ops

    monkeypatch.setattr(build, "ensure_built", lambda names, **kw: None)     # the stand-ins need no library
    flag = torch.zeros(1, dtype=torch.int32)
    for name, fn in dict(embedding=embedding, add_rmsnorm=add_rmsnorm, add_residual=add_residual, rope_table=rope_table,
                         qkv_rope_write=qkv_rope_write, paged_attention_generic=paged_attention_generic,
                         sgemm_nt=sgemm_nt, silu_mul=silu_mul, sample=sample, feed_tokens=feed_tokens).items():
        monkeypatch.setattr(ops, name, fn)
    monkeypatch.setattr(ops, "device_error_flag", lambda device: flag)
    monkeypatch.setattr(ops, "check_device_errors", lambda device="cpu": None)
    monkeypatch.setattr(step._Staging, "upload", lambda self, flat: torch.from_numpy(flat.copy()))
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)


# --------------------------------------------------------------------------- the bfloat16 path
# Stand-ins for the tensor-core kernels: bf16 operands, fp32 arithmetic, results rounded where the
# kernels round them.  The products honour the package's own plan (orientation, width, split of K), so
# split-K partial sums travel to their consumers as they do on the device; the attention stand-ins
# write only the rows of the entries that the kernel they stand for would take.

def _partial_sums_or_tensor(t):
    from pyre_b200.kernels import ops
    if isinstance(t, ops.DeferredProduct):      # a product not launched yet: the stand-ins never fold, they run it plainly
        t = t.partials()
    return t.parts.sum(0) if isinstance(t, ops.PartialSums) else t.float()


def add_rmsnorm_any(x, delta, weight, eps, out_dtype, rows=None, update_x=True, out=None, scaled_ok=False):
    return add_rmsnorm(x, None if delta is None else _partial_sums_or_tensor(delta), weight, eps, out_dtype, rows, update_x)


def qkv_rope_write_any(qkv, bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads, head_dim, rotary_dim,
                       page_size, q_out=None):
    act = qkv.dtype          # of the activations, for a tensor and for partial sums alike
    q = qkv_rope_write(_partial_sums_or_tensor(qkv), bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads,
                       head_dim, rotary_dim, page_size)
    return q.to(act)


def materialize(t):
    from pyre_b200.kernels import ops
    if isinstance(t, ops.DeferredProduct):
        t = t.partials()
    return t.parts.sum(0).to(t.dtype) if isinstance(t, ops.PartialSums) else t


def gemm_tc(x, w, out_dtype=torch.bfloat16, plan=None, reduce=True, gated=False, pair=None, checked=False):
    from pyre_b200.kernels import ops
    assert x.dtype == w.dtype == torch.bfloat16 and x.shape[1] == w.shape[1]
    M, K = x.shape
    N = w.shape[0]
    _rows, _bn, splits = plan or ops.tc_gemm_plan(M, N, K)
    kb = -(-K // 64)
    splits = max(1, min(splits, kb))
    if gated:
        assert N % (2 * ops.GATED_BLOCK) == 0
        y = (x.float() @ w.float().t()).view(M, N // (2 * ops.GATED_BLOCK), 2, ops.GATED_BLOCK)
        return (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(M, N // 2).to(torch.bfloat16)
    per = -(-kb // splits) * 64
    parts = torch.stack([x[:, s * per:(s + 1) * per].float() @ w[:, s * per:(s + 1) * per].float().t() for s in range(splits)])
    if splits == 1 and reduce:
        return parts[0].to(out_dtype)
    if not reduce:
        return ops.PartialSums(parts.contiguous(), out_dtype)
    return parts.sum(0).to(out_dtype)


def silu_mul_any(gate_up, out=None, block=0):
    if block == 0:
        return silu_mul(gate_up.float()).to(gate_up.dtype)
    T, two_i = gate_up.shape
    y = gate_up.float().view(T, two_i // (2 * block), 2, block)
    return (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(T, two_i // 2).to(gate_up.dtype)


def _attend_entries(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale, window,
                    out, takes):
    cu = cu_seqlens.tolist()
    taken = 0
    for b in range(n_seqs):
        n = cu[b + 1] - cu[b]
        if not takes(n):
            continue
        taken += n
        rows = slice(cu[b], cu[b + 1])
        out[rows] = paged_attention_generic(q[rows], cache_layer, block_table[b:b + 1], torch.zeros(n, dtype=torch.int32),
                                            positions[rows], n_heads, n_kv_heads, head_dim, scale, window)
    return taken


def paged_attention_mma(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale,
                        window=None, n_splits=1, out=None, scratch=None, max_len=0, uniform_len=0):
    from pyre_b200.kernels import ops
    assert q.dtype == cache_layer.dtype == torch.bfloat16 and head_dim <= ops.MMA_MAX_HEAD_DIM
    assert 1 <= n_splits <= ops.MAX_SCRATCH_SPLITS
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    assert not uniform_len or all(n == uniform_len for n in lens), "uniform_len promises entries of one length"
    if out is None:
        out = torch.empty_like(q)
    _attend_entries(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale, window,
                    out, lambda n: not (max_len > 0 and n > max_len))
    return out


def attention_prefill(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_long_tokens, n_heads, n_kv_heads,
                      head_dim, scale, window, out, min_len=32):
    from pyre_b200.kernels import ops
    assert head_dim in ops.PREFILL_HEAD_DIMS
    taken = _attend_entries(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_heads, n_kv_heads, head_dim, scale,
                            window, out, lambda n: n >= min_len)
    assert taken == n_long_tokens, "n_long_tokens must count the tokens of the entries this kernel takes"
    return out


def attention_prefill_tc(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_long_tokens, n_heads, n_kv_heads,
                         head_dim, scale, window, out, min_len, key_splits=1):
    page_size = cache_layer.shape[3]
    assert 1 <= key_splits <= 32
    assert page_size & (page_size - 1) == 0 and page_size >= 4, "the tcgen05 attention takes power-of-two pages"
    return attention_prefill(q, cache_layer, block_table, cu_seqlens, positions, n_seqs, n_long_tokens, n_heads, n_kv_heads,
                             head_dim, scale, window, out, min_len)


def install_bf16(monkeypatch, calls: "dict | None" = None) -> None:
    """The float32 stand-ins plus those of the bfloat16 path.  ``calls`` (optional) counts how often
    each attention kernel's stand-in ran."""
    from pyre_b200.kernels import ops

    install(monkeypatch)

    def counted(name, fn):
        def wrapper(*a, **k):
            if calls is not None:
                calls[name] = calls.get(name, 0) + 1
            return fn(*a, **k)
        return wrapper

    for name, fn in dict(add_rmsnorm=add_rmsnorm_any, qkv_rope_write=qkv_rope_write_any, materialize=materialize,
                         gemm_tc=gemm_tc, silu_mul=silu_mul_any).items():
        monkeypatch.setattr(ops, name, fn)
    for name, fn in dict(paged_attention_mma=paged_attention_mma, attention_prefill=attention_prefill,
                         attention_prefill_tc=attention_prefill_tc).items():
        monkeypatch.setattr(ops, name, counted(name, fn))
