"""Plain torch stand-ins for the CUDA kernels, float32 only, for tests without a GPU.

They state each kernel's contract (arguments, layouts, what is written where) in the simplest
terms and share no code with the kernels.  With them in place of ``pyre_b200.kernels.ops`` the
package's own parts, model, cache manager, step function and replay loop run on the CPU, so the
host side of the engine (the batch's layout, the block tables, the order of the schedule, the
bookkeeping of lengths and pages) is tested against the plain implementation where no GPU is."""

from __future__ import annotations

import torch


def embedding(table, ids, out=None, err_flag=None):
    return table[ids.long()].float()


def add_rmsnorm(x, delta, weight, eps, out_dtype, rows=None, update_x=True, out=None):
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
    from pyre_b200.kernels import ops

    flag = torch.zeros(1, dtype=torch.int32)
    for name, fn in dict(embedding=embedding, add_rmsnorm=add_rmsnorm, add_residual=add_residual, rope_table=rope_table,
                         qkv_rope_write=qkv_rope_write, paged_attention_generic=paged_attention_generic,
                         sgemm_nt=sgemm_nt, silu_mul=silu_mul, sample=sample, feed_tokens=feed_tokens).items():
        monkeypatch.setattr(ops, name, fn)
    monkeypatch.setattr(ops, "device_error_flag", lambda device: flag)
    monkeypatch.setattr(ops, "check_device_errors", lambda device="cpu": None)
    monkeypatch.setattr(step._Staging, "upload", lambda self, flat: torch.from_numpy(flat.copy()))
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
