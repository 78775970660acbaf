"""Plain, slow implementation of the Qwen2.5 dense decoder: the oracle of the tests.

Whole sequences, no cache, one function for each part, plain torch on whatever
device and dtype the tensors have.  It shares no code with ``pyre_b200``: it reads a
``config.json`` dictionary and a dictionary of tensors under their checkpoint names.
Every function is written from the reference's formulas and cites them by
``file:line`` within Lalitaditya-tickoo/pyre.  ``tests/golden/make_golden.py`` compared
it once with the reference's own ``PyreQwen2.forward`` on the CPU; the outputs of
that run are committed under ``tests/golden/`` and checked by
``tests/test_plain_vs_golden.py``.

The functions take two generalisations that the reference does not have, so that the
tests can drive the engine's parts at other settings: a sliding ``window`` in
``attention`` (None = all keys, the reference's behaviour) and a ``schedule`` in
``forward`` that may run a layer twice or let a layer read another layer's keys and
values.  With their defaults they compute the reference's model.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """pyre/model.py:33-38: variance in fp32, cast down, then multiply by the weight."""
    dtype = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return weight * xf.to(dtype)


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype):
    """pyre/model.py:41-51: inv_freq[j] = theta^(-2j/hd) in fp32, angle = position * inv_freq,
    table = cat[angle, angle], cos and sin cast to the model dtype.  ``positions`` (S,)
    holds absolute positions (the reference slices rows start_pos..start_pos+S,
    pyre/model.py:177-186)."""
    device = positions.device
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    freqs = torch.outer(positions.to(torch.float32), inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """pyre/model.py:54-56."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """pyre/model.py:59-63 for one of q, k: x (heads, S, hd); cos, sin (S, hd)."""
    return x * cos.unsqueeze(0) + rotate_half(x) * sin.unsqueeze(0)


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """pyre/model.py:66-72: (kv, S, hd) -> (kv*n_rep, S, hd); query head i reads kv head i // n_rep."""
    return x if n_rep == 1 else x.repeat_interleave(n_rep, dim=0)


def project_qkv(x: torch.Tensor, w: dict, prefix: str, n_heads: int, n_kv: int, head_dim: int):
    """pyre/model.py:92-94: biased q, k, v projections split into heads, head-major columns.
    x (S, H) -> q (nh, S, hd), k and v (nkv, S, hd)."""
    S = x.shape[0]
    q = torch.nn.functional.linear(x, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"])
    k = torch.nn.functional.linear(x, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"])
    v = torch.nn.functional.linear(x, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"])
    return (q.view(S, n_heads, head_dim).transpose(0, 1),
            k.view(S, n_kv, head_dim).transpose(0, 1),
            v.view(S, n_kv, head_dim).transpose(0, 1))


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """pyre/model.py:104-124 on a whole sequence (start_pos = 0, so the mask's diagonal
    is 1): scores = (q k^T) * hd^-0.5, causal mask with the dtype's most negative
    value, softmax in fp32 cast back, times v, heads merged.
    q (nh, S, hd), k and v (nkv, S, hd) -> (S, nh*hd).
    ``window`` (not in the reference): query i sees keys j with i - window < j <= i."""
    n_heads, S, head_dim = q.shape
    n_rep = n_heads // k.shape[0]
    k = repeat_kv(k, n_rep)
    v = repeat_kv(v, n_rep)
    scores = torch.matmul(q, k.transpose(-1, -2)) * (head_dim ** -0.5)
    neg = torch.finfo(scores.dtype).min
    if S > 1:
        mask = torch.triu(torch.full((S, S), neg, device=q.device, dtype=scores.dtype), diagonal=1)
        scores = scores + mask
    if window is not None:
        i = torch.arange(S, device=q.device)
        too_old = (i[:, None] - i[None, :]) >= window
        scores = scores.masked_fill(too_old, neg)
    probs = torch.softmax(scores.to(torch.float32), dim=-1).to(q.dtype)
    out = torch.matmul(probs, v)
    return out.transpose(0, 1).reshape(S, n_heads * head_dim)


def swiglu_mlp(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """pyre/model.py:128-139: down(silu(gate(x)) * up(x)), no biases."""
    lin = torch.nn.functional.linear
    gate = lin(x, w[prefix + "gate_proj.weight"])
    up = lin(x, w[prefix + "up_proj.weight"])
    return lin(torch.nn.functional.silu(gate) * up, w[prefix + "down_proj.weight"])


def decoder_layer(x, w, cfg, layer: int, cos, sin, kv_from=None, window=None):
    """pyre/model.py:150-153 with the attention of pyre/model.py:89-125:
    x = x + o_proj(attn(norm_in(x))); x = x + mlp(norm_post(x)).
    Returns the new x and the layer's rotated keys and values.  ``kv_from`` (not in the
    reference) replaces this layer's own keys and values by another layer's."""
    p = f"model.layers.{layer}."
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    q, k, v = project_qkv(h, w, p + "self_attn.", nh, nkv, hd)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    if kv_from is not None:
        k, v = kv_from
    a = attention(q, k, v, window)
    x = x + torch.nn.functional.linear(a, w[p + "self_attn.o_proj.weight"])
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + swiglu_mlp(h, w, p + "mlp.")
    return x, (k, v)


def normalise_config(raw: dict) -> dict:
    """pyre/config.py:45-61: the keys the reference reads, with its defaults."""
    heads = raw["num_attention_heads"]
    return {
        "hidden_size": raw["hidden_size"],
        "intermediate_size": raw["intermediate_size"],
        "num_hidden_layers": raw["num_hidden_layers"],
        "num_attention_heads": heads,
        "num_key_value_heads": raw.get("num_key_value_heads", heads),
        "vocab_size": raw["vocab_size"],
        "rms_norm_eps": raw.get("rms_norm_eps", 1e-6),
        "rope_theta": float(raw.get("rope_theta", 10000.0)),
        "tie_word_embeddings": bool(raw.get("tie_word_embeddings", False)),
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads,
    }


def forward(ids, w: dict, raw_cfg: dict, schedule=None, windows=None, return_hidden: bool = False):
    """pyre/model.py:188-201 without a cache: ids (S,) -> logits (S, V) at every position.

    ``w`` maps checkpoint names to tensors; a missing ``lm_head.weight`` with tied
    embeddings is the embedding matrix (pyre/loader.py:58-61).
    ``schedule`` (not in the reference): list of (layer, source) pairs run in order;
    ``source`` None means the layer uses its own keys and values, an index means it
    reads those that the schedule entry of that index produced.  Default: every layer once.
    ``windows``: per schedule entry, a window or None."""
    cfg = normalise_config(raw_cfg)
    ids = torch.as_tensor(ids, dtype=torch.long, device=w["model.embed_tokens.weight"].device)
    x = w["model.embed_tokens.weight"][ids]
    positions = torch.arange(ids.shape[0], device=x.device)
    cos, sin = rope_tables(positions, cfg["head_dim"], cfg["rope_theta"], x.dtype)
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    produced = []
    hidden = []
    for n, (layer, source) in enumerate(schedule):
        kv_from = produced[source] if source is not None else None
        window = windows[n] if windows is not None else None
        x, kv = decoder_layer(x, w, cfg, layer, cos, sin, kv_from, window)
        produced.append(kv)
        hidden.append(x)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w.get("lm_head.weight")
    if head is None:
        if not cfg["tie_word_embeddings"]:
            raise KeyError("lm_head.weight missing but tie_word_embeddings is false")
        head = w["model.embed_tokens.weight"]
    logits = torch.nn.functional.linear(x, head)
    return (logits, hidden) if return_hidden else logits


def greedy_generate(prompt, w: dict, raw_cfg: dict, max_new_tokens: int, eos_id=None) -> list[int]:
    """pyre/model.py:203-215: recompute the whole sequence for every token, argmax of
    the last row; the token equal to ``eos_id`` is kept and ends the output
    (pyre/scheduler.py:82)."""
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        logits = forward(ids, w, raw_cfg)
        nxt = int(logits[-1].to(torch.float32).argmax())
        out.append(nxt)
        ids.append(nxt)
        if eos_id is not None and nxt == eos_id:
            break
    return out


# ---------------------------------------------------------------------------
# Sampling.  The reference samples greedily only (pyre/scheduler.py:80,94); the
# temperature sampler below is the test's own statement of the engine's rule, in
# integer and double arithmetic on the host.
# ---------------------------------------------------------------------------

_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    """The splitmix64 finaliser on a 64-bit integer."""
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def gumbel_noise(seed: int, token_index: int, vocab_index: int) -> float:
    """Noise of one (request seed, index of the generated token, vocabulary entry):
    a 23-bit uniform in (0, 1) from two rounds of the mixer, then -log(-log(u))."""
    h = _mix64((seed & _M64) ^ _mix64((token_index << 32 | vocab_index) & _M64))
    u = ((h >> 41) + 0.5) / 8388608.0
    return -math.log(-math.log(u))


def sample(logits: torch.Tensor, temperature: float, seed: int, token_index: int) -> int:
    """Greedy when temperature is 0 (lowest index wins a tie), else the Gumbel-max rule
    argmax(logit / temperature + noise)."""
    row = logits.to(torch.float32).cpu()
    if temperature == 0.0:
        return int(row.argmax())
    best, best_score = 0, -math.inf
    inv_t = 1.0 / temperature
    for v in range(row.shape[0]):
        score = float(row[v]) * inv_t + gumbel_noise(seed, token_index, v)
        if score > best_score:
            best, best_score = v, score
    return best
