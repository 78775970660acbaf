"""The kernels as Python functions over torch tensors.

Each function checks shapes, dtypes, contiguity and device, then launches the CUDA
kernel on torch's current stream.  A size the kernels do not take is refused with a
clear error; nothing here computes on the CPU or falls back to a library.

The matrix products are the package's own kernels too (``gemm_tc`` on the tcgen05 tensor
cores for bfloat16, ``sgemm_nt`` for float32).  One case goes to a library (cuBLAS through
``torch``): a bfloat16 product whose rows are no multiple of 16 bytes, which a TMA copy
cannot fetch; the reference's engine uses a library for every projection (``nn.Linear``,
pyre/model.py:84-87,133-135,172).  See ``linear``.
"""

from __future__ import annotations

import ctypes

import torch

from . import lib

_DT = {torch.float32: 0, torch.bfloat16: 1}


class UnsupportedSize(ValueError):
    """A configuration whose sizes the kernels refuse."""


class PartialSums:
    """fp32 partial sums [n, T, N] of a matrix product whose inner dimension was split over
    CTAs.  The kernels that consume a product (``add_rmsnorm``, ``qkv_rope_write``) add the n
    parts themselves, in index order, so no separate reduction runs; anything else calls
    ``materialize``."""

    def __init__(self, parts: torch.Tensor, dtype: torch.dtype):
        self.parts = parts          # contiguous [n, T, N] float32
        self.dtype = dtype          # what materialize() rounds to

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def n(self) -> int:
        return self.parts.shape[0]


class ScaledRows:
    """Activations that carry a norm's weight but not yet its 1/rms: ``rows`` [T, H] bf16 and, per token, the
    sums of squares of the normalised vector's elements in tiles of 128 features (``ssq`` [tiles, T] fp32).  The
    normalised activations are ``rows[t] / sqrt(sum(ssq[:, t]) / H + eps)``.  A product that takes them applies the
    factor to its result rows in its epilogue (the factor is a scalar per row, so it commutes with the product);
    anything else calls ``materialize``."""

    def __init__(self, rows: torch.Tensor, ssq: torch.Tensor, eps: float):
        self.rows, self.ssq, self.eps = rows, ssq, float(eps)

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    @property
    def device(self):
        return self.rows.device


class DeferredProduct:
    """y = x w^T of a linear layer over few tokens, not launched yet.  The kernel that consumes it decides how it
    runs: the built-in norm launches it with a fix-up that adds the result to the residual stream and prepares the
    normalised activations (no norm kernel), the rotary position encoding with one that adds the bias, rotates and
    writes keys and values to the pages (no rotary kernel); anything else calls ``partials`` or ``materialize``."""

    def __init__(self, x: "torch.Tensor | ScaledRows", w: torch.Tensor, dtype: torch.dtype):
        self.x, self.w, self.dtype = x, w, dtype
        self.section = lib.current_section()      # the kernel class its launch counts for, whoever launches it

    @property
    def shape(self):
        return (self.x.shape[0], self.w.shape[0])

    @property
    def device(self):
        return self.w.device

    def partials(self) -> "torch.Tensor | PartialSums":
        """Launch the plain product: a tensor, or partial sums where K is split."""
        with lib.section(self.section):
            return gemm_tc(self.x, self.w, self.dtype, reduce=False)


def materialize(t: "torch.Tensor | PartialSums | DeferredProduct | ScaledRows") -> torch.Tensor:
    """A plain tensor in the activation dtype from a tensor or any of the lazy forms a branch output or a
    norm's output may take."""
    if isinstance(t, DeferredProduct):
        t = t.partials()
    if isinstance(t, ScaledRows):
        out = torch.empty_like(t.rows)
        T, H = t.rows.shape
        lib.call("pyre_scale_rows", t.rows.data_ptr(), t.ssq.data_ptr(), t.ssq.shape[0], out.data_ptr(), T, H, t.eps, _stream())
        return out
    if not isinstance(t, PartialSums):
        return t
    out = torch.empty(tuple(t.shape), dtype=t.dtype, device=t.parts.device)
    n = t.parts[0].numel()
    lib.call("pyre_sum_partials", t.parts.data_ptr(), t.n, n, out.data_ptr(), n, _dt(t.dtype), _stream())
    return out


# A step of prompt portions is a few hundred launches from Python, so the two questions every launch asks (which
# stream, which device) go to torch's C layer directly where it offers that (a fraction of a microsecond instead of
# several); the public calls stand in where it does not.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _current_device() -> int:
    return _raw_device() if _raw_device is not None else torch.cuda.current_device()


def _stream() -> int:
    """The current stream of the current device.  Kernels are launched in the current device's
    context, so the tensors of a call must live there (``_check`` refuses others)."""
    if _raw_stream is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def require_current_device(device, what: str = "a tensor") -> None:
    """Raise on the host if ``device`` (a CUDA device) is not the current one.  A kernel launched
    on another device's stream with this device's pointers would fault on the GPU instead."""
    current = _current_device()
    index = device.index if device.index is not None else current
    if index != current:
        raise ValueError(f"{what} is on cuda:{index} but the current device is cuda:{current}; "
                         f"enter torch.cuda.device({index}) around the call")


def _ptr(t: "torch.Tensor | None") -> "int | None":
    return None if t is None else t.data_ptr()


def _check(t: torch.Tensor, name: str, dtype=None, dim: "int | None" = None) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (pyre_b200 has no CPU path)")
    require_current_device(t.device, name)
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise ValueError(f"{name} must have {dim} dimensions, got shape {tuple(t.shape)}")


def _dt(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise ValueError(f"activations must be float32 or bfloat16, got {dtype}") from None


def embedding(table: torch.Tensor, ids: torch.Tensor, out: "torch.Tensor | None" = None,
              err_flag: "torch.Tensor | None" = None) -> torch.Tensor:
    """x[t] = float32(table[ids[t]]); ids int32 [T]; returns the fp32 residual stream [T, H]."""
    _check(table, "table", dim=2)
    _check(ids, "ids", torch.int32, 1)
    V, H = table.shape
    T = ids.shape[0]
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    else:
        _check(out, "out", torch.float32, 2)
    lib.call("pyre_embedding", table.data_ptr(), _dt(table.dtype), ids.data_ptr(), out.data_ptr(), T, H, V,
             _ptr(err_flag), _stream())
    return out


def add_rmsnorm(x: torch.Tensor, delta: "torch.Tensor | None", weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: "torch.Tensor | None" = None, update_x: bool = True,
                out: "torch.Tensor | None" = None, scaled_ok: bool = False) -> "torch.Tensor | ScaledRows":
    """out[r] = rmsnorm(x[src] + delta[src]) * weight with src = rows[r] (or r).

    ``x`` is the fp32 residual stream [T, H]; with ``update_x`` (and no ``rows``) the sum is
    written back to it.  ``delta`` has the activation dtype, or is a ``PartialSums`` whose
    parts the kernel adds, or a ``DeferredProduct``.  ``weight`` is fp32 [H].

    ``scaled_ok``: the caller's consumer takes ``ScaledRows``.  Then a deferred product is launched with the
    residual add and the norm's preparation as its fix-up, and no norm kernel runs at all."""
    _check(x, "x", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    T, H = x.shape
    if weight.shape[0] != H:
        raise ValueError(f"norm weight has {weight.shape[0]} entries, rows have {H}")
    if isinstance(delta, DeferredProduct):
        if tuple(delta.shape) != (T, H):
            raise ValueError(f"delta shape {tuple(delta.shape)} != x shape {(T, H)}")
        if scaled_ok and rows is None and update_x and out is None and out_dtype == torch.bfloat16 and H % 8 == 0 \
                and H <= 128 * _MAX_FIX_TILES and folds_residual(T, H, delta.x.shape[1]):
            return gemm_residual_norm(delta, x, weight, eps)
        delta = delta.partials()
    parts, n_parts, part_stride = None, 0, 0
    if isinstance(delta, PartialSums):
        if tuple(delta.shape) != (T, H):
            raise ValueError(f"delta shape {tuple(delta.shape)} != x shape {(T, H)}")
        parts, n_parts, part_stride, delta = delta.parts, delta.n, T * H, None
    elif delta is not None:
        _check(delta, "delta", out_dtype, 2)
        if tuple(delta.shape) != (T, H):
            raise ValueError(f"delta shape {tuple(delta.shape)} != x shape {(T, H)}")
    n_rows = T
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        n_rows = rows.shape[0]
        update_x = False
    if out is None:
        out = torch.empty((n_rows, H), dtype=out_dtype, device=x.device)
    else:
        _check(out, "out", out_dtype, 2)
    lib.call("pyre_add_rmsnorm", x.data_ptr(), _ptr(delta), _ptr(parts), n_parts, part_stride, weight.data_ptr(),
             out.data_ptr(), _ptr(rows), n_rows, H, float(eps),
             int(bool(update_x and (delta is not None or parts is not None))), _dt(out_dtype), _stream())
    return out


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """x += float32(delta) in place on the fp32 residual stream: for a block arrangement in which no
    norm follows a branch (the built-in pre-norm block adds its branches inside the next norm's kernel)."""
    _check(x, "x", torch.float32)
    _check(delta, "delta")
    if x.shape != delta.shape:
        raise ValueError("x and delta differ in shape")
    lib.call("pyre_add_residual", x.data_ptr(), delta.data_ptr(), x.numel(), _dt(delta.dtype), _stream())
    return x


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor):
    """cos, sin fp32 [T, rot/2] of float(position) * inv_freq."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    T, half = positions.shape[0], inv_freq.shape[0]
    cos = torch.empty((T, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    lib.call("pyre_rope_table", positions.data_ptr(), inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, half,
             _stream())
    return cos, sin


def qkv_rope_write(qkv: torch.Tensor, bias: "torch.Tensor | None", cos: torch.Tensor, sin: torch.Tensor,
                   cache_layer: "torch.Tensor | None", slot_mapping: "torch.Tensor | None",
                   n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, page_size: int,
                   q_out: "torch.Tensor | None" = None) -> torch.Tensor:
    """Bias, rotary and the paged K/V write in one pass; returns rotated q [T, nh*hd].

    ``cache_layer``: [pages, 2, nkv, page_size, hd] of the activation dtype, or None to
    store nothing (a layer that reads another layer's cache)."""
    if isinstance(qkv, DeferredProduct):
        width = (n_heads + 2 * n_kv_heads) * head_dim
        few = qkv.shape[0] <= 128 and 128 % head_dim == 0 and head_dim % 8 == 0 and width <= 128 * _MAX_FIX_TILES
        many = qkv.shape[0] > 128 and folds_rope(qkv.shape[0], width, qkv.x.shape[1], head_dim)
        if q_out is None and qkv.shape[1] == width and rotary_dim in (0, head_dim) and (few or many):
            return gemm_rope_write(qkv, bias, cos, sin, cache_layer, slot_mapping, n_heads, n_kv_heads, head_dim,
                                   rotary_dim, page_size)
        qkv = qkv.partials()
    parts, n_parts = None, 0
    if isinstance(qkv, PartialSums):
        parts, n_parts, act_dtype, device = qkv.parts, qkv.n, qkv.dtype, qkv.parts.device
    else:
        _check(qkv, "qkv", dim=2)
        act_dtype, device = qkv.dtype, qkv.device
    T = qkv.shape[0]
    width = (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise ValueError(f"qkv has {qkv.shape[1]} columns, expected (nh + 2 nkv) * hd = {width}")
    if head_dim % 8 or rotary_dim % 8 or not 0 <= rotary_dim <= head_dim:
        raise UnsupportedSize(f"head_dim ({head_dim}) and rotary_dim ({rotary_dim}) must be multiples of 8, "
                              f"rotary_dim <= head_dim")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
        if bias.shape[0] != width:
            raise ValueError(f"qkv bias has {bias.shape[0]} entries, expected {width}")
    half = rotary_dim // 2
    if rotary_dim:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, half) or tuple(sin.shape) != (T, half):
            raise ValueError(f"cos/sin must be [{T}, {half}], got {tuple(cos.shape)}")
    if cache_layer is not None:
        _check(cache_layer, "cache_layer", act_dtype, 5)
        if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match "
                             f"[pages, 2, {n_kv_heads}, {page_size}, {head_dim}]")
        if slot_mapping is None:
            raise ValueError("slot_mapping is required with a cache")
        _check(slot_mapping, "slot_mapping", torch.int32, 1)
        if slot_mapping.shape[0] != T:
            raise ValueError("slot_mapping must have one entry per token")
    if q_out is None:
        q_out = torch.empty((T, n_heads * head_dim), dtype=act_dtype, device=device)
    lib.call("pyre_qkv_rope_write", None if parts is not None else qkv.data_ptr(), _ptr(parts), n_parts, T * width,
             _ptr(bias), _ptr(cos) if rotary_dim else None,
             _ptr(sin) if rotary_dim else None, q_out.data_ptr(), _ptr(cache_layer),
             _ptr(slot_mapping) if cache_layer is not None else None, T, n_heads, n_kv_heads, head_dim,
             rotary_dim, page_size, _dt(act_dtype), cache_layer.shape[0] if cache_layer is not None else 0,
             device_error_flag(device).data_ptr(), _stream())
    return q_out


def silu_mul(gate_up: torch.Tensor, out: "torch.Tensor | None" = None, block: int = 0) -> torch.Tensor:
    """out[t, i] = silu(gate[t, i]) * up[t, i].  ``block == 0``: gate_up = [all gates | all ups];
    ``block == n``: gates and ups alternate in blocks of n features (n gates, their n ups, ...)."""
    _check(gate_up, "gate_up", dim=2)
    T, two_i = gate_up.shape
    if two_i % 2:
        raise ValueError("gate_up must have an even number of columns")
    inter = two_i // 2
    if block and (block % 8 or inter % block):
        raise UnsupportedSize(f"silu_mul: blocks of {block} features do not tile {inter} features in steps of 8")
    if out is None:
        out = torch.empty((T, inter), dtype=gate_up.dtype, device=gate_up.device)
    lib.call("pyre_silu_mul", gate_up.data_ptr(), out.data_ptr(), T, inter, int(block), _dt(gate_up.dtype), _stream())
    return out


def feed_tokens(token_ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """token_ids[dst[i]] = prev[src[i]] where dst[i] >= 0 (all int32, on the device): tokens sampled by
    the last step enter the next one without a trip through the host."""
    for t, name in ((token_ids, "token_ids"), (dst, "dst"), (src, "src"), (prev, "prev")):
        _check(t, name, torch.int32, 1)
    if dst.shape[0] != src.shape[0]:
        raise ValueError("dst and src must have one entry each per fed token")
    lib.call("pyre_feed_tokens", token_ids.data_ptr(), dst.data_ptr(), src.data_ptr(), prev.data_ptr(), dst.shape[0], _stream())


def delay(milliseconds: float) -> None:
    """Queue a kernel that idles for ``milliseconds`` (at most 1,000) on the current stream: a measured region
    queued behind it is in the stream in full before the GPU starts on it."""
    lib.call("pyre_delay", int(milliseconds * 1e6), _stream())


def sample(logits: torch.Tensor, temperature: "torch.Tensor | None" = None, seeds: "torch.Tensor | None" = None,
           token_index: "torch.Tensor | None" = None, out: "torch.Tensor | None" = None) -> torch.Tensor:
    """One token id per row of fp32 logits [R, V]: argmax where temperature is 0, else Gumbel-max."""
    if logits.dim() != 2 or logits.dtype != torch.float32 or not logits.is_cuda or logits.stride(1) != 1:
        raise ValueError("logits must be a CUDA float32 matrix with contiguous rows")
    R, V = logits.shape
    if temperature is not None:
        _check(temperature, "temperature", torch.float32, 1)
        if seeds is None or token_index is None:
            raise ValueError("temperature sampling needs seeds and token_index")
        _check(seeds, "seeds", torch.int64, 1)
        _check(token_index, "token_index", torch.int32, 1)
        if not (temperature.shape[0] == seeds.shape[0] == token_index.shape[0] == R):
            raise ValueError("temperature, seeds and token_index need one entry per row")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    slices = lib.call_value("pyre_sample_slices", V)
    scratch = torch.empty(R * slices * 2, dtype=torch.int32, device=logits.device) if slices else None
    lib.call("pyre_sample", logits.data_ptr(), logits.stride(0), _ptr(temperature), _ptr(seeds), _ptr(token_index),
             out.data_ptr(), R, V, _ptr(scratch), _stream())
    return out


def paged_attention_generic(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor,
                            seq_of_token: torch.Tensor, positions: torch.Tensor, n_heads: int, n_kv_heads: int,
                            head_dim: int, scale: float, window: "int | None" = None,
                            out: "torch.Tensor | None" = None) -> torch.Tensor:
    """Exact fp32-arithmetic attention of every query token over its sequence's pages."""
    _check(q, "q", dim=2)
    _check(cache_layer, "cache_layer", q.dtype, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(seq_of_token, "seq_of_token", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T = q.shape[0]
    if q.shape[1] != n_heads * head_dim:
        raise ValueError(f"q has {q.shape[1]} columns, expected nh * hd = {n_heads * head_dim}")
    if head_dim % 16 or head_dim > 256:
        raise UnsupportedSize(f"head_dim {head_dim}: the attention kernels take multiples of 16 up to 256")
    if n_heads % n_kv_heads:
        raise UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
        raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match the head sizes")
    if out is None:
        out = torch.empty_like(q)
    lib.call("pyre_paged_attention_generic", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), seq_of_token.data_ptr(), positions.data_ptr(), T,
             n_heads, n_kv_heads, head_dim, page_size, int(window or 0), float(scale), _dt(q.dtype), cache_layer.shape[0],
             device_error_flag(q.device).data_ptr(), _stream())
    return out


MMA_MAX_HEAD_DIM = 128
CLUSTER_MAX_SPLITS = 16      # splits of one group merge through a thread-block cluster up to this many
MAX_SCRATCH_SPLITS = 64      # beyond a cluster: partial results through scratch memory and the combining kernel
_DEFAULT_SM_COUNT = 148     # a B200; used only where no device can be asked (planning on a host without a GPU)
_sm_counts: dict = {}
_have_cuda: "bool | None" = None


def sm_count(device=None) -> int:
    """Multiprocessors of ``device`` (default: the current one), as the launch code asks the device
    too; the planners below size splits and rounds of tiles by it."""
    global _have_cuda
    if _have_cuda is None:
        _have_cuda = torch.cuda.is_available()
    if not _have_cuda:
        return _DEFAULT_SM_COUNT
    index = _current_device() if device is None or torch.device(device).index is None else torch.device(device).index
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count) or _DEFAULT_SM_COUNT
    return n


def attention_splits(n_tokens: int, n_seqs: int, n_heads: int, n_kv_heads: int, max_context: int,
                     window: "int | None", n_groups: "int | None" = None) -> int:
    """How many ways the tensor-core kernel splits each sequence's keys: enough CTAs for
    about one and a half per SM, at least two 16-key tiles per split, at most 16 (the
    splits of a group form one thread-block cluster), or 24 to 64 through scratch memory for
    one or two sequences with long contexts."""
    _SM_COUNT = sm_count()
    n_rep = n_heads // n_kv_heads
    hpg = min(n_rep, 16)
    tpg = 16 // hpg
    if n_groups is None:     # one token per entry (decode) when the counts agree, else an upper bound
        n_groups = n_seqs if n_tokens == n_seqs else n_tokens // tpg + n_seqs
    ctas = n_groups * n_kv_heads * (-(-n_rep // hpg))
    span = max_context if not window else min(max_context, window + tpg)
    tiles = -(-span // 16) + 1
    # Measured inside whole decode steps (7B shape, contexts of 2-3 thousand tokens): about one and a half CTAs per
    # SM in all is best (batch 8: 7 splits, 16: 4, 32: 2, 64: 1); with two per SM the product that follows
    # finds no SM on which to prefetch its weights while the attention runs.
    # One or two sequences with long contexts: a cluster's 16 CTAs per group leave most SMs idle and give every warp
    # dozens of tiles (0.6 us of dependent work each).  Many small CTAs (about 256 in all, at least 16 tiles each)
    # through scratch memory and the combining kernel win there: alone, 8,192 keys 10.9 -> 8.9 us, 16,384 keys
    # 16.9 -> 12.3, 32,768 keys 25.7 -> 17.0 (one sequence); 34.0 -> 25.9 for two sequences of 32,768.
    # Four sequences of 32,768 keys: 16 splits through scratch 47.4 us, 32: 49.3, clusters of 8 or 16: 62-68.
    many = min(256 // max(ctas, 1), tiles // 16, MAX_SCRATCH_SPLITS)
    if many >= 24 or (many >= 16 and tiles >= 512):
        return max(24, many // 8 * 8)
    want = max(1, min(int(1.57 * _SM_COUNT / max(ctas, 1) + 0.5), -(-tiles // 2), CLUSTER_MAX_SPLITS))
    if want > 8:
        # a cluster of 16 CTAs must sit in one GPC: it pays only while all of them fit on the chip at once
        if ctas * 16 > _SM_COUNT:
            return min(want, 10)
        # one or two sequences with tens of thousands of keys: 16 CTAs per group leave most SMs idle; 32 splits
        # through scratch memory and the combining kernel win from about 24 thousand keys on
        if ctas * 32 <= _SM_COUNT and tiles >= 1536:
            return 32
        return 16
    return int(want)


def paged_attention_mma(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor,
                        cu_seqlens: torch.Tensor, positions: torch.Tensor, n_seqs: int, n_heads: int,
                        n_kv_heads: int, head_dim: int, scale: float, window: "int | None" = None,
                        n_splits: int = 1, out: "torch.Tensor | None" = None,
                        scratch: "torch.Tensor | None" = None, max_len: int = 0, uniform_len: int = 0) -> torch.Tensor:
    """bfloat16 attention on the tensor cores over the block table (decode tokens and
    prompt portions alike); ``n_splits`` > 1 splits each sequence's keys over CTAs and needs
    ``T * nh * n_splits * (hd + 2)`` floats of scratch (allocated here if not given)."""
    _check(q, "q", torch.bfloat16, 2)
    _check(cache_layer, "cache_layer", torch.bfloat16, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    T = q.shape[0]
    if q.shape[1] != n_heads * head_dim:
        raise ValueError(f"q has {q.shape[1]} columns, expected nh * hd = {n_heads * head_dim}")
    if head_dim % 16 or not 16 <= head_dim <= MMA_MAX_HEAD_DIM:
        raise UnsupportedSize(f"head_dim {head_dim}: the tensor-core attention takes multiples of 16 up to {MMA_MAX_HEAD_DIM}")
    if n_heads % n_kv_heads:
        raise UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
        raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match the head sizes")
    if cu_seqlens.shape[0] != n_seqs + 1 or positions.shape[0] != T or block_table.shape[0] < n_seqs:
        raise ValueError("cu_seqlens, positions and block_table do not match the batch")
    if out is None:
        out = torch.empty_like(q)
    n_splits = int(n_splits)
    if n_splits > 1 and not (scratch is None and n_splits <= CLUSTER_MAX_SPLITS):
        need = T * n_heads * n_splits * (head_dim + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        elif scratch.dtype != torch.float32 or scratch.numel() < need or not scratch.is_contiguous():
            raise ValueError(f"scratch must be {need} contiguous floats")
    lib.call("pyre_paged_attention_mma", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), _ptr(scratch),
             block_table.data_ptr(), block_table.stride(0), cu_seqlens.data_ptr(), positions.data_ptr(), T, n_seqs,
             n_heads, n_kv_heads, head_dim, page_size, int(window or 0), float(scale), n_splits, int(max_len),
             cache_layer.shape[0], int(uniform_len), device_error_flag(q.device).data_ptr(), _stream())
    return out


PREFILL_HEAD_DIMS = (64, 128)
PREFILL_MIN_LEN = 32     # entries with at least this many tokens go to the prompt-portion kernel


def attention_prefill(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                      positions: torch.Tensor, n_seqs: int, n_long_tokens: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, scale: float, window: "int | None", out: torch.Tensor,
                      min_len: int = PREFILL_MIN_LEN) -> torch.Tensor:
    """bfloat16 attention of the entries with at least ``min_len`` tokens (64 queries of a head
    per CTA, keys and values tiled through shared memory); writes only those entries' rows of ``out``."""
    _check(q, "q", torch.bfloat16, 2)
    _check(cache_layer, "cache_layer", torch.bfloat16, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    _check(out, "out", torch.bfloat16, 2)
    if head_dim not in PREFILL_HEAD_DIMS:
        raise UnsupportedSize(f"head_dim {head_dim}: the prompt-portion attention kernel takes {PREFILL_HEAD_DIMS}")
    if n_heads % n_kv_heads:
        raise UnsupportedSize(f"{n_heads} query heads cannot be shared among {n_kv_heads} key/value heads")
    page_size = cache_layer.shape[3]
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim) or q.shape[1] != n_heads * head_dim:
        raise ValueError("q or the cache layer do not match the head sizes")
    if out.shape != q.shape or cu_seqlens.shape[0] != n_seqs + 1 or positions.shape[0] != q.shape[0]:
        raise ValueError("out, cu_seqlens and positions do not match the batch")
    lib.call("pyre_attention_prefill", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), cu_seqlens.data_ptr(), positions.data_ptr(), int(n_long_tokens), n_seqs, n_heads,
             n_kv_heads, head_dim, page_size, int(window or 0), float(scale), int(min_len), cache_layer.shape[0],
             device_error_flag(q.device).data_ptr(), _stream())
    return out


USE_TC_ATTENTION = True
TC_ATTENTION_MIN_LEN = 64    # entries with at least this many tokens go to the tcgen05 kernel (128-query tiles)


MAX_KEY_SPLITS = 8
KEY_SPLIT_SCRATCH_BYTES = 128 << 20      # of partial outputs per launch (fewer items than SMs keep it below this anyway)


def prefill_key_splits(n_items: int, mean_tiles: float, n_tokens: int, n_heads: int, head_dim: int) -> int:
    """Into how many shares of the keys the prompt attention cuts every (128-query tile, head).  Shares pay only
    while SMs would stand idle: an SM runs the tiles of one CTA alone as fast as those of two together, so what
    counts is that every SM has a CTA, and a share costs its partial output's trip through memory and a second
    kernel (measured: 2,048 tokens after 8,192, 448 items, 292 us whole, 350 in two shares; 512 tokens after 30,720,
    112 items, 492 us whole, 294 in two shares, 269 in five).  So: only with fewer items than SMs, as many shares as
    fill two CTAs per SM, each of at least 16 key tiles (1,024 keys); or as many as fill them twice over, if every
    share then still has 80 key tiles (two rounds of 97 tiles beat one round of 242; two rounds of 65 lose to one of
    131: 640 tokens after 16,384, 191 us in four shares against 186 in two)."""
    sms = sm_count()
    if n_items >= sms:
        return 1
    s = min(MAX_KEY_SPLITS, 2 * sms // max(n_items, 1), int(mean_tiles // 16))
    twice = min(MAX_KEY_SPLITS, 4 * sms // max(n_items, 1))
    if twice > s and mean_tiles / twice >= 80:
        s = twice
    while s > 1 and n_tokens * n_heads * s * head_dim * 4 > KEY_SPLIT_SCRATCH_BYTES:
        s -= 1
    return max(1, s)


def attention_prefill_tc(q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, cu_seqlens: torch.Tensor,
                         positions: torch.Tensor, n_seqs: int, n_long_tokens: int, n_heads: int, n_kv_heads: int,
                         head_dim: int, scale: float, window: "int | None", out: torch.Tensor, min_len: int,
                         key_splits: int = 1) -> torch.Tensor:
    """bfloat16 attention of the entries with at least ``min_len`` tokens on the tcgen05 tensor
    cores (scores and output in tensor memory, Q/K/V tiles by TMA); writes only those entries' rows.
    ``key_splits`` > 1: that many CTAs share the keys of every (query tile, head); a second kernel combines them."""
    _check(q, "q", torch.bfloat16, 2)
    _check(cache_layer, "cache_layer", torch.bfloat16, 5)
    _check(block_table, "block_table", torch.int32, 2)
    _check(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _check(positions, "positions", torch.int32, 1)
    _check(out, "out", torch.bfloat16, 2)
    page_size = cache_layer.shape[3]
    if head_dim not in PREFILL_HEAD_DIMS or page_size & (page_size - 1) or page_size < 4:
        raise UnsupportedSize(f"the tcgen05 attention takes head sizes {PREFILL_HEAD_DIMS} and power-of-two pages")
    if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim) or q.shape[1] != n_heads * head_dim:
        raise ValueError("q or the cache layer do not match the head sizes")
    if out.shape != q.shape or cu_seqlens.shape[0] != n_seqs + 1 or positions.shape[0] != q.shape[0]:
        raise ValueError("out, cu_seqlens and positions do not match the batch")
    key_splits = int(key_splits)
    if not 1 <= key_splits <= 32:
        raise ValueError(f"key_splits must be 1 to 32, got {key_splits}")
    part_o = part_ml = None
    if key_splits > 1:
        part_o = torch.empty((q.shape[0], n_heads, key_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((q.shape[0], n_heads, key_splits, 2), dtype=torch.float32, device=q.device)
    lib.call("pyre_attention_prefill_tc", q.data_ptr(), cache_layer.data_ptr(), out.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), cu_seqlens.data_ptr(), positions.data_ptr(), q.shape[0], int(n_long_tokens), n_seqs,
             n_heads, n_kv_heads, head_dim, page_size, cache_layer.shape[0], int(window or 0), float(scale), int(min_len),
             key_splits, _ptr(part_o), _ptr(part_ml), device_error_flag(q.device).data_ptr(), _stream())
    return out


def paged_attention_bf16(ctx, q: torch.Tensor, cache_layer: torch.Tensor, block_table: torch.Tensor, n_heads: int,
                         n_kv_heads: int, head_dim: int, scale: float, window: "int | None") -> torch.Tensor:
    """Attention of a whole step in bfloat16: entries with many tokens go to the
    prompt-portion kernel, the others (decoded tokens, short portions) to the split-KV kernel."""
    lens = ctx.cu_seqlens_host[1:] - ctx.cu_seqlens_host[:-1]
    page_size = cache_layer.shape[3]
    use_tc = USE_TC_ATTENTION and head_dim in PREFILL_HEAD_DIMS and page_size & (page_size - 1) == 0 and page_size >= 4
    min_len = TC_ATTENTION_MIN_LEN if use_tc else PREFILL_MIN_LEN
    long_mask = lens >= min_len if head_dim in PREFILL_HEAD_DIMS else lens < 0
    n_long = int(lens[long_mask].sum())
    n_short_seqs = int((~long_mask).sum())
    out = torch.empty_like(q)
    if n_long and use_tc:
        long_lens, long_starts = lens[long_mask], ctx.start_pos_host[long_mask]
        q_tiles = -(-long_lens // 128)
        # key tiles of 64 that a query tile walks, averaged over the tiles: from position 0 (or the window's start)
        # to the tile's last row
        keys = long_starts + long_lens / 2.0 + 64.0
        if window:
            keys = keys.clip(max=window + 192.0)
        mean_tiles = float((keys / 64.0 * q_tiles).sum() / q_tiles.sum())
        key_splits = prefill_key_splits(int(q_tiles.sum()) * n_heads, mean_tiles, q.shape[0], n_heads, head_dim)
        attention_prefill_tc(q, cache_layer, block_table, ctx.cu_seqlens, ctx.positions, ctx.num_seqs, n_long, n_heads,
                             n_kv_heads, head_dim, scale, window, out, min_len, key_splits)
    elif n_long:
        attention_prefill(q, cache_layer, block_table, ctx.cu_seqlens, ctx.positions, ctx.num_seqs, n_long, n_heads,
                          n_kv_heads, head_dim, scale, window, out)
    if n_short_seqs:
        n_short = ctx.num_tokens - n_long
        short_ctx = int((ctx.start_pos_host + lens)[~long_mask].max())
        tpg = max(1, 16 // min(n_heads // n_kv_heads, 16))
        groups = int((-(-lens[~long_mask] // tpg)).sum())
        splits = attention_splits(n_short, n_short_seqs, n_heads, n_kv_heads, short_ctx, window, groups)
        uniform = int(lens[0]) if not n_long and bool((lens == lens[0]).all()) else 0
        paged_attention_mma(q, cache_layer, block_table, ctx.cu_seqlens, ctx.positions, ctx.num_seqs, n_heads,
                            n_kv_heads, head_dim, scale, window, splits, out=out,
                            max_len=min_len - 1 if n_long else 0, uniform_len=uniform)
    return out


def sgemm_nt(a: torch.Tensor, w: torch.Tensor, bias: "torch.Tensor | None" = None,
             out: "torch.Tensor | None" = None) -> torch.Tensor:
    """C = A W^T (+ bias) in IEEE fp32 on the CUDA cores; a [M, K], w [N, K]."""
    for t, n in ((a, "a"), (w, "w")):
        if not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{n} must be a CUDA float32 matrix with contiguous rows")
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise ValueError(f"inner sizes differ: a is [{M}, {K}], w is [{N}, {K2}]")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    lib.call("pyre_sgemm_nt", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
             _ptr(bias), M, N, K, _stream())
    return out


_error_flags: dict = {}


def device_error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels raise when a bounded wait runs out or an index is out of range."""
    key = (device.index if isinstance(device, torch.device) else torch.device(device).index) or 0
    flag = _error_flags.get(key)
    if flag is None:
        flag = torch.zeros(1, dtype=torch.int32, device=device)
        _error_flags[key] = flag
    return flag


DEVICE_ERROR_MESSAGES = {
    1: "a kernel met an index outside its range (token id outside the vocabulary)",
    2: "a tensor-core GEMM gave up waiting on its pipeline (bounded wait ran out)",
    3: "the attention kernel gave up waiting for a tile copy (bounded wait ran out)",
    4: "the tcgen05 attention kernel gave up waiting on its pipeline (bounded wait ran out)",
    5: "the tcgen05 attention kernel found its shared memory misaligned",
    6: "a kernel met a cache page or slot outside the pool (debug checks): a block table or slot mapping names "
       "a page that was given back or never existed",
}


def device_error_message(code: int) -> str:
    """What a value of the device's error word means."""
    return DEVICE_ERROR_MESSAGES.get(int(code), f"a kernel raised error code {int(code)}")


def check_device_errors(device="cuda") -> None:
    flag = device_error_flag(device)
    code = int(flag.item())
    if code:
        flag.zero_()
        counters = _fix_counters.get(torch.device(device).index or 0)
        if counters is not None:
            counters.zero_()      # a product that gave up may have left arrivals uncounted
        raise lib.KernelError(device_error_message(code))


def tc_gemm_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The TMA-fed tcgen05 kernel takes bf16 operands whose rows are 16-byte multiples and 16-byte aligned."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


CTA_PAIRS = True     # prompt portions: two CTAs of a cluster share each 256-row tile (tcgen05 cta_group::2)


def tc_gemm_plan(M: int, N: int, K: int) -> tuple[bool, int, int]:
    """(weights_as_rows, bn, splits) for y[M, N] = a[M, K] w[N, K]^T.

    Up to 128 tokens the weights take the 128-row side of the MMA and the tokens the
    narrow side (bn = tokens rounded up to 16/32/64/128); K is split so that about one
    CTA lands on every SM, each split keeping at least four 64-wide K blocks.  Beyond
    that the tokens take the rows and 128 to 256 output features form a tile, whichever
    width fills the rounds of the persistent CTAs best."""
    _SM_COUNT = sm_count()
    kb = -(-K // 64)
    if M <= 128 or N % 8:
        bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128 if M <= 128 else 256
        tiles = -(-N // 128) * -(-M // bn)
        splits = max(1, min(_SM_COUNT // tiles if tiles < _SM_COUNT else 1, kb // 4, 16))
        # 33 to 128 tokens and few tiles (a split K): one 128-row tile of tokens against 128 weight rows per CTA, the
        # same tiles and splits with the operands' roles exchanged, is faster: the narrow operand then costs 16 KB per K
        # block whatever the token count.  Timed alone at 128 tokens (28 weight matrices in turn): down 34.4 -> 30.4 us,
        # q/k/v 16.6 -> 12.2, output 15.3 -> 11.3; the decode step of 128 requests 7.03 -> 6.66 ms.  From 33 tokens it
        # pays inside the step too since the fp32 partial sums leave the epilogue in whole lines (64 requests 4.71 ->
        # 4.67 ms, 40 requests 4.22 -> 4.19); up to 32 tokens the weights stay on the rows (16 requests: 3.51 against 3.61).
        if 32 < M <= 128 and N % 8 == 0 and splits > 1:
            return False, 128, splits
        return True, bn, splits
    # The tile width and the split of K with the least estimated time on the persistent CTAs (microseconds).
    # Measured on products of 256-2,048 tokens: the main loop is bound by loads, not by the MMAs.  One SM pulls
    # what its ring holds in flight (all stages but the one being multiplied) per memory latency, 1.1 us when
    # many row tiles share each weight tile in L2 and 1.6 us when few do; all SMs together pull about 18 TB/s
    # from L2 into shared memory.  Wide tiles move the fewest bytes, narrow ones fill the CTAs' rounds better,
    # and a split K fills the SMs when there are few tiles (512 tokens x 3,584 features over K = 18,944:
    # 224 wide with K in two takes 63 us, 112 tiles of 128 take 88 us).
    # With CTA pairs (two CTAs of a cluster on a 256-row tile, each loading half of the tile's weight rows) an SM
    # loads 128 (128 + bn / 2) bytes per K block, its ring is deeper, and the workers are the 74 pairs.
    pair = CTA_PAIRS
    workers = _SM_COUNT // 2 if pair else _SM_COUNT
    rows = -(-M // (256 if pair else 128))
    latency = 1.7 - 0.035 * min(-(-M // 128), 16)
    widths = ((256, 6), (224, 6), (208, 7), (192, 7), (160, 7), (128, 8)) if pair else \
        ((256, 4), (224, 5), (208, 5), (192, 5), (160, 5), (128, 6))
    best = [None, None]      # without and with a split K
    for cand, stages in widths:
        if cand > 128 and N < cand:
            continue
        cols = -(-N // cand)
        nbytes = ((256 + cand) if pair else (128 + cand)) * 128       # one K block of both operands, per worker
        per_block = max(cand * 2 / 1900.0, latency / (stages - 1))
        for sp in (1, 2, 3, 4):
            if sp > 1 and kb // sp < 8:
                break
            items = rows * cols * sp
            per_worker = -(-items // workers)
            blocks = -(-kb // sp)
            cost = max(per_worker * blocks * per_block, items * blocks * nbytes / 18e6) \
                + per_worker * (1.5 + cand / 64.0 * (2 if sp > 1 else 1))
            # near-ties go to the wider tile; a split K (fp32 partials, estimated less surely) has to gain a tenth
            if best[sp > 1] is None or cost < best[sp > 1][0] * 0.98:
                best[sp > 1] = (cost, cand, sp)
    whole, split = best
    if split is not None and split[0] < 0.9 * whole[0]:
        return False, split[1], split[2]
    return False, whole[1], whole[2]


GATED_BLOCK = 64     # gate and up rows of a fused feed-forward weight alternate in blocks of this many features


_MAX_FIX_TILES = 4096       # arrival counters per device: tiles of 128 features of one folded product
_fix_counters: dict = {}


def _tile_counters(device) -> torch.Tensor:
    """Arrival counters of the products with a fix-up (zero between launches: the kernel resets what it counts)."""
    key = torch.device(device).index or 0
    c = _fix_counters.get(key)
    if c is None:
        c = _fix_counters[key] = torch.zeros(_MAX_FIX_TILES, dtype=torch.int32, device=device)
    return c


def _scale_fields(fx: "lib.GemmFix", x: "ScaledRows") -> None:
    fx.scale_ssq, fx.scale_tiles = x.ssq.data_ptr(), x.ssq.shape[0]
    fx.scale_n, fx.scale_eps = float(x.rows.shape[1]), x.eps


def gemm_tc(x: "torch.Tensor | ScaledRows", w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
            plan: "tuple[bool, int, int] | None" = None, reduce: bool = True, gated: bool = False,
            pair: "bool | None" = None, checked: bool = False) -> torch.Tensor:
    """y = x w^T on the tensor cores (tcgen05, TMEM accumulators, TMA-fed), bf16 in, fp32 accumulate.

    With a split K the kernel leaves fp32 partial sums [splits, M, N]; ``reduce`` adds
    them up here (fixed order) and converts to ``out_dtype``.  ``reduce=False`` returns them
    as ``PartialSums`` for a consumer kernel that adds them itself.

    ``gated``: w holds gate and up rows alternating in blocks of ``GATED_BLOCK`` features; the
    result is silu(x gate^T) * (x up^T), [M, N / 2] bf16.  The activation runs in the product's
    epilogue (whole tiles, one split: the usual case in both orientations), otherwise after it.

    ``x`` may be ``ScaledRows``: the result rows are scaled by the tokens' 1/rms in the epilogue, before the
    activation of a gated product."""
    scaled = x if isinstance(x, ScaledRows) else None
    if scaled is not None:
        x = scaled.rows
    if not checked and not tc_gemm_supported(x, w):      # ``checked``: the caller has asked already
        raise UnsupportedSize("gemm_tc needs bf16 operands with K and leading dimensions that are multiples of 8")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise ValueError(f"inner sizes differ: x is [{M}, {K}], w is [{N}, {K2}]")
    weights_as_rows, bn, splits = plan or tc_gemm_plan(M, N, K)
    if gated and plan is None and M == 128 and N % 256 == 0:
        # exactly 128 tokens: 58.6 us with the weights on the rows, 52.4 so; with 72-120 tokens (a tile of token rows
        # that is not full) this orientation takes 66 us and the other 54-58
        weights_as_rows, bn, splits = False, 256, 1
    if scaled is not None and weights_as_rows and (M > bn or bn > 128):      # more than one tile of at most 128 tokens on the narrow side: not served
        x, scaled = materialize(scaled), None
    splits = max(1, min(splits, -(-K // 64)))
    if pair is None:
        pair = CTA_PAIRS
    pair = int(bool(pair) and not weights_as_rows and M > 128 and bn in (128, 160, 192, 208, 224, 256))
    err = device_error_flag(x.device)
    fx = None
    if scaled is not None:
        fold = lib.GemmFix()
        _scale_fields(fold, scaled)
        fx = ctypes.byref(fold)

    if gated:
        if N % (2 * GATED_BLOCK) or out_dtype != torch.bfloat16:
            raise UnsupportedSize("a gated product needs whole blocks of gate and up rows and a bfloat16 result")
        if not weights_as_rows and plan is None and N % 256 == 0:
            bn, splits = 256, 1      # the fused activation needs whole 256-wide tiles and saves more than a better fit
        if not weights_as_rows and bn == 256 and splits == 1 and N % 256 == 0:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
            lib.call("pyre_gemm_tc", x.data_ptr(), M, x.stride(0), w.data_ptr(), N, w.stride(0), K, out.data_ptr(), 0,
                     N // 2, 1, 0, 1, bn, 0, 1, pair, err.data_ptr(), fx, _stream())
            return out
        if weights_as_rows and bn <= 128 and splits == 1 and N % 128 == 0:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
            lib.call("pyre_gemm_tc", w.data_ptr(), N, w.stride(0), x.data_ptr(), M, x.stride(0), K, out.data_ptr(), 0,
                     1, N // 2, 0, 1, bn, 1, 1, 0, err.data_ptr(), fx, _stream())
            return out
        return silu_mul(gemm_tc(scaled if scaled is not None else x, w, torch.bfloat16, (weights_as_rows, bn, splits), pair=bool(pair)),
                        block=GATED_BLOCK)
    if splits == 1 and reduce:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        target, split_stride = out, 0
    else:
        target = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        split_stride = M * N
    f32 = int(target.dtype == torch.float32)
    if weights_as_rows:
        lib.call("pyre_gemm_tc", w.data_ptr(), N, w.stride(0), x.data_ptr(), M, x.stride(0), K, target.data_ptr(), f32,
                 1, N, split_stride, splits, bn, 1, 0, 0, err.data_ptr(), fx, _stream())
    else:
        lib.call("pyre_gemm_tc", x.data_ptr(), M, x.stride(0), w.data_ptr(), N, w.stride(0), K, target.data_ptr(), f32,
                 N, 1, split_stride, splits, bn, 0, 0, pair, err.data_ptr(), fx, _stream())
    if target.dim() == 2:
        return target
    if not reduce:
        return PartialSums(target, out_dtype)
    return materialize(PartialSums(target, out_dtype))


def _launch_with_fixup(prod: DeferredProduct, fx: "lib.GemmFix", rows_out: "torch.Tensor | None" = None,
                       row_plan: "tuple[bool, int, int] | None" = None) -> None:
    """The product of a ``DeferredProduct`` with work folded in.  Few tokens (weights on the MMA's rows, all tokens
    in one tile, K split as the plan says): fp32 partial sums that only the kernel's own fix-up reads.  Many tokens
    (tokens on the rows, one split): the epilogue itself folds, and what it stores is ``rows_out``."""
    x = prod.x
    if isinstance(x, ScaledRows):
        _scale_fields(fx, x)
        x = x.rows
    w = prod.w
    M, K = x.shape
    N = w.shape[0]
    weights_as_rows, bn, splits = row_plan or tc_gemm_plan(M, N, K)
    if M <= 128 and not weights_as_rows:
        # the fix-up lives in the orientation with the weights on the rows; the same tiles and splits serve it
        weights_as_rows, bn = True, 128
    err = device_error_flag(x.device).data_ptr()
    with lib.section(prod.section):
        if weights_as_rows:
            splits = max(1, min(splits, -(-K // 64)))
            parts = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
            fx.tile_counters = _tile_counters(x.device).data_ptr()
            lib.call("pyre_gemm_tc", w.data_ptr(), N, w.stride(0), x.data_ptr(), M, x.stride(0), K, parts.data_ptr(), 1,
                     1, N, M * N, splits, bn, 1, 0, 0, err, ctypes.byref(fx), _stream())
        else:
            if splits != 1 or rows_out is None:
                raise UnsupportedSize("a product of many tokens folds only with one split and the residual fix-up")
            pair = int(CTA_PAIRS and bn in (128, 160, 192, 208, 224, 256))
            lib.call("pyre_gemm_tc", x.data_ptr(), M, x.stride(0), w.data_ptr(), N, w.stride(0), K, rows_out.data_ptr(), 0,
                     N, 1, 0, 1, bn, 0, 0, pair, err, ctypes.byref(fx), _stream())


def folds_residual(M: int, N: int, K: int) -> bool:
    """Does a product of this shape take the residual add and the next norm's preparation as folded work?  Very few
    tokens (the fix-up of the last CTA per tile), or many tokens in one split (the epilogue's threads own token rows)."""
    if not FOLD_SMALL_KERNELS or N % 8:
        return False
    if M <= FOLD_MAX_TOKENS:
        return True
    if M <= 128:
        return False
    weights_as_rows, _bn, splits = tc_gemm_plan(M, N, K)
    return not weights_as_rows and splits == 1


def rope_fold_width(N: int, head_dim: int) -> int:
    """The tile width with which a q/k/v product of many tokens carries bias, rotary and the cache write in its
    epilogue (tiles of whole heads), or 0."""
    for bn in (256, 128):
        if N % bn == 0 and bn % head_dim == 0 and head_dim % 32 == 0:
            return bn
    return 0


def folds_rope(M: int, N: int, K: int, head_dim: int) -> bool:
    """Does the stacked q/k/v product of this shape take bias, rotary and the paged write as folded work?  Very few
    tokens (the fix-up of the last CTA per tile), or a prompt portion whose plan is one split of the row store."""
    if not FOLD_SMALL_KERNELS or N % 8:
        return False
    if M <= FOLD_MAX_TOKENS:
        return True
    if M <= 128 or not rope_fold_width(N, head_dim):
        return False
    weights_as_rows, _bn, splits = tc_gemm_plan(M, N, K)
    return not weights_as_rows and splits == 1


def gemm_residual_norm(prod: DeferredProduct, x: torch.Tensor, weight: torch.Tensor, eps: float) -> ScaledRows:
    """x += prod (the fp32 residual stream, in place), and the activations of the RMSNorm that follows as
    ``ScaledRows``: one kernel, the product; the CTA that finishes a tile of 128 features last adds the splits'
    partial sums and the residual, stores bf16(x * weight) and the tile's sums of squares per token."""
    T, H = x.shape
    rows = torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
    ssq = torch.empty((-(-H // 128), T), dtype=torch.float32, device=x.device)
    fx = lib.GemmFix()
    fx.fix = 1
    fx.resid, fx.norm_w, fx.h_out, fx.ssq_out = x.data_ptr(), weight.data_ptr(), rows.data_ptr(), ssq.data_ptr()
    if T > 128:
        # tokens on the rows: a tile is up to 256 features wide, so the sums of squares come per such tile
        _rows, bn, _splits = tc_gemm_plan(T, H, prod.x.shape[1])
        ssq = torch.empty((-(-H // bn), T), dtype=torch.float32, device=x.device)
        fx.ssq_out = ssq.data_ptr()
    _launch_with_fixup(prod, fx, rows)
    return ScaledRows(rows, ssq, eps)


def gemm_rope_write(prod: DeferredProduct, bias, cos, sin, cache_layer, slot_mapping, n_heads: int, n_kv_heads: int,
                    head_dim: int, rotary_dim: int, page_size: int) -> torch.Tensor:
    """The stacked q/k/v projection with bias, rotary and the paged K/V write as its fix-up (what
    ``qkv_rope_write`` does in a kernel of its own); returns the queries [T, nh * hd]."""
    T = prod.shape[0]
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    if rotary_dim:
        _check(cos, "cos", torch.float32, 2)
        _check(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, rotary_dim // 2) or tuple(sin.shape) != (T, rotary_dim // 2):
            raise ValueError(f"cos/sin must be [{T}, {rotary_dim // 2}], got {tuple(cos.shape)}")
    q_out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=prod.device)
    fx = lib.GemmFix()
    fx.fix = 2
    fx.bias = _ptr(bias)
    fx.cos_t, fx.sin_t = (_ptr(cos), _ptr(sin)) if rotary_dim else (None, None)
    fx.q_out = q_out.data_ptr()
    fx.nh, fx.nkv, fx.hd, fx.rot, fx.page_size = n_heads, n_kv_heads, head_dim, rotary_dim, page_size
    if cache_layer is not None:
        _check(cache_layer, "cache_layer", torch.bfloat16, 5)
        if tuple(cache_layer.shape[1:]) != (2, n_kv_heads, page_size, head_dim):
            raise ValueError(f"cache layer shape {tuple(cache_layer.shape)} does not match "
                             f"[pages, 2, {n_kv_heads}, {page_size}, {head_dim}]")
        _check(slot_mapping, "slot_mapping", torch.int32, 1)
        if slot_mapping.shape[0] != T:
            raise ValueError("slot_mapping must have one entry per token")
        fx.kv_cache, fx.slot_mapping, fx.n_pages = cache_layer.data_ptr(), slot_mapping.data_ptr(), cache_layer.shape[0]
    if T > 128:
        # tokens on the rows: the epilogue thread that owns a token row rotates and stores whole heads
        _launch_with_fixup(prod, fx, q_out, (False, rope_fold_width(prod.shape[1], head_dim), 1))
    else:
        _launch_with_fixup(prod, fx)
    return q_out


USE_TC_GEMM = True


# Very few tokens (a decode step of one to four requests): residual add + norm and bias + rotary + K/V write run as
# fix-ups of the products before them instead of kernels of their own.  Measured inside whole decode steps of the 7B
# shape: 4 % faster at one request; at eight requests the fix-up's chain of global round trips (store, fence, arrival
# counter, reload) is longer than the small kernel it replaces, and at 64 its loop over the tokens in the one CTA per
# tile that arrives last costs several times what the norm kernel's one CTA per token does.
FOLD_SMALL_KERNELS = True
FOLD_MAX_TOKENS = 4


def linear(x: "torch.Tensor | ScaledRows", w: torch.Tensor, out_dtype: "torch.dtype | None" = None, partials_ok: bool = False,
           deferred_ok: "bool | str | tuple" = False):
    """y = x W^T for a weight in the linear-layer layout [out, in].

    float32: the package's own fp32 kernel (no reduced-precision matrix mode).
    bfloat16: the package's tcgen05 kernel (``gemm_tc``); rows that are no 16-byte multiple
    (K not a multiple of 8) go to a library product instead, as the reference uses a library
    for every projection.  ``out_dtype=torch.float32`` keeps the accumulator's precision
    (used for the logits).  ``partials_ok``: the caller's consumer adds split-K partial
    sums itself, so a ``PartialSums`` may come back instead of a tensor.  ``deferred_ok``: the caller's
    consumer is one of the kernels that take a ``DeferredProduct`` (the built-in norm, ``qkv_rope_write``) or
    calls ``materialize``; for very few tokens (``FOLD_MAX_TOKENS``) the product is then not launched here.
    ``deferred_ok="residual"`` says that the consumer is the norm (the product is a branch output): then a product
    of many tokens in one split is deferred too, since its epilogue can fold the residual add (``folds_residual``).
    ``deferred_ok=("rope", head_dim)``: the consumer is a position encoding that may fold bias, rotation and the cache
    write into the stacked q/k/v product (``folds_rope``)."""
    if x.dtype == torch.float32:
        return sgemm_nt(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ValueError(f"linear: unsupported dtypes {x.dtype} x {w.dtype}")
    rows = x.rows if isinstance(x, ScaledRows) else x
    if USE_TC_GEMM and tc_gemm_supported(rows, w):
        if deferred_ok and FOLD_SMALL_KERNELS and out_dtype in (None, torch.bfloat16) and w.shape[0] % 4 == 0:
            M = rows.shape[0]
            if M <= FOLD_MAX_TOKENS or (deferred_ok == "residual" and folds_residual(M, w.shape[0], w.shape[1])) or \
                    (isinstance(deferred_ok, tuple) and deferred_ok[0] == "rope" and folds_rope(M, w.shape[0], w.shape[1], deferred_ok[1])):
                return DeferredProduct(x, w, torch.bfloat16)
        return gemm_tc(x, w, out_dtype or torch.bfloat16, reduce=not partials_ok, checked=True)
    x = materialize(x)
    if out_dtype is None or out_dtype == torch.bfloat16:
        if partials_ok:     # the consumer adds fp32 partial sums: hand it the accumulator unrounded, as one part
            return PartialSums(torch.mm(x, w.t(), out_dtype=torch.float32).unsqueeze(0), torch.bfloat16)
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int = GATED_BLOCK) -> torch.Tensor:
    """[2 I, K]: ``block`` gate rows, the up rows of the same features, the next gate rows, ... (I % block == 0)."""
    inter, K = gate.shape
    if up.shape != gate.shape or inter % block:
        raise UnsupportedSize(f"cannot interleave {tuple(gate.shape)} and {tuple(up.shape)} in blocks of {block}")
    return torch.stack([gate.view(inter // block, block, K), up.view(inter // block, block, K)], dim=1).reshape(2 * inter, K).contiguous()


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for the stacked weight of a gated feed-forward: [gates | ups] rows, or
    (``interleaved``) blocks of ``GATED_BLOCK`` gate rows and up rows in turn, which lets the bfloat16
    tensor-core product apply the activation in its epilogue."""
    rows = x.rows if isinstance(x, ScaledRows) else x
    if interleaved and x.dtype == torch.bfloat16 and USE_TC_GEMM and tc_gemm_supported(rows, w_gate_up):
        return gemm_tc(x, w_gate_up, torch.bfloat16, gated=True, checked=True)
    return silu_mul(linear(x, w_gate_up), block=GATED_BLOCK if interleaved else 0)
