"""The engine at layer sizes at which the fast kernels run, with two layers and a small
vocabulary: the benchmark model's (hidden 3584, 28 query heads over 4 key/value heads of
size 128, intermediate 18944) and those of the reference's own test model
(tests/test_parity.py:26 of the reference: hidden 896, 14 query heads over 2 key/value heads
of size 64, intermediate 4864, tied embeddings).  Here the TMA-fed attention tiles, the
tcgen05 prompt-portion attention, the mma.sync prompt-portion attention and the split-K
tensor-core products run; the tiny configurations never reach those paths.  The oracle is
the plain implementation in fp32; it runs on the GPU here (it is plain torch either way)
because a CPU would need minutes for these widths."""

import numpy as np
import pytest
import torch

import helpers as H
from plain import qwen2_plain

pytestmark = pytest.mark.gpu

SHAPES = {
    "hd128": dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, intermediate_size=18944, num_hidden_layers=2,
                  num_attention_heads=28, num_key_value_heads=4, head_dim=128, vocab_size=4096, rope_theta=1e6,
                  rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096),
    "hd64": dict(architectures=["Qwen2ForCausalLM"], hidden_size=896, intermediate_size=4864, num_hidden_layers=2,
                 num_attention_heads=14, num_key_value_heads=2, head_dim=64, vocab_size=1536, rope_theta=1e6,
                 rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096),
}
BIG = SHAPES["hd128"]
# N(0, 0.02) matrices at the wide shape already give activations of order one; the narrow one needs a little more.
# Only the query/key projections are sharpened so that attention is peaked.
SCALES = {"hd128": dict(sharpen=2.0, matrix_scale=1.0), "hd64": dict(sharpen=3.0, matrix_scale=1.6)}
LENGTHS = {"p": 300, "q": 170, "r": 45, "s": 700}


def plain_on_gpu(d, raw, reqs):
    """{dtype: {request: logits}} and the rms error of the reference's own arithmetic in bfloat16."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    plain = {}
    for dt in ("float32", "bfloat16"):
        w = {k: v.cuda() for k, v in H.load_plain_weights(d, round_matrices_to_bf16=(dt == "bfloat16")).items()}
        with torch.inference_mode():
            plain[dt] = {rid: qwen2_plain.forward(ids, w, raw).cpu().numpy() for rid, ids in reqs.items()}
            if dt == "bfloat16":
                wb = {k: v.to(torch.bfloat16) for k, v in w.items()}
                sq = cnt = 0
                for rid, ids in reqs.items():
                    e = qwen2_plain.forward(ids, wb, raw).float().cpu().numpy() - plain[dt][rid]
                    sq, cnt = sq + float((e.astype(np.float64) ** 2).sum()), cnt + e.size
                plain["bf16_rms"] = (sq / cnt) ** 0.5
                del wb
        del w
    torch.cuda.empty_cache()
    torch.backends.cuda.matmul.allow_tf32 = prev
    return plain


@pytest.fixture(scope="module", params=list(SHAPES))
def big(request, tmp_path_factory):
    name = request.param
    raw = SHAPES[name]
    d = tmp_path_factory.mktemp(f"big_{name}")
    state = H.make_model_dir(d, raw, seed=77, **SCALES[name])
    del state
    reqs = {rid: H.random_ids(raw["vocab_size"], n, seed=k + 1) for k, (rid, n) in enumerate(LENGTHS.items())}
    return d, raw, reqs, plain_on_gpu(d, raw, reqs)


def check(got, want, dtype, bf16_rms, what):
    sq = cnt = 0
    for rid in want:
        g, w = got[rid], want[rid]
        assert g.shape == w.shape and np.isfinite(g).all(), f"{what} {rid}"
        err = np.abs(g - w)
        # float32: sums of up to 18,944 products in another order; bfloat16: the same yardstick as
        # for the tiny models (the reference's own arithmetic in bfloat16, 8 times its rms for one logit)
        bound = (2e-4 + 2e-4 * np.abs(w)) if dtype == "float32" else np.full_like(w, 8.0 * bf16_rms)
        bad = err > bound
        if bad.any():
            row = int(np.where(bad.any(axis=1))[0][0])
            raise AssertionError(f"{what} {rid} ({dtype}): first wrong token at position {row} of {g.shape[0]}, "
                                 f"error {err[row].max():.3e}, bound {bound[row].max():.3e}, logits std {w.std():.3f}")
        sq, cnt = sq + float((err.astype(np.float64) ** 2).sum()), cnt + err.size
    if dtype == "bfloat16":
        assert (sq / cnt) ** 0.5 <= bf16_rms, f"{what}: rms error {(sq / cnt) ** 0.5:.3e} > {bf16_rms:.3e}"


def long_mixed_trace(reqs):
    """Up to four live requests whose prompt portions are 30 to 300 tokens long, so that single steps hold
    a portion for the tcgen05 attention (64 tokens or more), a portion of 32 to 63 tokens and decoded
    tokens together; every request twice, so that pages are used again."""
    many = dict(reqs, **{k + "2": v for k, v in reqs.items()})
    steps = H.trace_mixed(many, seed=3, max_live=4, prefill_head=0.85, portion=(30, 300))
    kinds = [sorted(len(e["tokens"]) for e in st["entries"]) for st in steps]
    assert any(k[0] == 1 and k[-1] >= 64 for k in kinds), "no step mixes a long portion with a decoded token"
    assert any(k[0] == 1 and k[-1] >= 64 and any(32 <= n < 64 for n in k) for k in kinds), \
        "no step holds a long portion, a middle one and a decoded token"
    return steps, many


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_shape_every_way_of_cutting(big, dtype):
    d, raw, reqs, plain = big
    want = plain[dtype]
    short = {k: v for k, v in reqs.items() if k != "s"}
    runs = {
        "whole": (H.trace_whole(reqs), reqs),
        "decode tail": (sum((H.trace_decode_tail(rid, ids, 32, first_step=1000 * n)
                             for n, (rid, ids) in enumerate(reqs.items())), []), reqs),
        "portions": (sum((H.trace_portions(rid, ids, [33, 2, 64, 100, 7], first_step=1000 * n)
                          for n, (rid, ids) in enumerate(reqs.items())), []), reqs),
        "mixed": (H.trace_mixed(dict(short, **{k + "2": v for k, v in short.items()}), seed=5, max_live=3), short),
    }
    for what, (steps, which) in runs.items():
        for n, st in enumerate(steps):
            st["step"] = n
        got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), 16)
        ref = {k: want[k] for k in which}
        if what == "mixed":
            ref.update({k + "2": want[k] for k in which})
        check(got, ref, dtype, plain["bf16_rms"], f"{raw['head_dim']} {what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_beside_decoded_tokens(big, dtype):
    """The scheduler's usual step: long prompt portions beside decoded tokens, in one output tensor
    written by two attention kernels, on exactly as many pages as the live requests need."""
    d, raw, reqs, plain = big
    steps, many = long_mixed_trace(reqs)
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), 16)
    want = {rid: plain[dtype][rid.rstrip("2")] for rid in many}
    check(got, want, dtype, plain["bf16_rms"], f"{raw['head_dim']} long mixed")


def test_long_portions_with_their_keys_in_shares(big, monkeypatch):
    """The same steps with the prompt attention forced to cut every (query tile, head) into three shares of its
    keys (the planner asks for shares only after contexts of thousands of tokens, which these requests do not
    reach): partial outputs, the combining kernel and empty shares inside whole model steps, beside the decode
    kernel that writes the other rows of the same tensor."""
    from pyre_b200.kernels import ops
    d, raw, reqs, plain = big
    calls = []
    monkeypatch.setattr(ops, "prefill_key_splits", lambda *a: calls.append(a) or 3)
    steps, many = long_mixed_trace(reqs)
    got = H.run_trace_in_process(d, "bfloat16", steps, H.max_live_tokens(steps), 16)
    assert calls, "no step reached the tcgen05 prompt attention"
    want = {rid: plain["bfloat16"][rid.rstrip("2")] for rid in many}
    check(got, want, "bfloat16", plain["bf16_rms"], f"{raw['head_dim']} long mixed in shares")


@pytest.mark.parametrize("lookahead", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_returns_the_plain_logits(big, dtype, lookahead):
    """``Engine.generate`` as the benchmark drives it (captured decode steps with padded rows, tokens fed
    on the device, a cache so small that a request is preempted and recomputed): the logits each token
    was sampled from are those of the plain implementation on the same history."""
    from pyre_b200 import Engine, SamplingParams
    d, raw, _reqs, plain = big
    lens = [40, 400, 130, 64, 257, 333, 90]
    prompts = [H.random_ids(raw["vocab_size"], n, seed=500 + n) for n in lens]
    params = [SamplingParams(max_new_tokens=40, return_logits=True, temperature=0.0 if k % 2 else 0.8, seed=k)
              for k in range(len(lens))]
    eng = Engine(d, dtype=dtype, page_size=16, num_pages=64, max_num_seqs=8, max_num_batched_tokens=512,
                 prefill_chunk=256, debug_poison_freed_pages=True, lookahead=lookahead)
    outs = eng.generate(prompts, params)
    assert eng.stats()["preempted"] >= 1
    if dtype == "bfloat16":
        assert eng.stepper.graph_replays > 0
    eng.cache.check()
    assert eng.stats()["pages_free"] == eng.stats()["pages_total"]
    eng.stepper.check_device_errors()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    w = {k: v.cuda() for k, v in H.load_plain_weights(d, round_matrices_to_bf16=(dtype == "bfloat16")).items()}
    got, want = {}, {}
    with torch.inference_mode():
        for k, (p, o) in enumerate(zip(prompts, outs)):
            assert len(o.token_ids) == 40 and o.logits.shape == (40, raw["vocab_size"])
            full = qwen2_plain.forward(list(p) + o.token_ids[:-1], w, raw).cpu().numpy()
            got[k], want[k] = o.logits, full[len(p) - 1:]
            for j, (tok, sp) in enumerate(zip(o.token_ids, [params[k]] * 40)):
                # the engine's own logits give the engine's token
                assert tok == qwen2_plain.sample(torch.from_numpy(o.logits[j]), sp.temperature, sp.seed, j)
    torch.backends.cuda.matmul.allow_tf32 = prev
    check(got, want, dtype, plain["bf16_rms"], f"{raw['head_dim']} generate (lookahead {lookahead})")
