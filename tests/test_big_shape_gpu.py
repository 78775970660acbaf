"""The engine at the layer sizes of the benchmark model (hidden 3584, 28 query heads over 4
key/value heads of size 128, intermediate 18944), with two layers and a small vocabulary:
the sizes at which the TMA-fed attention tiles, the prompt-portion attention kernel and
the split-K tensor-core products run.  The tiny configurations never reach those paths.
The oracle is the plain implementation in fp32; it runs on the GPU here (it is plain torch
either way) because a CPU would need minutes for these widths."""

import numpy as np
import pytest
import torch

import helpers as H
from plain import qwen2_plain

pytestmark = pytest.mark.gpu

BIG = dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, intermediate_size=18944, num_hidden_layers=2,
           num_attention_heads=28, num_key_value_heads=4, head_dim=128, vocab_size=4096, rope_theta=1e6,
           rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    d = tmp_path_factory.mktemp("big_shape")
    # N(0, 0.02) matrices at these widths already give activations of order one; only the
    # query/key projections are sharpened so that attention is peaked
    state = H.make_model_dir(d, BIG, seed=77, sharpen=2.0, matrix_scale=1.0)
    del state
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    reqs = {"p": H.random_ids(BIG["vocab_size"], 300, seed=1), "q": H.random_ids(BIG["vocab_size"], 170, seed=2),
            "r": H.random_ids(BIG["vocab_size"], 45, seed=3)}
    plain = {}
    for dt in ("float32", "bfloat16"):
        w = {k: v.cuda() for k, v in H.load_plain_weights(d, round_matrices_to_bf16=(dt == "bfloat16")).items()}
        with torch.inference_mode():
            plain[dt] = {rid: qwen2_plain.forward(ids, w, BIG).cpu().numpy() for rid, ids in reqs.items()}
            if dt == "bfloat16":
                wb = {k: v.to(torch.bfloat16) for k, v in w.items()}
                sq = cnt = 0
                for rid, ids in reqs.items():
                    e = qwen2_plain.forward(ids, wb, BIG).float().cpu().numpy() - plain[dt][rid]
                    sq, cnt = sq + float((e.astype(np.float64) ** 2).sum()), cnt + e.size
                plain["bf16_rms"] = (sq / cnt) ** 0.5
                del wb
        del w
    torch.cuda.empty_cache()
    torch.backends.cuda.matmul.allow_tf32 = prev
    return d, reqs, plain


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_shape_every_way_of_cutting(big, dtype):
    d, reqs, plain = big
    want = plain[dtype]
    runs = {
        "whole": H.trace_whole(reqs),
        "decode tail": sum((H.trace_decode_tail(rid, ids, 32, first_step=1000 * n)
                            for n, (rid, ids) in enumerate(reqs.items())), []),
        "portions": sum((H.trace_portions(rid, ids, [33, 2, 64, 100, 7], first_step=1000 * n)
                         for n, (rid, ids) in enumerate(reqs.items())), []),
        "mixed": H.trace_mixed(dict(reqs, **{k + "2": v for k, v in reqs.items()}), seed=5, max_live=3),
    }
    for what, steps in runs.items():
        for n, st in enumerate(steps):
            st["step"] = n
        got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), 16)
        ref = want if what != "mixed" else dict(want, **{k + "2": v for k, v in want.items()})
        check(got, ref, dtype, plain["bf16_rms"], what)
