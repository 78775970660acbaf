"""The engine against the plain implementation, through the replay loop: each request
alone and whole; most of it in one step and the last 32 tokens one by one; in portions
of changing size down to two tokens; and mixed, up to four live requests with so few
pages that they are used again (pages that go back to the pool are filled with NaN
first, so a stale read shows).  In 32-bit and in bfloat16, for three tiny
configurations that differ in every size."""

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

# Tolerances.  float32: the engine and the plain implementation differ only in the order
# of fp32 sums.  bfloat16: the yardstick is the reference's own arithmetic in that dtype.
# The plain implementation is run twice on the bf16-rounded weights, in fp32 ("truth")
# and with every tensor in bfloat16 as the reference would run it (pyre/loader.py:74
# casts the whole model to one dtype).  The engine passes if, over a configuration's
# requests, its rms error against the truth is no larger than that of the bf16 run, and
# if no single logit is off by more than 8 times that rms (a wrong key, page or position
# moves logits by their whole spread, 50 to 100 times the rms).
TOL = {"float32": dict(rtol=2e-4, atol=2e-5)}
BF16_MAX_OVER_RMS = 8.0

LENGTHS = {"A": [5, 17, 33, 70, 100], "B": [1, 7, 40, 63, 100, 131], "C": [3, 64, 97]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for n, (name, raw) in enumerate(H.TINY.items()):
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        H.make_model_dir(d, raw, seed=100 + n)
        reqs = {f"{name}{i}": H.random_ids(raw["vocab_size"], L, seed=7 * n + i)
                for i, L in enumerate(LENGTHS[name])}
        plain = {dt: {rid: H.plain_logits(d, ids, bf16_weights=(dt == "bfloat16")) for rid, ids in reqs.items()}
                 for dt in ("float32", "bfloat16")}
        sq, cnt = 0.0, 0
        for rid, ids in reqs.items():
            e = H.plain_logits_in_bf16(d, ids) - plain["bfloat16"][rid]
            sq, cnt = sq + float((e.astype(np.float64) ** 2).sum()), cnt + e.size
        plain["bf16_rms"] = (sq / cnt) ** 0.5
        out[name] = (d, reqs, plain)
    return out


def compare(got: dict, want: dict, dtype: str, what: str, bf16_rms: float = 0.0):
    assert set(got) == set(want), f"{what}: requests differ"
    sq, cnt = 0.0, 0
    for rid in want:
        g, w = got[rid], want[rid]
        assert g.shape == w.shape, f"{what} {rid}: shape {g.shape} != {w.shape}"
        assert np.isfinite(g).all(), f"{what} {rid}: non-finite logits at rows {np.unique(np.where(~np.isfinite(g))[0])[:8]}"
        err = np.abs(g - w)
        if dtype == "float32":
            bound = TOL[dtype]["atol"] + TOL[dtype]["rtol"] * np.abs(w)
        else:
            bound = np.full_like(w, BF16_MAX_OVER_RMS * bf16_rms)
            sq, cnt = sq + float((err.astype(np.float64) ** 2).sum()), cnt + err.size
        bad = err > bound
        if bad.any():
            row = int(np.where(bad.any(axis=1))[0][0])
            raise AssertionError(f"{what} {rid} ({dtype}): first wrong token at position {row} of {g.shape[0]}; "
                                 f"max |diff| there {err[row].max():.3e}, bound {bound[row].max():.3e}, "
                                 f"overall max {err.max():.3e}, logits std {w.std():.3f}")
    if dtype == "bfloat16":
        rms = (sq / cnt) ** 0.5
        assert rms <= bf16_rms, (f"{what} (bfloat16): rms error {rms:.3e} of the engine exceeds the "
                                 f"{bf16_rms:.3e} of the reference's arithmetic in bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole(models, name, dtype):
    d, reqs, plain = models[name]
    steps = H.trace_whole(reqs)
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), H.PAGE_SIZE[name])
    compare(got, plain[dtype], dtype, "whole", plain["bf16_rms"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_one_by_one(models, name, dtype):
    d, reqs, plain = models[name]
    steps = []
    for rid, ids in reqs.items():
        steps += H.trace_decode_tail(rid, ids, 32, first_step=len(steps))
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), H.PAGE_SIZE[name])
    compare(got, plain[dtype], dtype, "decode tail", plain["bf16_rms"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions(models, name, dtype):
    d, reqs, plain = models[name]
    steps = []
    for k, (rid, ids) in enumerate(reqs.items()):
        sizes = [[2, 9, 3, 17, 2, 31], [5, 2, 16, 8], [24, 2, 2, 7]][k % 3]
        steps += H.trace_portions(rid, ids, sizes, first_step=len(steps))
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), H.PAGE_SIZE[name])
    compare(got, plain[dtype], dtype, "portions", plain["bf16_rms"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_with_page_reuse(models, name, dtype):
    d, reqs, plain = models[name]
    # every request twice under different ids, so that later ones land on pages the earlier ones gave back
    many = {}
    for rep in range(2):
        for rid, ids in reqs.items():
            many[f"{rid}r{rep}"] = ids
    steps = H.trace_mixed(many, seed=11, max_live=4)
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), H.PAGE_SIZE[name])
    want = {f"{rid}r{rep}": plain[dtype][rid] for rep in range(2) for rid in reqs}
    compare(got, want, dtype, "mixed", plain["bf16_rms"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cutting_does_not_change_logits(models, dtype):
    """The same request whole, token by token and in portions gives logits that agree far
    more closely than the engine agrees with the plain implementation."""
    d, reqs, _ = models["B"]
    rid, ids = list(reqs.items())[-1]
    runs = []
    for steps in (H.trace_whole({rid: ids}), H.trace_decode_tail(rid, ids, len(ids) - 1),
                  H.trace_portions(rid, ids, [2, 13, 5, 32])):
        runs.append(H.run_trace_in_process(d, dtype, steps, 256, 8)[rid])
    tol = 1e-5 if dtype == "float32" else 2e-2
    for other in runs[1:]:
        assert np.abs(other - runs[0]).max() <= tol * max(1.0, np.abs(runs[0]).max())
