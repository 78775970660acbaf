"""The engine against the plain implementation, through the replay loop: each request
alone and whole; most of it in one step and the last 32 tokens one by one; in portions
of changing size down to two tokens; and mixed, up to four live requests with so few
pages that they are used again (pages that go back to the pool are filled with NaN
first, so a stale read shows).  In 32-bit and in bfloat16, for four tiny
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

LENGTHS = {"A": [5, 17, 33, 70, 100], "B": [1, 7, 40, 63, 100, 131], "C": [3, 64, 97], "D": [2, 130, 165, 300]}


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
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole(models, name, dtype):
    d, reqs, plain = models[name]
    steps = H.trace_whole(reqs)
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), H.PAGE_SIZE[name])
    compare(got, plain[dtype], dtype, "whole", plain["bf16_rms"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_last_32_one_by_one(models, name, dtype):
    d, reqs, plain = models[name]
    steps = []
    for rid, ids in reqs.items():
        steps += H.trace_decode_tail(rid, ids, 32, first_step=len(steps))
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), H.PAGE_SIZE[name])
    compare(got, plain[dtype], dtype, "decode tail", plain["bf16_rms"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions(models, name, dtype):
    d, reqs, plain = models[name]
    steps = []
    for k, (rid, ids) in enumerate(reqs.items()):
        sizes = [[2, 9, 3, 17, 2, 31], [5, 2, 16, 8], [24, 2, 2, 7]][k % 3]
        steps += H.trace_portions(rid, ids, sizes, first_step=len(steps))
    got = H.run_trace_in_process(d, dtype, steps, H.max_live_tokens(steps), H.PAGE_SIZE[name])
    compare(got, plain[dtype], dtype, "portions", plain["bf16_rms"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
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


def random_config(seed: int) -> tuple[dict, int, list[int]]:
    """A configuration, a page size and request lengths drawn from a seed: head sizes in steps of 16 up to 256, any
    number of heads and groups, widths and vocabularies that are no power of two."""
    rng = np.random.default_rng(seed)
    nkv, grp = int(rng.integers(1, 5)), int(rng.integers(1, 8))
    raw = dict(architectures=["Qwen2ForCausalLM"], hidden_size=int(rng.choice([8, 4, 2])) * int(rng.integers(9, 40)),
               intermediate_size=int(rng.choice([8, 2, 16])) * int(rng.integers(11, 50)), num_hidden_layers=int(rng.integers(1, 5)),
               num_attention_heads=nkv * grp, num_key_value_heads=nkv,
               head_dim=int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 160, 256])), vocab_size=int(rng.integers(100, 3000)),
               rope_theta=float(rng.choice([1e4, 1e6, 5e5, 12345.0])), rms_norm_eps=float(rng.choice([1e-6, 1e-5, 2e-6])),
               tie_word_embeddings=bool(rng.integers(0, 2)), max_position_embeddings=2048)
    page = int(rng.choice([64, 16, 128, 32]))
    lengths = [int(x) for x in rng.integers(1, 200, 3)] + [int(rng.integers(300, 700))]
    return raw, page, lengths


@pytest.mark.parametrize("seed", [11, 12, 13, 14])
def test_random_configurations(tmp_path, seed):
    """Sizes other than the three fixed configurations', whole, in portions and mixed.  bfloat16 is judged as above.
    float32 is judged against the plain implementation run in 64-bit: the engine's error is no larger (rms) than
    that of the plain implementation in 32-bit, and no single logit is off by more than twice its largest error."""
    import torch
    from plain import qwen2_plain
    raw, page, lengths = random_config(seed)
    H.make_model_dir(tmp_path, raw, seed=1000 + seed)
    reqs = {f"r{i}": H.random_ids(raw["vocab_size"], L, seed=31 * seed + i) for i, L in enumerate(lengths)}
    portions = []
    for k, (rid, ids) in enumerate(reqs.items()):
        portions += H.trace_portions(rid, ids, [[2, 9, 3, 17, 2, 31], [5, 2, 16, 8], [24, 2, 2, 7], [130, 2, 64, 33]][k % 4],
                                     first_step=len(portions))
    many = {f"{rid}x{rep}": ids for rep in range(2) for rid, ids in reqs.items()}
    traces = {"whole": H.trace_whole(reqs), "portions": portions, "mixed": H.trace_mixed(many, seed=seed, max_live=4)}
    w64 = {k: v.double() for k, v in H.load_plain_weights(tmp_path).items()}
    with torch.inference_mode():
        p64 = {rid: qwen2_plain.forward(ids, w64, raw).numpy() for rid, ids in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        plain = {rid: H.plain_logits(tmp_path, ids, bf16_weights=(dtype == "bfloat16")) for rid, ids in reqs.items()}
        if dtype == "float32":
            e = np.concatenate([(plain[r] - p64[r]).ravel() for r in reqs])
            plain_rms, plain_max = float(np.sqrt((e ** 2).mean())), float(np.abs(e).max())
        else:
            e = np.concatenate([(H.plain_logits_in_bf16(tmp_path, ids) - plain[rid]).ravel() for rid, ids in reqs.items()])
            bf16_rms = float(np.sqrt((e.astype(np.float64) ** 2).mean()))
        for what, steps in traces.items():
            got = H.run_trace_in_process(tmp_path, dtype, steps, H.max_live_tokens(steps, max(64, page)), page)
            mixed = what == "mixed"
            if dtype == "bfloat16":
                want = {f"{rid}x{rep}": plain[rid] for rep in range(2) for rid in reqs} if mixed else plain
                compare(got, want, dtype, f"{what} of {raw}", bf16_rms)
                continue
            want = {f"{rid}x{rep}": p64[rid] for rep in range(2) for rid in reqs} if mixed else p64
            assert set(got) == set(want)
            e = np.concatenate([(got[r].astype(np.float64) - want[r]).ravel() for r in want])
            assert np.isfinite(e).all(), f"{what} of {raw}: non-finite logits"
            rms, worst = float(np.sqrt((e ** 2).mean())), float(np.abs(e).max())
            assert rms <= plain_rms and worst <= 2 * plain_max, \
                f"{what} of {raw} (float32): engine rms {rms:.2e} max {worst:.2e}, plain 32-bit rms {plain_rms:.2e} max {plain_max:.2e}"
