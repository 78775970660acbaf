"""Generation through the Python entry point and the command line: greedy tokens against
the plain implementation, batched against alone, temperature sampling, preemption with
recompute, long decoding, and the first tokens of a sequence."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
from plain import qwen2_plain

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    out = {}
    for n, (name, raw) in enumerate(H.TINY.items()):
        d = tmp_path_factory.mktemp(f"eng_{name}")
        H.make_model_dir(d, raw, seed=300 + n)
        out[name] = d
    return out


def check_greedy_against_plain(d, prompt, generated, dtype, margin):
    """Teacher-forced check: at every generated position the engine's token is the plain
    implementation's argmax (fp32), or within ``margin`` of the best logit (bf16, where
    rounding may flip a near-tie)."""
    ids = list(prompt) + list(generated)
    logits = H.plain_logits(d, ids[:-1], bf16_weights=(dtype == "bfloat16"))
    for k, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + k]
        if dtype == "float32":
            assert tok == int(row.argmax()), f"token {k}: engine {tok}, plain {int(row.argmax())}, margin {np.sort(row)[-1] - np.sort(row)[-2]:.3e}"
        else:
            assert row[tok] >= row.max() - margin, f"token {k}: engine chose {tok} with plain logit {row[tok]:.4f}, best {row.max():.4f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(model_dirs, name, dtype):
    from pyre_b200 import Engine, SamplingParams
    d = model_dirs[name]
    raw = H.TINY[name]
    lens = [5, 17, 33] if name == "A" else [1, 7, 40, 63, 100]
    prompts = [H.random_ids(raw["vocab_size"], L, seed=L) for L in lens]
    eng = Engine(d, dtype=dtype, page_size=H.PAGE_SIZE[name], max_cache_tokens=1024, max_num_seqs=8,
                 max_num_batched_tokens=64, prefill_chunk=24, debug_poison_freed_pages=True)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=16))
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 16 and o.finish_reason == "length"
        check_greedy_against_plain(d, p, o.token_ids, dtype, margin=0.05)
    if dtype == "float32":
        w = H.load_plain_weights(d)
        assert outs[0].token_ids == qwen2_plain.greedy_generate(prompts[0], w, raw, 16)
    eng.cache.check()
    assert eng.stats()["pages_free"] == eng.stats()["pages_total"] and eng.stats()["kernel_launches"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batched_equals_alone_and_temperature_is_per_request(model_dirs, dtype):
    """tests/test_scheduler.py:20-64 of the reference: requests that finish at different
    steps give the tokens they give alone; here also under temperature sampling."""
    from pyre_b200 import Engine, SamplingParams
    d, raw = model_dirs["B"], H.TINY["B"]
    prompts = [H.random_ids(raw["vocab_size"], L, seed=50 + L) for L in (9, 30, 2, 55)]
    params = [SamplingParams(temperature=0.8, seed=11 + i, max_new_tokens=n) for i, n in enumerate((24, 16, 32, 8))]
    kw = dict(dtype=dtype, page_size=8, max_cache_tokens=2048, max_num_seqs=4, max_num_batched_tokens=48, prefill_chunk=24)
    together = Engine(d, **kw).generate(prompts, params)
    one = Engine(d, **kw)
    for p, sp, o in zip(prompts, params, together):
        solo = one.generate([p], sp)[0]
        assert solo.token_ids == o.token_ids
        assert len(o.token_ids) == sp.max_new_tokens
    # another seed gives other tokens; temperature 0 is greedy
    other = one.generate([prompts[0]], SamplingParams(temperature=0.8, seed=999, max_new_tokens=24))[0]
    assert other.token_ids != together[0].token_ids
    # the sampled tokens follow the plain sampler on the plain logits (fp32: exactly)
    if dtype == "float32":
        p, sp, o = prompts[2], params[2], together[2]
        ids = list(p)
        for k, tok in enumerate(o.token_ids[:6]):
            row = torch.from_numpy(H.plain_logits(d, ids)[-1])
            assert tok == qwen2_plain.sample(row, sp.temperature, sp.seed, k)
            ids.append(tok)


def test_eos_stops_and_is_kept(model_dirs):
    from pyre_b200 import Engine, SamplingParams
    d, raw = model_dirs["A"], H.TINY["A"]
    prompt = H.random_ids(raw["vocab_size"], 12, seed=3)
    eng = Engine(d, dtype="float32", max_cache_tokens=512)
    free = eng.generate([prompt], SamplingParams(max_new_tokens=20))[0].token_ids
    eos = free[5]
    first = free.index(eos)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=20, eos_id=eos))[0]
    assert out.token_ids == free[:first + 1] and out.finish_reason == "eos"
    # the reference's two calls: add_request + run
    sid = eng.add_request(prompt, max_new_tokens=7)
    assert eng.run() == {sid: free[:7]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_recomputes_and_keeps_tokens(model_dirs, dtype):
    from pyre_b200 import Engine, SamplingParams
    d, raw = model_dirs["A"], H.TINY["A"]
    prompts = [H.random_ids(raw["vocab_size"], L, seed=70 + L) for L in (30, 28, 26)]
    sp = SamplingParams(max_new_tokens=40, temperature=0.7, seed=5)
    roomy = Engine(d, dtype=dtype, page_size=16, max_cache_tokens=4096, max_num_seqs=4).generate(prompts, sp)
    tight = Engine(d, dtype=dtype, page_size=16, num_pages=9, max_num_seqs=4, debug_poison_freed_pages=True)
    outs = tight.generate(prompts, sp)          # 3 x 70 tokens = 15 pages wanted, 9 there
    assert tight.stats()["preempted"] >= 1
    assert sum(o.preemptions for o in outs) >= 1
    for a, b in zip(roomy, outs):
        if dtype == "float32":
            assert a.token_ids == b.token_ids
        else:
            # a recomputed prefix is rounded differently than the decoded one; tokens agree
            # until rounding flips a near-tie, after which the histories differ legitimately
            assert len(a.token_ids) == len(b.token_ids) == 40
            assert a.token_ids[:4] == b.token_ids[:4]
    tight.cache.check()
    assert tight.stats()["pages_free"] == tight.stats()["pages_total"]


@pytest.mark.parametrize("name", ["A", "B"])
def test_lookahead_gives_the_same_tokens(model_dirs, name):
    """Starting a step before the ids of the step before have reached the host (they are fed on
    the device) changes no token: greedy and temperature requests, ends of sequence (where one token
    too many is computed and dropped), length limits, and preemption in a tight cache, in 32-bit."""
    from pyre_b200 import Engine, SamplingParams
    d, raw = model_dirs[name], H.TINY[name]
    prompts = [H.random_ids(raw["vocab_size"], L, seed=40 + L) for L in (30, 3, 17, 26, 9)]
    kw = dict(dtype="float32", page_size=H.PAGE_SIZE[name], max_num_seqs=4, max_num_batched_tokens=24, prefill_chunk=16)
    probe = Engine(d, max_cache_tokens=2048, lookahead=False, **kw)
    free = probe.generate(prompts, SamplingParams(max_new_tokens=24))
    params = [SamplingParams(max_new_tokens=24, eos_id=free[0].token_ids[6]),        # ends early
              SamplingParams(max_new_tokens=1),                                     # one token only
              SamplingParams(max_new_tokens=24, temperature=0.8, seed=11),
              SamplingParams(max_new_tokens=13, eos_id=free[3].token_ids[12]),       # end of sequence on the last allowed token
              SamplingParams(max_new_tokens=24, temperature=1.3, seed=5, eos_id=free[4].token_ids[2])]
    long_prompts = [H.random_ids(raw["vocab_size"], L, seed=70 + L) for L in (30, 28, 26)]
    long_params = [SamplingParams(max_new_tokens=40, temperature=0.7, seed=5)] * 3
    scenarios = [(prompts, params, dict(max_cache_tokens=2048)),
                 # 3 x 70 tokens wanted, about 60 % of the pages there: requests are preempted and recomputed
                 (long_prompts, long_params, dict(num_pages={16: 9, 8: 18}[H.PAGE_SIZE[name]], debug_poison_freed_pages=True))]
    for ps, sps, cache_kw in scenarios:
        plain = Engine(d, lookahead=False, **cache_kw, **kw)
        ahead = Engine(d, lookahead=True, **cache_kw, **kw)
        a, b = plain.generate(ps, sps), ahead.generate(ps, sps)
        assert [o.token_ids for o in a] == [o.token_ids for o in b]
        assert [o.finish_reason for o in a] == [o.finish_reason for o in b]
        if "num_pages" in cache_kw:
            assert ahead.stats()["preempted"] >= 1
        else:
            assert a[0].finish_reason == "eos" and len(a[1].token_ids) == 1
        for eng in (plain, ahead):
            eng.cache.check()
            assert eng.stats()["pages_free"] == eng.stats()["pages_total"] and not eng.has_unfinished()
        ahead.stepper.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, dtype):
    """300 decoded tokens across many pages, checked teacher-forced against the plain
    implementation at the end (a drift or a page fault late in a sequence shows here)."""
    from pyre_b200 import Engine, SamplingParams
    d, raw = model_dirs["B"], H.TINY["B"]
    prompt = H.random_ids(raw["vocab_size"], 11, seed=1)
    eng = Engine(d, dtype=dtype, page_size=8, max_cache_tokens=512)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=300, temperature=0.9, seed=4))[0]
    assert len(out.token_ids) == 300
    ids = prompt + out.token_ids
    steps = H.trace_decode_tail("x", ids, tail=len(ids) - 11)
    got = H.run_trace_in_process(d, dtype, steps, 320, 8)["x"]
    want = H.plain_logits(d, ids, bf16_weights=(dtype == "bfloat16"))
    err = np.abs(got - want)
    bound = 2e-4 if dtype == "float32" else 8 * np.sqrt(((H.plain_logits_in_bf16(d, ids) - want) ** 2).mean())
    assert err.max() <= bound, f"first wrong position {int(np.where(err.max(axis=1) > bound)[0][0])}, max {err.max():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(model_dirs, dtype):
    """Position 0 alone, positions 0-1, and a one-token prompt that is then decoded."""
    d, raw = model_dirs["C"], H.TINY["C"]
    ids = H.random_ids(raw["vocab_size"], 6, seed=9)
    want = H.plain_logits(d, ids, bf16_weights=(dtype == "bfloat16"))
    tol = 2e-4 if dtype == "float32" else 0.06
    for steps in (H.trace_decode_tail("x", ids, tail=5), H.trace_portions("x", ids, [2, 1, 3]),
                  H.trace_portions("x", ids, [1, 2, 3])):
        got = H.run_trace_in_process(d, dtype, steps, 64, 32)["x"]
        assert np.abs(got - want).max() <= tol


def test_positions_beyond_the_nominal_maximum(model_dirs):
    """max_position_embeddings (256 for configuration A) is advisory, as in the reference: a
    longer sequence replays and matches the plain implementation."""
    d, raw = model_dirs["A"], H.TINY["A"]
    ids = H.random_ids(raw["vocab_size"], 300, seed=12)
    got = H.run_trace_in_process(d, "float32", H.trace_portions("x", ids, [128, 1, 60]), 320, 16)["x"]
    assert np.abs(got - H.plain_logits(d, ids)).max() <= 2e-4


def test_command_line_and_trace_run_program(model_dirs, tmp_path):
    """The two programs as a user runs them: bin/pyre_generate and bin/trace_run."""
    d, raw = model_dirs["A"], H.TINY["A"]
    prompt = H.random_ids(raw["vocab_size"], 9, seed=2)
    res = subprocess.run([sys.executable, str(ROOT / "bin" / "pyre_generate"), "--model", str(d), "--dtype", "float32",
                          "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6",
                          "--out", str(tmp_path / "r.json")], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    toks = [int(t) for t in res.stdout.strip().splitlines()[-1].split()]
    assert toks == qwen2_plain.greedy_generate(prompt, H.load_plain_weights(d), raw, 6)
    assert json.loads((tmp_path / "r.json").read_text())["outputs"][0]["token_ids"] == toks

    ids = H.random_ids(raw["vocab_size"], 40, seed=8)
    steps = H.trace_portions("a", ids, [7, 2, 16])
    steps[0]["entries"][0]["want"] = []                  # a step in which nothing is wanted writes no file
    inp = "\n".join(json.dumps(s) for s in steps) + "\n"
    out = tmp_path / "logits"
    res = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
                          "--max-tokens", "64"], input=inp, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    assert res.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    assert not (out / "0.f32").exists()
    got = H.collect_trace_logits(steps, lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, raw["vocab_size"]))["a"]
    want = H.plain_logits(d, ids)[7:]
    assert np.abs(got - want).max() <= 2e-4


def test_a_raised_error_flag_stops_generation(model_dirs):
    """Kernels report a bounded wait that ran out (or an index out of range) through one flag per
    device; the engine reads it with every step's ids.  Here the flag is set by hand (nothing on the
    GPU goes wrong): the next step that is read raises, and the flag is clear afterwards."""
    from pyre_b200 import Engine, SamplingParams
    from pyre_b200.kernels import lib, ops
    d, raw = model_dirs["A"], H.TINY["A"]
    eng = Engine(d, dtype="bfloat16", max_cache_tokens=512)
    prompt = H.random_ids(raw["vocab_size"], 9, seed=8)
    assert len(eng.generate([prompt], SamplingParams(max_new_tokens=4))[0].token_ids) == 4
    ops.device_error_flag(eng.model.device).fill_(2)
    with pytest.raises(lib.KernelError, match="bounded wait"):
        eng.generate([prompt], SamplingParams(max_new_tokens=4))
    assert int(ops.device_error_flag(eng.model.device).item()) == 0


def test_cache_sized_by_a_fraction_of_free_memory(model_dirs):
    """Without a page count the pools can take a fraction of what the device has free after loading."""
    from pyre_b200 import Engine, SamplingParams
    d, raw = model_dirs["A"], H.TINY["A"]
    free_before, _ = torch.cuda.mem_get_info()
    eng = Engine(d, dtype="bfloat16", cache_memory_fraction=0.02, max_num_seqs=4)
    pool_bytes = sum(g.pool.numel() * g.pool.element_size() for g in eng.cache.groups)
    assert 0 < pool_bytes <= 0.02 * free_before
    assert pool_bytes >= 0.02 * free_before - (3 << 30)          # what is not reserved for activations is used
    out = eng.generate([H.random_ids(raw["vocab_size"], 20, seed=1)], SamplingParams(max_new_tokens=5))[0]
    assert len(out.token_ids) == 5
    with pytest.raises(ValueError):
        Engine(d, cache_memory_fraction=1.5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padded_captured_steps_give_the_same_logits(model_dirs, dtype):
    """A captured decode step of 5 to 13 tokens is padded to the next of a few sizes with rows that belong to no
    request.  The entries' logits are those of the same step launched kernel by kernel without padding (bit for
    bit in 32-bit, where a row's arithmetic does not depend on the batch), the pages of the requests stay intact,
    and few graphs serve all the sizes."""
    from pyre_b200.engine import replay as rp
    from pyre_b200.engine.step import StepEntry, Stepper
    d, raw = model_dirs["B"], H.TINY["B"]
    n_req = 13
    prompts = [H.random_ids(raw["vocab_size"], 3 + 5 * i, seed=50 + i) for i in range(n_req)]
    runs = []
    for graphs in (True, False):
        model, cache, _ = rp.build_runtime(d, dtype, 2048, 8, max_requests=n_req, poison=True)
        stepper = Stepper(model, cache, max_positions=None, cuda_graphs=graphs)
        for i, p in enumerate(prompts):
            cache.begin(i)
            stepper.step([StepEntry(i, p, [])])
        live, out = list(range(n_req)), []
        for k in range(3 * n_req):
            entries = [StepEntry(i, [(7 * i + k) % raw["vocab_size"]], [0]) for i in live]
            out.append(stepper.step(entries).float().cpu().numpy().copy())
            if k % 3 == 2:                                   # a request ends every third step: 13, 12, ... 1 rows
                cache.end(live.pop(k % len(live)))
        cache.check()
        assert all(f == t for f, t in zip(cache.stats().pages_free, cache.stats().pages_total))
        runs.append(out)
        if graphs:
            assert stepper.graph_replays > 0
            sizes = {Stepper.padded_size(n) for n in range(1, n_req + 1)}
            assert sizes == {1, 2, 3, 4, 8, 12, 16}
            assert stepper.graph_captures <= 2 * len(sizes)   # the width of the tables changes once on the way
    for a, b in zip(*runs):
        assert a.shape == b.shape
        if dtype == "float32":
            assert np.array_equal(a, b)
        else:
            assert np.abs(a - b).max() <= 2e-2 * max(1.0, np.abs(b).max())


def test_kernel_times_per_class(model_dirs):
    """``time_kernels``: every step runs kernel by kernel with events around each launch; the engine sums device
    time per kernel class and the step log carries each step's own.  The tokens are those of a normal run."""
    from pyre_b200 import Engine, SamplingParams
    d, raw = model_dirs["B"], H.TINY["B"]
    prompts = [H.random_ids(raw["vocab_size"], L, seed=60 + L) for L in (9, 30)]
    sp = SamplingParams(max_new_tokens=6)
    kw = dict(dtype="bfloat16", page_size=8, max_cache_tokens=512)
    plain = Engine(d, **kw).generate(prompts, sp)
    eng = Engine(d, time_kernels=True, record_steps=True, **kw)
    timed = eng.generate(prompts, sp)
    assert [o.token_ids for o in timed] == [o.token_ids for o in plain]
    assert {"embed", "norm", "qkv", "rotary+write", "attention", "o", "gate_up", "down", "head", "sampler"} <= set(eng.kernel_times)
    layers = raw["num_hidden_layers"]
    steps = len(eng.step_log)
    assert eng.kernel_times["qkv"]["launches"] == layers * steps and eng.kernel_times["head"]["launches"] == steps
    assert all(t["us"] > 0 for t in eng.kernel_times.values())
    assert all("kernel_us" in rec and rec["kernel_us"]["attention"] > 0 for rec in eng.step_log)
    assert eng.stepper.graph_replays == 0          # the measuring mode captures nothing
