"""The engine's host side on the CPU: the package's parts, model, cache manager, step function and
replay loop with plain torch stand-ins for the kernels (``tests/standins.py``), in float32, against
the plain implementation.  The four ways of cutting a trace (whole, the tail token by token, portions
down to two tokens, mixed with so few pages that they are used again, freed pages filled with NaN)
must give the plain logits: what differs here is a fault of the batch's layout, the block tables,
the schedule or the bookkeeping, not of a kernel."""

import json
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import standins

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 7, 40, 63, 81]}


def runtime(model_dir, max_tokens, page_size, spec_edit=None):
    from pyre_b200.config import architecture_of, load_config
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.models import Model

    cfg = load_config(model_dir)
    spec = architecture_of(cfg).build(cfg)
    if spec_edit is not None:
        spec_edit(spec)
    model = Model(spec, torch.float32, "cpu")
    model.load_weights(model_dir)
    cache, stepper = runtime_for_model(model, max_tokens, page_size, poison=True, cuda_graphs=False)
    return model, cache, stepper


def run_trace(model_dir, steps, max_tokens, page_size, spec_edit=None):
    from pyre_b200.engine import replay as rp

    model, cache, stepper = runtime(model_dir, max_tokens, page_size, spec_edit)
    with tempfile.TemporaryDirectory() as out:
        rp.replay(stepper, [json.dumps(s) for s in steps], Path(out), done=lambda m: None)
        got = H.collect_trace_logits(steps, lambda n: np.fromfile(Path(out) / f"{n}.f32", dtype="<f4").reshape(-1, model.vocab_size))
    cache.check()
    assert not cache.live() and cache.stats().pages_free == cache.stats().pages_total
    return got


def compare(got, want, what):
    assert set(got) == set(want)
    for rid in want:
        g, w = got[rid], want[rid]
        assert g.shape == w.shape and np.isfinite(g).all(), f"{what} {rid}"
        bad = np.abs(g - w) > 2e-5 + 2e-4 * np.abs(w)
        if bad.any():
            row = int(np.where(bad.any(axis=1))[0][0])
            raise AssertionError(f"{what} {rid}: first wrong token at position {row} of {g.shape[0]}, "
                                 f"max |diff| there {np.abs(g - w)[row].max():.3e}")


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for n, name in enumerate(LENGTHS):
        raw = H.TINY[name]
        d = tmp_path_factory.mktemp(f"cpu_{name}")
        H.make_model_dir(d, raw, seed=300 + n)
        reqs = {f"{name}{i}": H.random_ids(raw["vocab_size"], L, seed=11 * n + i) for i, L in enumerate(LENGTHS[name])}
        out[name] = (d, reqs, {rid: H.plain_logits(d, ids) for rid, ids in reqs.items()})
    return out


@pytest.mark.parametrize("name", list(LENGTHS))
def test_every_way_of_cutting_gives_the_plain_logits(models, name, monkeypatch):
    standins.install(monkeypatch)
    d, reqs, want = models[name]
    page = H.PAGE_SIZE[name]
    steps = H.trace_whole(reqs)
    compare(run_trace(d, steps, H.max_live_tokens(steps), page), want, "whole")
    rid = max(reqs, key=lambda r: len(reqs[r]))
    steps = H.trace_decode_tail(rid, reqs[rid], tail=32)
    compare(run_trace(d, steps, H.max_live_tokens(steps), page), {rid: want[rid]}, "tail token by token")
    steps = H.trace_portions(rid, reqs[rid], [7, 2, 19, 3, 2, 30])
    compare(run_trace(d, steps, H.max_live_tokens(steps), page), {rid: want[rid]}, "portions")
    for seed in (1, 2):
        steps = H.trace_mixed(reqs, seed=seed, max_live=3)
        compare(run_trace(d, steps, H.max_live_tokens(steps), page), want, f"mixed (seed {seed})")


def test_a_schedule_with_a_repeated_layer_a_shared_cache_and_a_window(models, monkeypatch):
    """Layer 0 twice, layer 1 with a window of 9 keys whose second run reads the first run's cache:
    the plain implementation with the same schedule and window, in portions that straddle pages."""
    from pyre_b200.models import LayerCall
    from pyre_b200.parts import PartSpec
    from plain import qwen2_plain

    standins.install(monkeypatch)
    d, reqs, _ = models["A"]
    raw = H.TINY["A"]

    def edit(spec):
        b = spec.blocks[1]
        spec.blocks[1] = PartSpec(b.kind, dict(b.params, mixer=PartSpec("attention", dict(b.params["mixer"].params, window=9))))
        spec.schedule = [LayerCall(0), LayerCall(1, cache="s"), LayerCall(0), LayerCall(1, cache="s", write=False)]

    rid = "A3"
    ids = reqs[rid]
    with torch.inference_mode():
        want = qwen2_plain.forward(ids, H.load_plain_weights(d), raw, schedule=[(0, None), (1, None), (0, None), (1, 1)],
                                   windows=[None, 9, None, 9]).numpy()
    for sizes in ([len(ids)], [5, 2, 11, 1, 1, 1, 17], [40] + [1] * 30):
        steps = H.trace_portions(rid, ids, sizes)
        got = run_trace(d, steps, 128, 4, edit)
        compare(got, {rid: want}, f"portions {sizes[:4]}")


class HostSampler:
    """The sampler's two calls without pinned memory or events: greedy ids straight from the stand-in."""

    def sample_async(self, logits, params, token_index):
        import types

        from pyre_b200.kernels import ops
        assert all(p.temperature == 0.0 for p in params)
        return types.SimpleNamespace(ids=ops.sample(logits))

    def read(self, ticket):
        return ticket.ids.tolist()


@pytest.mark.parametrize("lookahead", [True, False])
def test_greedy_generation_through_the_engine_loop(models, monkeypatch, lookahead):
    """``Engine.generate`` with the real model, stepper, cache manager and scheduler (kernels and sampler
    stood in for): few pages, so requests are preempted and recomputed; with ``lookahead`` the token a
    step needs from the step before never passes through the host.  Ids equal the plain greedy ids."""
    import contextlib

    from pyre_b200.config import EngineConfig
    from pyre_b200.engine.engine import Engine
    from pyre_b200.engine.scheduler import Scheduler
    from pyre_b200.sampling import SamplingParams
    from plain import qwen2_plain

    standins.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "device", lambda device: contextlib.nullcontext())
    d, reqs, _ = models["B"]
    raw = H.TINY["B"]
    model, cache, stepper = runtime(d, max_tokens=15 * 8, page_size=8)
    eng = object.__new__(Engine)
    eng.engine_config = EngineConfig(dtype="float32", lookahead=lookahead, record_steps=True)
    eng.model, eng.cache, eng.stepper, eng.sampler = model, cache, stepper, HostSampler()
    eng.max_model_len = 15 * 8
    eng.scheduler = Scheduler(cache, 4, 48, 20, eng.max_model_len, admit_whole_prompts=False)
    eng._requests, eng._flight, eng.step_log = {}, None, []
    eng._err_host, eng._err_turn = [torch.zeros(1, dtype=torch.int32) for _ in range(2)], 0
    prompts = [ids for ids in reqs.values()]
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=9))
    w = H.load_plain_weights(d)
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and o.token_ids == qwen2_plain.greedy_generate(p, w, raw, 9), len(p)
    assert eng.stats()["preempted"] > 0, "the cache was meant to be too small for all requests at once"
    cache.check()
    assert not cache.live() and cache.stats().pages_free == cache.stats().pages_total
    assert len(eng.step_log) == eng.scheduler.stats.steps


# --------------------------------------------------------------------------- the bfloat16 path's host side
TINY_D = dict(architectures=["Qwen2ForCausalLM"], hidden_size=512, intermediate_size=640, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=300, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=512)


def bf16_runtime(model_dir, max_tokens, page_size):
    from pyre_b200.config import architecture_of, load_config
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.models import Model

    cfg = load_config(model_dir)
    model = Model(architecture_of(cfg).build(cfg), torch.bfloat16, "cpu")
    model.load_weights(model_dir)
    return (model, *runtime_for_model(model, max_tokens, page_size, poison=True, cuda_graphs=False))


@pytest.mark.parametrize("page_size", [16, 24])
def test_bfloat16_dispatch_of_a_mixed_step(tmp_path, monkeypatch, page_size):
    """Head size 64: entries of 64 tokens or more go to the prompt-portion attention (the tcgen05 kernel with
    power-of-two pages, else the mma.sync one from 32 tokens on), the rest of the same step to the split-KV
    kernel; split-K partial sums reach the norm and the rotary kernel; the gated feed-forward's rows are
    interleaved.  With stand-ins that write only what each kernel takes, logits stay within the error of
    bfloat16 arithmetic of the plain implementation."""
    from pyre_b200.engine import replay as rp

    calls = {}
    standins.install_bf16(monkeypatch, calls)
    H.make_model_dir(tmp_path, TINY_D, seed=77)
    reqs = {"a": H.random_ids(300, 150, seed=1), "b": H.random_ids(300, 90, seed=2), "c": H.random_ids(300, 50, seed=3)}
    a, b, c = reqs["a"], reqs["b"], reqs["c"]

    def entry(rid, toks):
        return {"id": rid, "tokens": toks, "want": list(range(len(toks)))}

    steps = [
        {"step": 0, "entries": [entry("a", a[:70])], "end": []},                                   # one long entry
        {"step": 1, "entries": [entry("a", a[70:71]), entry("b", b[:66]), entry("c", c[:5])], "end": []},   # decode + long + short
        {"step": 2, "entries": [entry("a", a[71:72]), entry("b", b[66:67]), entry("c", c[5:6])], "end": []},  # decode only
        {"step": 3, "entries": [entry("c", c[6:46]), entry("a", a[72:150])], "end": ["a"]},        # 40 tokens and 78 tokens
        {"step": 4, "entries": [entry("b", b[67:90]), entry("c", c[46:50])], "end": ["b", "c"]},
    ]
    model, cache, stepper = bf16_runtime(tmp_path, 512, page_size)
    assert model.blocks[0].ffn.interleaved
    with tempfile.TemporaryDirectory() as out:
        rp.replay(stepper, [json.dumps(s) for s in steps], Path(out), done=lambda m: None)
        got = H.collect_trace_logits(steps, lambda n: np.fromfile(Path(out) / f"{n}.f32", dtype="<f4").reshape(-1, 300))
    cache.check()
    assert not cache.live()
    layers = TINY_D["num_hidden_layers"]
    if page_size == 16:
        assert calls.get("attention_prefill_tc") == 3 * layers and "attention_prefill" not in calls    # steps 0, 1, 3
        assert calls["paged_attention_mma"] == 4 * layers                                          # steps 1-4
    else:
        assert calls.get("attention_prefill") == 3 * layers and "attention_prefill_tc" not in calls    # 40 tokens count as long here
        assert calls["paged_attention_mma"] == 3 * layers                                          # steps 1, 2, 4
    sq_e = sq_r = cnt = 0.0
    for rid, ids in reqs.items():
        truth = H.plain_logits(tmp_path, ids, bf16_weights=True)
        e, r = got[rid] - truth, H.plain_logits_in_bf16(tmp_path, ids) - truth
        assert np.isfinite(got[rid]).all()
        sq_e, sq_r, cnt = sq_e + float((e.astype(np.float64) ** 2).sum()), sq_r + float((r.astype(np.float64) ** 2).sum()), cnt + e.size
    rms_e, rms_r = (sq_e / cnt) ** 0.5, (sq_r / cnt) ** 0.5
    assert rms_e <= rms_r, f"rms error {rms_e:.3e} exceeds the {rms_r:.3e} of plain bfloat16 arithmetic"
    for rid, ids in reqs.items():
        e = np.abs(got[rid] - H.plain_logits(tmp_path, ids, bf16_weights=True))
        bad = np.where(e.max(axis=1) > 8 * rms_r)[0]
        assert not len(bad), f"{rid}: first wrong token at position {int(bad[0])}, error {e[bad[0]].max():.3e} (rms {rms_r:.3e})"


def test_toy_mixer_with_state_registers_builds_and_steps_on_the_cpu(tmp_path, monkeypatch):
    """The scenario of ``tests/toy_parts.py`` (a recurrent mixer with state in the cache manager's slots and an
    architecture of its own, registered from the test) with the stand-ins: the package's files need no change
    for it, and the state slots, their zeroing and the mixed steps work without a GPU too."""
    import toy_parts

    standins.install(monkeypatch)
    toy_parts.toy_decay_model_scenario(tmp_path, "cpu")


def test_toy_routed_ffn_and_toy_positions_on_the_cpu(tmp_path, monkeypatch):
    """The second scenario of ``tests/toy_parts.py``: a routed feed-forward and a position encoding of the
    test's own beside the package's attention part (which takes the toy positions' tables)."""
    import toy_parts

    standins.install(monkeypatch)
    toy_parts.toy_routed_model_scenario(tmp_path, "cpu")


def test_trace_run_program_and_load_model_on_the_cpu(models, tmp_path, monkeypatch, capsys):
    """``trace_run``'s own main (arguments, the model through ``load_model`` and the registry, steps from
    standard input, a ``done`` line per step, the .f32 files) with the stand-ins and ``--device cpu``."""
    import io
    import sys

    import pyre_b200
    from pyre_b200.engine import replay as rp

    standins.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    d, reqs, want = models["A"]
    model, cfg = pyre_b200.load_model(d, device="cpu", dtype="float32")
    assert type(cfg).__name__ == "Qwen2Config" and cfg.hidden_size == 64 and model.loaded and model.dtype is torch.float32
    ids = reqs["A2"]
    steps = H.trace_portions("A2", ids, [9, 2, 16]) + [{"step": 99, "entries": [], "end": []}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps) + "\n"))
    out = tmp_path / "logits"
    assert rp.main(["--model", str(d), "--dtype", "float32", "--out", str(out), "--max-tokens", "64", "--device", "cpu"]) == 0
    assert capsys.readouterr().out.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    got = H.collect_trace_logits(steps, lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, 512))
    compare(got, {"A2": want["A2"]}, "trace_run main")
    assert not (out / "99.f32").exists()                       # nothing wanted, nothing written
    # any page size the engine takes, also one that does not divide 64
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    out24 = tmp_path / "logits24"
    assert rp.main(["--model", str(d), "--dtype", "float32", "--out", str(out24), "--max-tokens", "64", "--device", "cpu",
                    "--page-size", "24"]) == 0
    got = H.collect_trace_logits(steps, lambda n: np.fromfile(out24 / f"{n}.f32", dtype="<f4").reshape(-1, 512))
    compare(got, {"A2": want["A2"]}, "trace_run main, pages of 24 tokens")
    with pytest.raises(SystemExit):
        rp.main(["--model", str(d), "--dtype", "float32", "--out", str(out), "--max-tokens", "64", "--page-size", "0"])
    assert rp.pages_for_max_tokens(256, 16) == 16 and rp.pages_for_max_tokens(256, 128) == 2
    assert rp.pages_for_max_tokens(256, 24) == 11 + 3          # four requests of 64: three pages each, not 11 in all


def test_a_trace_that_cannot_be_run_ends_with_one_clear_line(models, tmp_path, monkeypatch, capsys):
    import io
    import sys

    from pyre_b200.engine import replay as rp

    standins.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    d, _, _ = models["A"]
    good = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": []})
    cases = [('{"step": 1, "entries": [', "line 2: not JSON"),
             ('[1, 2]', 'line 2: a step is an object with a "step" field'),
             ('{"step": 1, "entries": [{"id": "a", "tokens": "5"}]}', "line 2 (step 1): an entry is an object"),
             ('{"step": 1, "entries": [{"id": "a", "tokens": [1.5]}]}', "line 2 (step 1): tokens and wanted places are integers"),
             ('{"step": 1, "entries": [{"id": "a", "tokens": [4], "want": [1]}]}', "line 2 (step 1): request 'a': wanted place 1"),
             ('{"step": 1, "entries": [{"id": "a", "tokens": [512]}]}', "line 2 (step 1): request 'a': token id outside"),
             ('{"step": 1, "entries": [], "end": ["b"]}', "line 2 (step 1): request 'b' is not live"),
             ('{"step": 1, "entries": [{"id": "b", "tokens": ' + str(list(range(100))) + '}]}', "line 2 (step 1): request 'b': no pages left")]
    for bad, message in cases:
        monkeypatch.setattr(sys, "stdin", io.StringIO(good + "\n" + bad + "\n"))
        rc = rp.main(["--model", str(d), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64", "--device", "cpu"])
        captured = capsys.readouterr()
        assert rc == 1 and captured.out == "done 0\n", bad
        assert captured.err.strip().startswith("trace_run: " + message), (captured.err, message)


def test_command_line_generates_and_writes_its_result_and_step_log(models, tmp_path, monkeypatch, capsys):
    """``python -m pyre_b200 generate`` end to end on the CPU: the real ``Engine`` constructor, scheduler and loop
    (kernels and sampler stood in for, ``--device cpu``), token ids on standard output, ``--out`` and ``--step-log``."""
    import contextlib

    from pyre_b200 import cli
    from pyre_b200.sampling import Sampler
    from plain import qwen2_plain

    standins.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device", lambda device: contextlib.nullcontext())
    monkeypatch.setattr(Sampler, "sample_async", HostSampler.sample_async)
    monkeypatch.setattr(Sampler, "read", HostSampler.read)
    d, reqs, _ = models["A"]
    prompts = [reqs["A0"], reqs["A1"]]
    (tmp_path / "prompts.txt").write_text(" ".join(map(str, prompts[1])) + "\n")
    rc = cli.main(["generate", "--model", str(d), "--device", "cpu", "--dtype", "float32", "--max-new-tokens", "6",
                   "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids-file", str(tmp_path / "prompts.txt"),
                   "--num-pages", "12", "--page-size", "8", "--prefill-chunk", "8", "--max-batched-tokens", "16",
                   "--out", str(tmp_path / "result.json"), "--step-log", str(tmp_path / "steps.jsonl")])
    assert rc == 0
    w = H.load_plain_weights(d)
    want = [qwen2_plain.greedy_generate(p, w, H.TINY["A"], 6) for p in prompts]
    printed = [[int(t) for t in line.split()] for line in capsys.readouterr().out.strip().split("\n")]
    assert printed == want
    result = json.loads((tmp_path / "result.json").read_text())
    assert [o["token_ids"] for o in result["outputs"]] == want and result["new_tokens"] == 12
    assert [o["finish_reason"] for o in result["outputs"]] == ["length", "length"] and result["stats"]["finished"] == 2
    log = [json.loads(line) for line in (tmp_path / "steps.jsonl").read_text().splitlines()]
    assert len(log) == result["stats"]["steps"] and sum(r["tokens"] for r in log) == result["stats"]["scheduled_tokens"]
    assert log[0]["prompt_tokens"] == log[0]["tokens"] and log[-1]["decoded_tokens"] >= 1
    assert cli.main(["generate", "--model", str(d), "--device", "cpu"]) == 2          # no prompts


def test_temperature_sampling_is_per_request_whatever_the_batch(models, monkeypatch):
    """The engine hands the sampler each row's own parameters and the index of the token being drawn (tokens
    still in flight included), so a request's draw depends on its seed and its own history only: together,
    alone, with or without a step in flight, with preemption, the ids are those of the plain sampler run on
    the plain logits."""
    import contextlib
    import types

    from pyre_b200 import Engine, SamplingParams
    from pyre_b200.sampling import Sampler
    from plain import qwen2_plain

    def sample_async(self, logits, params, token_index):
        ids = [qwen2_plain.sample(row, p.temperature, p.seed, k) for row, p, k in zip(logits, params, token_index)]
        return types.SimpleNamespace(ids=torch.tensor(ids, dtype=torch.int32))

    standins.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device", lambda device: contextlib.nullcontext())
    monkeypatch.setattr(Sampler, "sample_async", sample_async)
    monkeypatch.setattr(Sampler, "read", HostSampler.read)
    d, reqs, _ = models["B"]
    raw, w = H.TINY["B"], H.load_plain_weights(d)
    prompts = [reqs["B1"], reqs["B2"], reqs["B0"]]
    params = [SamplingParams(temperature=0.8, seed=5, max_new_tokens=7), SamplingParams(temperature=0.0, max_new_tokens=5),
              SamplingParams(temperature=1.3, seed=6, max_new_tokens=8)]

    def plain_ids(prompt, p):
        ids = list(prompt)
        for k in range(p.max_new_tokens):
            with torch.inference_mode():
                ids.append(qwen2_plain.sample(qwen2_plain.forward(ids, w, raw)[-1], p.temperature, p.seed, k))
        return ids[len(prompt):]

    want = [plain_ids(p, sp) for p, sp in zip(prompts, params)]
    kw = dict(device="cpu", dtype="float32", page_size=8, prefill_chunk=16, max_num_batched_tokens=24)
    for lookahead, num_pages in ((True, 64), (False, 64), (True, 7)):
        eng = Engine(d, lookahead=lookahead, num_pages=num_pages, admit_whole_prompts=False, **kw)
        outs = eng.generate(prompts, params)
        assert [o.token_ids for o in outs] == want, (lookahead, num_pages)
        if num_pages == 7:
            assert eng.stats()["preempted"] > 0
    alone = Engine(d, num_pages=64, **kw)
    assert [alone.generate([p], sp)[0].token_ids for p, sp in zip(prompts, params)] == want


@pytest.mark.parametrize("lookahead", [True, False])
def test_logits_come_back_with_the_tokens_when_asked_for(models, monkeypatch, lookahead):
    """``SamplingParams.return_logits``: one row per generated token, the logits it was chosen from (the plain
    logits at that position), also for a request that stops at its end-of-sequence token (whose overshoot is
    dropped) and for one that was preempted and recomputed; a request that does not ask gets none."""
    import contextlib

    from pyre_b200 import Engine, SamplingParams
    from pyre_b200.sampling import Sampler
    from plain import qwen2_plain

    standins.install(monkeypatch)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device", lambda device: contextlib.nullcontext())
    monkeypatch.setattr(Sampler, "sample_async", HostSampler.sample_async)
    monkeypatch.setattr(Sampler, "read", HostSampler.read)
    d, reqs, _ = models["B"]
    raw, w = H.TINY["B"], H.load_plain_weights(d)
    prompts = [reqs["B1"], reqs["B2"], reqs["B0"]]
    greedy = [qwen2_plain.greedy_generate(p, w, raw, 8) for p in prompts]
    params = [SamplingParams(max_new_tokens=8, return_logits=True),
              SamplingParams(max_new_tokens=8, return_logits=True, eos_id=greedy[1][3]),      # stops at its fourth token at the latest
              SamplingParams(max_new_tokens=8)]
    eng = Engine(d, device="cpu", dtype="float32", page_size=8, num_pages=8, prefill_chunk=16, max_num_batched_tokens=24,
                 lookahead=lookahead, admit_whole_prompts=False)
    outs = eng.generate(prompts, params)
    assert eng.stats()["preempted"] > 0
    assert outs[2].logits is None and outs[2].token_ids == greedy[2]
    stop = greedy[1].index(greedy[1][3]) + 1
    assert outs[1].token_ids == greedy[1][:stop] and outs[1].finish_reason == "eos" and outs[0].token_ids == greedy[0]
    for p, o in zip(prompts[:2], outs[:2]):
        with torch.inference_mode():
            want = qwen2_plain.forward(list(p) + o.token_ids[:-1], w, raw)[len(p) - 1:].numpy()
        assert o.logits.shape == (len(o.token_ids), raw["vocab_size"]) and o.logits.dtype == np.float32
        np.testing.assert_allclose(o.logits, want, rtol=2e-4, atol=2e-5)
        assert o.logits.argmax(axis=1).tolist() == o.token_ids


def test_replay_answers_each_line_before_the_next_one_is_written(models, monkeypatch):
    """The next step of a trace may come only after ``done <step>``: the loop must answer a line as soon as it
    has it, without waiting for more input.  Lines go through a pipe one at a time; each answer is awaited."""
    import os
    import queue
    import threading

    from pyre_b200.engine import replay as rp

    standins.install(monkeypatch)
    d, reqs, want = models["A"]
    _, cache, stepper = runtime(d, 128, 16)
    steps = H.trace_portions("A1", reqs["A1"], [4, 2, 5])
    r_fd, w_fd = os.pipe()
    answers: "queue.Queue[str]" = queue.Queue()
    failure = []

    def loop(out):
        try:
            with os.fdopen(r_fd, "r") as lines:
                rp.replay(stepper, lines, Path(out), done=answers.put)
        except Exception as e:          # handed to the main thread
            failure.append(e)
            answers.put("failed")

    with tempfile.TemporaryDirectory() as out:
        t = threading.Thread(target=loop, args=(out,), daemon=True)
        t.start()
        with os.fdopen(w_fd, "w") as pipe:
            for s in steps:
                pipe.write(json.dumps(s) + "\n")
                pipe.flush()
                assert answers.get(timeout=60) == f"done {s['step']}", failure
        t.join(timeout=60)
        assert not t.is_alive() and not failure
        got = H.collect_trace_logits(steps, lambda n: np.fromfile(Path(out) / f"{n}.f32", dtype="<f4").reshape(-1, 512))
    compare(got, {"A1": want["A1"]}, "line by line through a pipe")


def test_a_tail_of_the_tests_own_ends_the_model(models, monkeypatch):
    """The model's skeleton is data: embed, the scheduled blocks, a tail.  A tail registered from this test (no final
    norm; two heads whose logits are averaged and scaled) replaces the usual norm + head without a change to the
    package; the step function, the replay loop and the loader serve it as they serve the built-in one."""
    from pyre_b200.config import architecture_of, load_config
    from pyre_b200.engine.replay import runtime_for_model
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import ops
    from pyre_b200.models import Model
    from pyre_b200.parts import Part, PartSpec, register_part
    from pyre_b200.weights import TensorSpec

    standins.install(monkeypatch)

    class ToyTwoHeadTail(Part):
        def __init__(self, dtype, device, vocab, width, scale):
            super().__init__(dtype, device)
            self.vocab, self.width, self.scale = vocab, width, scale

        def tensors(self):
            return {"head_a.weight": TensorSpec((self.vocab, self.width)), "head_b.weight": TensorSpec((self.vocab, self.width))}

        def load(self, tensors):
            self.a, self.b = tensors["head_a.weight"], tensors["head_b.weight"]

        def forward(self, ctx, x, pending):
            v = x + ops.materialize(pending).float()            # the last block's branch output is still pending
            rows = v[ctx.logit_rows.long()]
            return (rows @ self.a.float().t() + rows @ self.b.float().t()) * (0.5 * self.scale)

    register_part("tail", "toy_two_heads", ToyTwoHeadTail, replace=True)
    d, reqs, _ = models["A"]
    cfg = load_config(d)
    spec = architecture_of(cfg).build(cfg)
    spec.tail = PartSpec("toy_two_heads", {"vocab": cfg.vocab_size, "width": cfg.hidden_size, "scale": 3.0})
    spec.tail_prefix = "out."
    model = Model(spec, torch.float32, "cpu")
    table = model.tensor_table()
    assert "out.head_a.weight" in table and "model.norm.weight" not in table and "lm_head.weight" not in table
    w = H.load_plain_weights(d)
    g = torch.Generator().manual_seed(4)
    extra = {"out.head_a.weight": torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.1,
             "out.head_b.weight": torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.1}
    from safetensors.torch import save_file
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        tensors = {k: v for k, v in w.items() if k in table}
        tensors.update(extra)
        save_file(tensors, str(Path(tmp) / "model.safetensors"))
        (Path(tmp) / "config.json").write_text((Path(d) / "config.json").read_text())
        model.load_weights(tmp)
    cache, stepper = runtime_for_model(model, 128, 16, cuda_graphs=False)
    ids = reqs["A3"]
    cache.begin("r")
    got = torch.cat([stepper.step([StepEntry("r", ids[:30], list(range(30)))]),
                     stepper.step([StepEntry("r", ids[30:], list(range(len(ids) - 30)))])])
    with torch.inference_mode():
        _, hidden = qwen2_plain_forward_hidden(ids, w, H.TINY["A"])
    want = (hidden @ extra["out.head_a.weight"].t() + hidden @ extra["out.head_b.weight"].t()) * 1.5
    assert np.abs(got.numpy() - want.numpy()).max() <= 2e-5 + 2e-4 * float(want.abs().max())


def qwen2_plain_forward_hidden(ids, w, raw):
    from plain import qwen2_plain
    logits, hidden = qwen2_plain.forward(ids, w, raw, return_hidden=True)
    return logits, hidden[-1]
