"""Shared fixtures of the tests: the tiny configurations, model folders with random
weights in a temporary place, the plain implementation's logits, and trace builders."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch
from safetensors.torch import load_file, save_file

from plain import qwen2_plain

# Two tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], hidden_size=64, intermediate_size=176, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=512, rope_theta=10000.0,
              rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256)
TINY_B = dict(architectures=["Qwen2ForCausalLM"], hidden_size=96, intermediate_size=256, num_hidden_layers=3,
              num_attention_heads=3, num_key_value_heads=1, head_dim=32, vocab_size=1000, rope_theta=1e6,
              rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512)
# A third one with sizes that are no power of two anywhere and nh * hd != hidden.
TINY_C = dict(architectures=["Qwen2ForCausalLM"], hidden_size=120, intermediate_size=200, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, vocab_size=777, rope_theta=50000.0,
              rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=384)
# A fourth one whose width and feed-forward size are no multiples of 8: rows that a TMA copy cannot fetch, so the
# bfloat16 products with those inner sizes take the library fallback, and the vector paths of the small kernels
# their scalar form.
TINY_D = dict(architectures=["Qwen2ForCausalLM"], hidden_size=92, intermediate_size=66, num_hidden_layers=2,
              num_attention_heads=10, num_key_value_heads=2, head_dim=80, vocab_size=333, rope_theta=12345.0,
              rms_norm_eps=2e-6, tie_word_embeddings=True, max_position_embeddings=512)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
PAGE_SIZE = {"A": 16, "B": 8, "C": 32, "D": 64}


def make_model_dir(path: Path, raw_cfg: dict, seed: int, sharpen: float = 6.0, matrix_scale: float = 2.5) -> dict[str, torch.Tensor]:
    """Write config.json + model.safetensors (fp32) with the package's random mode, then
    scale the query and key projections so that attention is peaked: with N(0, 0.02)
    weights every score is near zero and a wrong key would change nothing.  Returns the
    tensors as written."""
    from pyre_b200.config import config_from_dict
    from pyre_b200.weights import random_state

    path.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(raw_cfg)
    state = random_state(cfg, seed)
    for name in state:
        if name.endswith(("q_proj.weight", "k_proj.weight", "q_proj.bias", "k_proj.bias")):
            state[name] = state[name] * sharpen
        elif state[name].dim() == 2:
            state[name] = state[name] * matrix_scale
    (path / "config.json").write_text(json.dumps(raw_cfg))
    save_file({k: v.contiguous() for k, v in state.items()}, str(path / "model.safetensors"))
    return state


def load_plain_weights(path: Path, round_matrices_to_bf16: bool = False) -> dict[str, torch.Tensor]:
    w = load_file(str(Path(path) / "model.safetensors"))
    if round_matrices_to_bf16:
        w = {k: (v.to(torch.bfloat16).to(torch.float32) if v.dim() == 2 else v) for k, v in w.items()}
    return w


def plain_logits(path: Path, ids, bf16_weights: bool = False) -> np.ndarray:
    raw = json.loads((Path(path) / "config.json").read_text())
    w = load_plain_weights(path, bf16_weights)
    with torch.inference_mode():
        return qwen2_plain.forward(list(ids), w, raw).numpy()


def plain_logits_in_bf16(path: Path, ids) -> np.ndarray:
    """The plain implementation with every tensor in bfloat16, as the reference runs a
    model in a 16-bit dtype (pyre/loader.py:74)."""
    raw = json.loads((Path(path) / "config.json").read_text())
    w = {k: v.to(torch.bfloat16) for k, v in load_plain_weights(path).items()}
    with torch.inference_mode():
        return qwen2_plain.forward(list(ids), w, raw).float().numpy()


def random_ids(vocab: int, n: int, seed: int) -> list[int]:
    g = np.random.default_rng(seed)
    return [int(x) for x in g.integers(0, vocab, n)]


# --------------------------------------------------------------------------- traces
def trace_whole(reqs: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one after the other."""
    steps = []
    for n, (rid, ids) in enumerate(reqs.items()):
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]})
    return steps


def trace_decode_tail(rid: str, ids: list[int], tail: int = 32, first_step: int = 0) -> list[dict]:
    """Most of the request in one step, the last ``tail`` tokens one by one."""
    head = max(1, len(ids) - tail)
    steps = [{"step": first_step, "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []}]
    for i in range(head, len(ids)):
        steps.append({"step": first_step + len(steps), "entries": [{"id": rid, "tokens": [ids[i]], "want": [0]}], "end": []})
    steps[-1]["end"] = [rid]
    return steps


def trace_portions(rid: str, ids: list[int], sizes: list[int], first_step: int = 0) -> list[dict]:
    """In portions of changing size (cycled), down to two tokens."""
    steps, pos, k = [], 0, 0
    while pos < len(ids):
        n = min(sizes[k % len(sizes)], len(ids) - pos)
        steps.append({"step": first_step + len(steps),
                      "entries": [{"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))}], "end": []})
        pos += n
        k += 1
    steps[-1]["end"] = [rid]
    return steps


def trace_mixed(reqs: dict[str, list[int]], seed: int, max_live: int = 4, prefill_head: float = 0.6,
                portion: tuple[int, int] = (2, 24)) -> list[dict]:
    """Up to ``max_live`` requests at a time: a request first gets portions of random size
    (``portion``: smallest and largest, 2..24 tokens by default) for the first part of its
    tokens, then single tokens, beside whatever the other live requests get in the same step;
    a finished request is ended and the next one begins, so its pages are used again."""
    rng = np.random.default_rng(seed)
    waiting = list(reqs.items())
    live: dict[str, dict] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            live[rid] = {"ids": ids, "pos": 0, "head": max(1, int(len(ids) * prefill_head))}
        entries, end = [], []
        for rid, st in list(live.items()):
            if rng.random() < 0.2 and len(live) > 1:
                continue  # left out of this step, goes on later
            if st["pos"] < st["head"]:
                n = int(min(rng.integers(portion[0], portion[1] + 1), st["head"] - st["pos"]))
            else:
                n = 1
            n = min(n, len(st["ids"]) - st["pos"])
            toks = st["ids"][st["pos"]:st["pos"] + n]
            entries.append({"id": rid, "tokens": toks, "want": list(range(n))})
            st["pos"] += n
            if st["pos"] == len(st["ids"]):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def collect_trace_logits(steps: list[dict], read_step) -> dict[str, np.ndarray]:
    """Reassemble per-request logits [n_tokens, vocab] from per-step outputs.
    ``read_step(step_number)`` returns the [wanted, vocab] array of that step."""
    rows: dict[str, list] = {}
    for st in steps:
        if not any(e["want"] for e in st["entries"]):
            continue
        arr = read_step(st["step"])
        k = 0
        for e in st["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(arr[k])
                k += 1
        assert k == arr.shape[0]
    return {rid: np.stack(r) for rid, r in rows.items()}


def max_live_tokens(steps: list[dict], quantum: int = 64) -> int:
    """The most tokens that live requests hold at any time, each rounded up to ``quantum``."""
    held: dict[str, int] = {}
    worst = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // quantum) * quantum for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return worst


def run_trace_in_process(model_dir: Path, dtype: str, steps: list[dict], max_tokens: int, page_size: int,
                         poison: bool = True) -> dict[str, np.ndarray]:
    """Drive the engine's replay loop in this process and return per-request logits."""
    import tempfile
    from pyre_b200.engine import replay as rp

    _, cache, stepper = rp.build_runtime(model_dir, dtype, max_tokens, page_size, poison=poison)
    with tempfile.TemporaryDirectory() as out:
        out = Path(out)
        rp.replay(stepper, [json.dumps(s) for s in steps], out, done=lambda m: None)
        vocab = stepper.model.vocab_size
        result = collect_trace_logits(steps, lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, vocab))
    cache.check()
    assert not cache.live(), "requests left alive after the trace"
    assert all(f == t for f, t in zip(cache.stats().pages_free, cache.stats().pages_total)), "pages leaked"
    return result
