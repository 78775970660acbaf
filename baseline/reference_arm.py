"""The reference arm of bench.py: the unmodified reference, installed offline into
``baseline/_ref``, measured through its own public API on the same metric and config.

Install (once, no network):

    python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
        --target baseline/_ref <checkout of Lalitaditya-tickoo/pyre>

What runs is the reference's stock path: ``pyre.loader.load_model`` on a model folder,
``pyre.scheduler.Scheduler.add_request`` and ``run`` (continuous batching with its Triton
paged-attention kernel).  Nothing of ``pyre_b200`` computes on that path; the package's
random-weights writer only prepares the folder the reference loads (it has no random
mode of its own).  Decode throughput follows the reference's own method
(bench/harness.py:8-16): ``(N - 1) * batch / (t_total - t_ttft)`` from two ``run()`` calls,
one capped at one new token and one at N.
"""

from __future__ import annotations

import json
import shutil
import sys
import tempfile
import time
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}


def _write_model_folder(folder: Path, cfg_raw: dict, seed: int) -> None:
    """config.json + bf16 safetensors shards under the checkpoint names, one layer per shard,
    drawn on the GPU so that 15 GB take seconds."""
    import torch
    from safetensors.torch import save_file

    from pyre_b200.config import config_from_dict
    from pyre_b200.weights import expected_tensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg_raw))
    table = expected_tensors(config_from_dict(cfg_raw))
    gen = torch.Generator(device="cuda").manual_seed(seed)
    shard, n, size = {}, 0, 0
    for name, spec in table.items():
        if spec.optional_alias is not None:
            continue
        _, mean, std = spec.init
        t = torch.empty(spec.shape, dtype=torch.float32, device="cuda").normal_(mean, std, generator=gen)
        shard[name] = t.to(torch.bfloat16).cpu()
        size += shard[name].numel() * 2
        if size > 1 << 30:
            save_file(shard, str(folder / f"model-{n:05d}.safetensors"))
            shard, n, size = {}, n + 1, 0
    if shard:
        save_file(shard, str(folder / f"model-{n:05d}.safetensors"))


def run(args, cfg_raw: dict, prompt_len: int, config_block: "dict | None" = None) -> dict:
    if not (REF / "pyre" / "scheduler.py").is_file():
        return unavailable("baseline/_ref is empty: the reference is not installed on this machine")
    try:
        import numpy as np
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        sys.path.insert(0, str(REF))
        from pyre.loader import load_model
        from pyre.scheduler import Scheduler
    except Exception as e:  # noqa: BLE001
        return unavailable(f"the reference does not import here: {type(e).__name__}: {e}")

    cfg_raw = dict(cfg_raw)
    layers_full = cfg_raw["num_hidden_layers"]
    if args.layers:
        cfg_raw["num_hidden_layers"] = args.layers
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    tmp = Path(tempfile.mkdtemp(prefix="pyre_ref_model_"))
    try:
        _write_model_folder(tmp, cfg_raw, seed=0)
        model, cfg = load_model(str(tmp), device="cuda", dtype=torch.bfloat16)
    except Exception as e:  # noqa: BLE001
        shutil.rmtree(tmp, ignore_errors=True)
        return unavailable(f"the reference could not load the model folder: {type(e).__name__}: {e}")
    shutil.rmtree(tmp, ignore_errors=True)

    rng = np.random.default_rng(0)

    def timed_run(batch: int, new_tokens: int) -> float:
        blocks = (prompt_len + new_tokens) // 16 + 2
        sched = Scheduler(model, cfg, num_blocks=blocks * batch + 8, max_batch=batch, device="cuda", dtype=torch.bfloat16)
        for _ in range(batch):
            sched.add_request(rng.integers(0, cfg.vocab_size, prompt_len).tolist(), new_tokens)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        sched.run()
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    try:
        timed_run(B, W + 1)                       # warm-up: W decode steps, JIT of the Triton kernel
        t_ttft = timed_run(B, 1)
        t_total = timed_run(B, K + 1)
        t_one = timed_run(1, 1)                   # one prompt of 2,048 tokens: the prefill
    except Exception as e:  # noqa: BLE001
        return unavailable(f"the reference's scheduler failed on this GPU: {type(e).__name__}: {e}")
    decode_s = max(t_total - t_ttft, 1e-9)
    value = K * B / decode_s
    return {
        "impl": "reference", "metric": "decode tok/s (Qwen2.5-7B shape, batch 8, 2,048-token prompts)",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(decode_s / K * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        # the same keys and values as the other arm prints; how this arm is timed stands beside it
        "config": config_block or {"model": "Qwen2.5-7B-shaped, random weights", "layers": cfg_raw["num_hidden_layers"],
                                   "layers_full": layers_full, "global_batch": B, "prompt_len": prompt_len, "page_size": 16},
        "timing": "wall clock around Scheduler.run(), (t_total - t_ttft) as in the reference's harness",
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "note": "the reference's run() is host tokens in, host tokens out"},
        "prefill": {"value": round(prompt_len / t_one, 1), "tokens": prompt_len, "ms": round(t_one * 1e3, 1)},
    }
