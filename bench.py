"""Benchmark of the serving step: decode tokens/s and prefill tokens/s of a
Qwen2.5-7B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests whose prompts of 2,048 tokens are
already cached (context 2,048 + tokens decoded so far, inside the benchmark context of
4,096).  It prints ONE JSON line:

  value            decoded tokens/s of the timed K steps, timed on the device with CUDA
                   events (host tokens chosen beforehand, sampling kernel included)
  e2e              the same through the Python entry point (Engine.step): every step
                   uploads its integer arrays from pinned host memory and reads the sampled
                   ids back to the host
  prefill          one prompt of 2,048 tokens in one step: tokens/s, ms, fraction of the
                   bf16 peak that its flops reach
  roofline         bytes the decode step must read (every weight once + the cache of the
                   live requests) / its time, against the HBM peak
  points           decode tokens/s at batch 1 and 64; at contexts of 8,192 and 32,768 tokens (batch 1 and 8); and at
                   the 14B and 32B shapes of the same architecture (batch 8, 2,048-token prompts), each with its
                   fraction of the copy roofline (`hbm_frac_*`)
  kernels          per workload (decode at batch 1, 8 and 64, the 2,048-token prefill) and kernel class
                   (norm, qkv, rotary+write, attention, o, gate_up, down, head, sampler): device
                   microseconds with every kernel alone (CUDA events between the launches of an
                   eager step), the bytes or flops the class has to do, and the fraction of the
                   measured peak; ``sum_over_step`` compares the classes' sum with that step's time
  env              GPU, compute capability, torch and CUDA versions, commit, time

Peaks come from MEASURED_PEAKS.json beside this file if it is there, else from the
fallback figures (6.65 TB/s copy bandwidth, 1.59 PFLOP/s bf16).  Every step streams
15 GB of weights, far more than the 126 MB of L2, so no separate L2 flush is needed.
"""

from __future__ import annotations

import argparse
import json
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# the headline configuration: the Qwen2.5-7B shape
CONFIG_7B = dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, intermediate_size=18944,
                 num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                 vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                 max_position_embeddings=32768)
PROMPT_LEN = 2048
CONTEXT = 4096
PAGE_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# Decode steps run untimed before the W warm-up steps of a decode measurement: the prompts before them are a burst of
# dense products that leaves the SM clock low under the power cap for a while, and a decode step measured right after
# it reads 2-3 % slower than the same step a tenth of a second later.
SETTLE_STEPS = 32


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                    "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index, self.rows, self.proc, self.thread = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self) -> int:
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, lo: int = 0, hi: "int | None" = None) -> dict:
        rows = [r for r in self.rows[lo:hi] if len(r) == 6] or [r for r in self.rows if len(r) == 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        mhz = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": int(rows[0][1]) if rows[0][1].isdigit() else None, "reasons": reasons,
                "samples": len(rows)}


def bench_config(cfg_raw: dict, layers: int, layers_full: int, batch: int) -> dict:
    """The ``config`` block of the bench line: every size of the measured model and workload, flat.
    Both arms (this engine and the reference) print the same keys with the same values."""
    return {"model": "Qwen2.5-7B-shaped, random weights", "layers": layers, "layers_full": layers_full,
            "hidden": cfg_raw["hidden_size"], "heads": cfg_raw["num_attention_heads"],
            "kv_heads": cfg_raw["num_key_value_heads"], "head_dim": cfg_raw["head_dim"],
            "intermediate": cfg_raw["intermediate_size"], "vocab": cfg_raw["vocab_size"],
            "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "page_size": PAGE_SIZE,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (15 GB of weights per step)"}


def model_numbers(cfg: dict, layers: int):
    """Weight bytes a decode step reads, cache bytes per token, and flops of a step of T tokens."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I
    small = layers * (2 * H + (nh + 2 * nkv) * hd) * 4 + H * 4
    weight_bytes = (layers * per_layer + V * H) * 2 + small
    kv_bytes_per_token = layers * 2 * nkv * hd * 2

    def flops(T: int, context_start: int, logit_rows: int) -> float:
        linear = 2.0 * T * layers * per_layer
        # causal attention of T new tokens over context_start cached ones: QK^T and PV
        keys = T * context_start + T * (T + 1) / 2
        attn = 4.0 * layers * nh * hd * keys
        return linear + attn + 2.0 * logit_rows * H * V
    return weight_bytes, kv_bytes_per_token, flops


def class_work(cfg: dict, layers: int, T: int, B: int, context_before: int, logit_rows: int) -> dict:
    """Per kernel class of one step (T tokens in B entries, each with ``context_before`` tokens cached): the
    bytes it has to move and the flops it has to do, summed over the layers.  Bytes: every weight once, the
    cache of the live requests once, activations in and out once (bf16; the residual stream and logits fp32)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q, kv = nh * hd, nkv * hd
    keys = B * ((T // B) * context_before + (T // B) * (T // B + 1) / 2)      # query-key pairs under the causal mask
    cached = B * (context_before + T // B)                                    # tokens whose keys and values are read
    return {
        "embed": {"bytes": T * H * (2 + 4), "flops": 0},
        # per launch: how many norm kernels run depends on the step (products of very few or of many tokens fold them in)
        "norm": {"bytes": T * H * (4 + 2 + 4 + 2) + H * 4, "flops": 0, "per_launch": True},
        "qkv": {"bytes": layers * ((q + 2 * kv) * H * 2 + T * (H + q + 2 * kv) * 2), "flops": 2.0 * layers * T * H * (q + 2 * kv)},
        # per launch too: the step's one table of angles, then a kernel per layer unless the q/k/v product carries the
        # rotation in its epilogue (very few tokens, or a prompt portion)
        "rotary+write": {"bytes": T * (q + 2 * kv) * 2 * 2, "flops": 0, "per_launch": True, "first_launch_bytes": T * (hd * 4 + 4)},
        "attention": {"bytes": layers * (cached * 2 * kv * 2 + 2 * T * q * 2), "flops": 4.0 * layers * nh * hd * keys},
        "o": {"bytes": layers * (H * q * 2 + T * (q + H) * 2), "flops": 2.0 * layers * T * q * H},
        "gate_up": {"bytes": layers * (2 * I * H * 2 + T * (H + I) * 2), "flops": 4.0 * layers * T * H * I},
        "down": {"bytes": layers * (H * I * 2 + T * (I + H) * 2), "flops": 2.0 * layers * T * H * I},
        "head": {"bytes": V * H * 2 + logit_rows * (H * 2 + V * 4), "flops": 2.0 * logit_rows * H * V},
        "sampler": {"bytes": logit_rows * V * 4, "flops": 0},
    }


def kernel_table(totals: dict, work: dict, step_us: float, peaks: dict) -> dict:
    """The ``kernels`` block of one workload: per class its device microseconds (every kernel alone, one event
    between two launches), the bytes and flops it has to do, what it achieved, and the fraction of the measured
    peak that binds it: the copy bandwidth, or the cuBLAS burst figure (the right one for a kernel timed alone)
    where the flops are the larger share."""
    classes = {}
    for name, t in sorted(totals.items(), key=lambda kv: -kv[1]["us"]):
        w = work.get(name)
        row = {"us": round(t["us"], 1), "launches": t["launches"]}
        if w is not None and t["us"] > 0:
            if w.get("per_launch"):
                first = w.get("first_launch_bytes")
                n = t["launches"] if first is None else t["launches"] - 1
                w = {"bytes": w["bytes"] * n + (first or 0), "flops": w["flops"] * t["launches"]}
            # both yardsticks; the class is judged by the one that binds it (the larger fraction)
            gbs = w["bytes"] / (t["us"] * 1e-6) / 1e9
            tf = w["flops"] / (t["us"] * 1e-6) / 1e12
            f_mem, f_flop = gbs / peaks["hbm_gbs"], tf / peaks["bf16_tflops"]
            row.update(bytes=int(w["bytes"]), gbs=round(gbs, 1))
            if w["flops"]:
                row.update(flops=w["flops"], tflops=round(tf, 1))
            if f_flop > f_mem:
                row.update(frac=round(f_flop, 3), of="bf16_tflops")
            else:
                row.update(frac=round(f_mem, 3), of="hbm_gbs")
        classes[name] = row
    total = sum(t["us"] for t in totals.values())
    return {"step_us": round(step_us, 1), "sum_us": round(total, 1), "sum_over_step": round(total / step_us, 3) if step_us else None,
            "classes": classes}


def run_ours(args) -> dict:
    import numpy as np
    import torch

    from pyre_b200 import Engine, SamplingParams
    from pyre_b200.config import config_from_dict
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import lib, ops

    peaks = load_peaks()
    cfg_raw = dict(CONFIG_7B)
    layers_full = cfg_raw["num_hidden_layers"]
    layers = args.layers or layers_full
    cfg_raw["num_hidden_layers"] = layers
    cfg = config_from_dict(cfg_raw)
    B = args.batch
    steps, warmup = args.steps, max(args.warmup, 3)
    biggest = max(B, 64 if not args.skip_points else B)
    tokens_needed = biggest * (PROMPT_LEN + 64 + SETTLE_STEPS + warmup + steps + PAGE_SIZE) + B * (2 * B + 64) + 2 * CONTEXT
    torch.cuda.set_device(0)
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", device="cuda:0", page_size=PAGE_SIZE,
                    max_cache_tokens=tokens_needed, max_num_seqs=biggest, max_num_batched_tokens=PROMPT_LEN,
                    prefill_chunk=PROMPT_LEN, max_model_len=max(CONTEXT, PROMPT_LEN + SETTLE_STEPS + warmup + steps + 2 * B + 128))
    stepper, cache = engine.stepper, engine.cache
    vocab = cfg.vocab_size
    rng = np.random.default_rng(0)
    weight_bytes, kv_per_token, flops = model_numbers(cfg_raw, layers)
    clocks = ClockSampler(0)
    clocks.start()

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---------------------------------------------------------------- prefill, 2,048 tokens in one step
    def prefill_once(rid):
        cache.begin(rid)
        ids = rng.integers(0, vocab, PROMPT_LEN).tolist()
        logits = stepper.step([StepEntry(rid, ids, [PROMPT_LEN - 1])])
        return ops.sample(logits)

    for i in range(2):
        prefill_once(("warm", i))
        cache.end(("warm", i))
    torch.cuda.synchronize()
    times = []
    for i in range(args.prefill_reps):
        a, b = ev(), ev()
        a.record()
        prefill_once(("pf", i))
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        cache.end(("pf", i))
    pf_ms = sorted(times)[len(times) // 2]
    pf_flops = flops(PROMPT_LEN, 0, 1)
    prefill = {"value": round(PROMPT_LEN / pf_ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(pf_ms, 3),
               "frac": round(pf_flops / (pf_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
               # the same against the figure of a seconds-long loop under the power cap (this step repeats back to back)
               "frac_of_sustained": round(pf_flops / (pf_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4),
               "first_ms": round(times[0], 3)}

    # ---------------------------------------------------------------- decode, device-timed
    def decode_run(batch: int, n_warm: int, n_steps: int, tag: str):
        reqs = [(tag, i) for i in range(batch)]
        for r in reqs:
            cache.begin(r)
            stepper.step([StepEntry(r, rng.integers(0, vocab, PROMPT_LEN).tolist(), [])])
        n_warm += SETTLE_STEPS
        toks = rng.integers(0, vocab, (n_warm + n_steps, batch))

        def one(k):
            logits = stepper.step([StepEntry(r, [int(toks[k, i])], [0]) for i, r in enumerate(reqs)])
            return ops.sample(logits)

        for k in range(n_warm):
            one(k)
        torch.cuda.synchronize()
        launches0, mark0 = lib.launch_count, clocks.mark()
        a, b = ev(), ev()
        a.record()
        for k in range(n_warm, n_warm + n_steps):
            one(k)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / n_steps
        info = {"ms": ms, "launches": lib.launch_count - launches0, "clock_rows": (mark0, clocks.mark()),
                "mean_context": PROMPT_LEN + n_warm + (n_steps + 1) / 2}
        for r in reqs:
            cache.end(r)
        return batch / ms * 1e3, info

    value, info = decode_run(B, warmup, steps, "dec")
    ms_per_step = info["ms"]
    step_bytes = weight_bytes + kv_per_token * info["mean_context"] * B
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"]}
    clock_summary = clocks.summary(*info["clock_rows"])

    points = {}
    if not args.skip_points:
        for b_ in (1, 64):
            v, _ = decode_run(b_, 3, max(8, steps // 2), f"p{b_}")
            points[f"decode_b{b_}"] = round(v, 1)

    # ---------------------------------------------------------------- per kernel class, every kernel alone
    kernels = {}
    if not args.no_per_kernel:
        def timed(run_step, work):
            run_step()                                     # warm: the eager path's buffers and plans
            samples = []
            for _ in range(3):
                torch.cuda.synchronize()
                a, b = ev(), ev()
                with stepper.kernel_timing() as timer:
                    a.record()
                    run_step()
                    b.record()
                    totals = timer.totals()
                samples.append((a.elapsed_time(b) * 1e3, totals))
            samples.sort(key=lambda s_: s_[0])
            step_us, totals = samples[1]
            return kernel_table(totals, work, step_us, peaks)

        for b_ in ([1, 8, 64] if not args.skip_points else [B]):
            reqs = [("k", b_, i) for i in range(b_)]
            for r in reqs:
                cache.begin(r)
                stepper.step([StepEntry(r, rng.integers(0, vocab, PROMPT_LEN).tolist(), [])])
            kernels[f"decode_b{b_}"] = timed(
                lambda: ops.sample(stepper.step([StepEntry(r, [int(rng.integers(0, vocab))], [0]) for r in reqs])),
                class_work(cfg_raw, layers, b_, b_, PROMPT_LEN + 2, b_))
            for r in reqs:
                cache.end(r)
        serial = [0]

        def one_prefill():
            serial[0] += 1
            prefill_once(("kp", serial[0]))
            cache.end(("kp", serial[0]))
        kernels[f"prefill_{PROMPT_LEN}"] = timed(one_prefill, class_work(cfg_raw, layers, PROMPT_LEN, 1, 0, 1))

    # ---------------------------------------------------------------- end to end through Engine.step
    # every request must outlive the timed steps: the first one decodes while the others' prompts (cut to what the
    # token budget leaves beside the decoded tokens) are still being read, about B * PROMPT_LEN / (budget - B) steps
    sp = SamplingParams(max_new_tokens=SETTLE_STEPS + warmup + steps + 2 * B + 64, ignore_eos=True)
    sids = [engine.add_request(rng.integers(0, vocab, PROMPT_LEN).tolist(), params=sp) for _ in range(B)]
    live = [engine._requests[sid] for sid in sids]
    while any(not r.generated for r in live):
        engine.step()                      # the prompts, one per step under the token budget
    for _ in range(SETTLE_STEPS + warmup):
        engine.step()
    torch.cuda.synchronize()
    up0 = stepper._staging.bytes_uploaded + engine.sampler.bytes_uploaded
    down0 = engine.sampler.bytes_downloaded
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    e2e = {"value": round(B * steps / dt, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": (stepper._staging.bytes_uploaded + engine.sampler.bytes_uploaded - up0) // steps,
           "d2h_bytes_per_step": (engine.sampler.bytes_downloaded - down0) // steps}
    while engine.has_unfinished():
        engine.step()
    clocks.stop()
    stepper.check_device_errors()      # a kernel that gave up waiting would have raised the device's error word

    # ---------------------------------------------------------------- further sizes of the same architecture
    # decode tokens/s at longer contexts (this model) and at the 14B and 32B shapes (full layer counts, batch 8,
    # 2,048-token prompts): device-timed like `value`, each with its fraction of the copy roofline beside it
    if not args.skip_points and not args.skip_sizes:
        def decode_point(eng, cfg_raw_, n_layers, batch, context, n_warm=SETTLE_STEPS + 8, n_steps=24):
            st_, cache_ = eng.stepper, eng.cache
            wb, kvb, _ = model_numbers(cfg_raw_, n_layers)
            reqs = [("x", batch, context, i) for i in range(batch)]
            for r in reqs:
                cache_.begin(r)
                for lo in range(0, context, 8192):
                    st_.step([StepEntry(r, rng.integers(0, cfg_raw_["vocab_size"], min(8192, context - lo)).tolist(), [])])
            toks = rng.integers(0, cfg_raw_["vocab_size"], (n_warm + n_steps, batch))
            for k in range(n_warm):      # the clocks recover from the prefill's power cap meanwhile
                ops.sample(st_.step([StepEntry(r, [int(toks[k, i])], [0]) for i, r in enumerate(reqs)]))
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            for k in range(n_warm, n_warm + n_steps):
                ops.sample(st_.step([StepEntry(r, [int(toks[k, i])], [0]) for i, r in enumerate(reqs)]))
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / n_steps
            for r in reqs:
                cache_.end(r)
            frac = (wb + kvb * (context + n_warm + n_steps / 2) * batch) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]
            return round(batch / ms * 1e3, 1), round(frac, 3)

        del stepper, cache, engine
        torch.cuda.empty_cache()
        long_cfg = dict(cfg_raw, max_position_embeddings=40960)
        eng = Engine(config=config_from_dict(long_cfg), seed=0, dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=8 * (32768 + SETTLE_STEPS + 256),
                     max_num_seqs=8, max_num_batched_tokens=8192, prefill_chunk=8192, max_model_len=40960)
        for batch, context in ((1, 8192), (1, 32768), (8, 8192), (8, 32768)):
            points[f"decode_b{batch}_ctx{context // 1024}k"], points[f"hbm_frac_b{batch}_ctx{context // 1024}k"] = \
                decode_point(eng, long_cfg, layers, batch, context)
        del eng
        torch.cuda.empty_cache()
        # many requests at the benchmark's context
        eng = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=256 * (PROMPT_LEN + SETTLE_STEPS + 64),
                     max_num_seqs=256, max_num_batched_tokens=PROMPT_LEN, prefill_chunk=PROMPT_LEN, max_model_len=CONTEXT)
        for batch in (128, 256):
            points[f"decode_b{batch}"], points[f"hbm_frac_b{batch}"] = decode_point(eng, cfg_raw, layers, batch, PROMPT_LEN, n_steps=16)
        del eng
        torch.cuda.empty_cache()
        if layers == layers_full:      # the other shapes only beside the full model
            for name in ("14b", "32b"):
                raw = dict(SHAPES[name])
                eng = Engine(config=config_from_dict(raw), seed=0, dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=8 * 2200 + 4096,
                             max_num_seqs=8, max_num_batched_tokens=2048, prefill_chunk=2048, max_model_len=4096)
                points[f"decode_b8_{name}"], points[f"hbm_frac_b8_{name}"] = decode_point(eng, raw, raw["num_hidden_layers"], 8, PROMPT_LEN)
                del eng
                torch.cuda.empty_cache()

    return {
        "metric": "decode tok/s (Qwen2.5-7B shape, batch 8, 2,048-token prompts)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "untimed_steps": SETTLE_STEPS + warmup,
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": bench_config(cfg_raw, layers, layers_full, B),
        "clocks": clock_summary, "e2e": e2e, "gpu_launches": info["launches"], "prefill": prefill,
        "roofline": roofline, "points": points, "kernels": kernels, "impl": "ours",
    }


SHAPES = {
    # the two further workloads: continuous batching at the 14B shape, mixed steps at the 32B shape
    "14b": dict(architectures=["Qwen2ForCausalLM"], hidden_size=5120, intermediate_size=13824, num_hidden_layers=48,
                num_attention_heads=40, num_key_value_heads=8, head_dim=128, vocab_size=152064, rope_theta=1e6,
                rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=32768),
    "32b": dict(architectures=["Qwen2ForCausalLM"], hidden_size=5120, intermediate_size=27648, num_hidden_layers=64,
                num_attention_heads=40, num_key_value_heads=8, head_dim=128, vocab_size=152064, rope_theta=1e6,
                rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=32768),
}


def run_workload(args) -> dict:
    """The two other workloads of the baseline description, outside the one-line contract:
    ``serve14b``: continuous batching of 64 requests (prompts uniform in 128-4096 tokens, outputs
    uniform in 64-512) on the 14B shape through Engine.generate;
    ``mixed32b``: steps of 16 decoded tokens plus a 1,024-token prompt portion at contexts up
    to 8,192 on the 32B shape."""
    import numpy as np
    import torch

    from pyre_b200 import Engine, SamplingParams
    from pyre_b200.config import config_from_dict
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import ops

    rng = np.random.default_rng(1)
    if args.workload == "serve14b":
        raw = dict(SHAPES["14b"])
        if args.layers:
            raw["num_hidden_layers"] = args.layers
        cfg = config_from_dict(raw)
        n_req = 64
        prompts = [rng.integers(0, cfg.vocab_size, int(rng.integers(128, 4097))).tolist() for _ in range(n_req)]
        outs_len = [int(rng.integers(64, 513)) for _ in range(n_req)]
        need = sum(len(p) + o for p, o in zip(prompts, outs_len))
        eng = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=int(need * args.cache_fraction),
                     max_num_seqs=64, max_num_batched_tokens=4096, prefill_chunk=2048, max_model_len=8192, record_steps=True)
        params = [SamplingParams(max_new_tokens=o, ignore_eos=True) for o in outs_len]
        eng.generate(prompts[:2], params[:2])       # warm-up: builds, graphs of small shapes
        torch.cuda.synchronize()
        eng.step_log.clear()
        t0 = time.perf_counter()
        res = eng.generate(prompts, params)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        st = eng.stats()
        eng.cache.check()
        n_out = sum(len(r.token_ids) for r in res)
        n_in = sum(len(p) for p in prompts)
        # the host's share: its own work per step against the time it spent waiting for the GPU.  Steps with prompt
        # tokens run kernel by kernel (hundreds of launches), decode-only steps replay a captured graph.
        log = eng.step_log
        mixed = [r for r in log if r["prompt_tokens"]]
        host = {"steps": len(log), "steps_with_prompt_tokens": len(mixed),
                "host_ms_total": round(sum(r["host_ms"] for r in log), 1), "wait_ms_total": round(sum(r["wait_ms"] for r in log), 1),
                "host_ms_per_prompt_step": round(sum(r["host_ms"] for r in mixed) / max(1, len(mixed)), 3),
                "host_ms_per_decode_step": round(sum(r["host_ms"] for r in log if not r["prompt_tokens"]) / max(1, len(log) - len(mixed)), 3),
                "steps_the_host_did_not_wait_in": sum(1 for r in log if r["wait_ms"] < 0.05)}
        return {"workload": "serve14b", "layers": cfg.num_hidden_layers, "requests": n_req, "prompt_tokens": n_in,
                "output_tokens": n_out, "seconds": round(dt, 3), "output_tok_s": round(n_out / dt, 1),
                "total_tok_s": round((n_in + n_out) / dt, 1), "steps": st["steps"], "preempted": st["preempted"],
                "cache_tokens": int(need * args.cache_fraction), "finished": sum(r.finish_reason == "length" for r in res),
                "graph_captures": eng.stepper.graph_captures, "graph_replays": eng.stepper.graph_replays,
                "capture_seconds": round(eng.stepper.capture_seconds, 3), "host": host}
    raw = dict(SHAPES["32b"])
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = config_from_dict(raw)
    n_dec, chunk, ctx = 16, 1024, 8192
    eng = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=(n_dec + 1) * (ctx + 64),
                 max_num_seqs=n_dec + 1, max_num_batched_tokens=4096, prefill_chunk=4096, max_model_len=ctx + 64)
    st, cache = eng.stepper, eng.cache
    reqs = list(range(n_dec))
    for r in reqs:                              # decoding requests at contexts between 2,048 and 8,000
        cache.begin(r)
        n = int(rng.integers(2048, ctx - 200))
        for lo in range(0, n, 4096):
            st.step([StepEntry(r, rng.integers(0, cfg.vocab_size, min(4096, n - lo)).tolist(), [])])
    cache.begin("p")
    times = []
    for k in range(ctx // chunk - 1):           # the prompt grows by 1,024 tokens per step beside 16 decoded tokens
        entries = [StepEntry(r, [int(rng.integers(0, cfg.vocab_size))], [0]) for r in reqs]
        entries.append(StepEntry("p", rng.integers(0, cfg.vocab_size, chunk).tolist(), [chunk - 1]))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ops.sample(st.step(entries))
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    cache.check()
    ms = sorted(times[1:])[len(times[1:]) // 2]
    return {"workload": "mixed32b", "layers": cfg.num_hidden_layers, "tokens_per_step": n_dec + chunk,
            "ms_per_step_median": round(ms, 2), "tok_s": round((n_dec + chunk) / ms * 1e3, 1),
            "ms_first_last": [round(times[1], 2), round(times[-1], 2)]}


def run_sweep(args) -> dict:
    """Decode throughput over a grid of batch sizes and context lengths and prefill throughput over
    several portion lengths on the 7B shape, each with its fraction of the roofline (device-timed,
    the same way as the headline numbers).  One JSON object; not part of the one-line contract."""
    import numpy as np
    import torch

    from pyre_b200 import Engine
    from pyre_b200.config import config_from_dict
    from pyre_b200.engine.step import StepEntry
    from pyre_b200.kernels import ops

    peaks = load_peaks()
    cfg_raw = dict(CONFIG_7B)
    layers = args.layers or cfg_raw["num_hidden_layers"]
    cfg_raw["num_hidden_layers"] = layers
    cfg_raw["max_position_embeddings"] = 40960
    cfg = config_from_dict(cfg_raw)
    weight_bytes, kv_per_token, flops = model_numbers(cfg_raw, layers)
    grid = [(1, 512), (1, 8192), (1, 32768), (8, 512), (8, 2048), (8, 8192), (8, 32768), (32, 2048), (64, 512), (64, 2048),
            (64, 8192), (128, 2048)]
    biggest = max(b * (c + SETTLE_STEPS + 64) for b, c in grid)
    eng = Engine(config=cfg, seed=0, dtype="bfloat16", page_size=PAGE_SIZE, max_cache_tokens=biggest + 8192,
                 max_num_seqs=128, max_num_batched_tokens=8192, prefill_chunk=8192, max_model_len=40960)
    st, cache = eng.stepper, eng.cache
    rng = np.random.default_rng(0)
    vocab = cfg.vocab_size

    def ev():
        return torch.cuda.Event(enable_timing=True)

    decode = []
    for batch, ctx in grid:
        reqs = [("d", batch, ctx, i) for i in range(batch)]
        for r in reqs:
            cache.begin(r)
            for lo in range(0, ctx, 8192):
                st.step([StepEntry(r, rng.integers(0, vocab, min(8192, ctx - lo)).tolist(), [])])
        n_warm, n_steps = SETTLE_STEPS + 8, 32
        toks = rng.integers(0, vocab, (n_warm + n_steps, batch))
        for k in range(n_warm):
            ops.sample(st.step([StepEntry(r, [int(toks[k, i])], [0]) for i, r in enumerate(reqs)]))
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for k in range(n_warm, n_warm + n_steps):
            ops.sample(st.step([StepEntry(r, [int(toks[k, i])], [0]) for i, r in enumerate(reqs)]))
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / n_steps
        step_bytes = weight_bytes + kv_per_token * (ctx + n_warm + n_steps / 2) * batch
        decode.append({"batch": batch, "context": ctx, "ms_per_step": round(ms, 3), "tok_s": round(batch / ms * 1e3, 1),
                       "hbm_frac": round(step_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3)})
        for r in reqs:
            cache.end(r)
    prefill = []
    for T, start in ((512, 0), (2048, 0), (4096, 0), (8192, 0), (2048, 8192), (2048, 30720), (512, 30720), (128, 30720)):
        times = []
        for rep in range(4):
            r = ("p", T, start, rep)
            cache.begin(r)
            for lo in range(0, start, 8192):
                st.step([StepEntry(r, rng.integers(0, vocab, min(8192, start - lo)).tolist(), [])])
            ids = rng.integers(0, vocab, T).tolist()
            torch.cuda.synchronize()
            a, b = ev(), ev()
            a.record()
            ops.sample(st.step([StepEntry(r, ids, [T - 1])]))
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
            cache.end(r)
        ms = sorted(times[1:])[len(times[1:]) // 2]
        prefill.append({"tokens": T, "context_before": start, "ms": round(ms, 3), "tok_s": round(T / ms * 1e3, 1),
                        "flops_frac": round(flops(T, start, 1) / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 3)})
    cache.check()
    st.check_device_errors()
    return {"workload": "sweep", "layers": layers, "peaks": peaks, "decode": decode, "prefill": prefill}


def environment() -> dict:
    """Where a number was measured, recorded with it as the reference's harness does (bench/harness.py:49-67):
    GPU, compute capability, torch and CUDA versions, the checkout's commit, the time."""
    env = {"gpu": None, "capability": None, "torch": None, "cuda": None, "git": None,
           "time": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
    try:
        import torch
        env["torch"], env["cuda"] = torch.__version__, torch.version.cuda
        if torch.cuda.is_available():
            env["gpu"] = torch.cuda.get_device_name(0)
            env["capability"] = ".".join(str(v) for v in torch.cuda.get_device_capability(0))
    except Exception:       # the record must never cost the measurement
        pass
    try:
        out = subprocess.run(["git", "-C", str(ROOT), "rev-parse", "--short", "HEAD"], capture_output=True, text=True,
                             timeout=10)
        env["git"] = out.stdout.strip() or None
    except (OSError, subprocess.SubprocessError):
        pass
    return env


def run_reference(args) -> dict:
    from baseline import reference_arm
    layers = args.layers or CONFIG_7B["num_hidden_layers"]
    return reference_arm.run(args, CONFIG_7B, PROMPT_LEN,
                             bench_config(CONFIG_7B, layers, CONFIG_7B["num_hidden_layers"], args.batch))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0 = all)")
    ap.add_argument("--prefill-reps", type=int, default=5)
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    ap.add_argument("--skip-sizes", action="store_true",
                    help="leave out the points at longer contexts and at the 14B and 32B shapes")
    ap.add_argument("--no-per-kernel", action="store_true",
                    help="leave out the `kernels` block (device time, bytes or flops and fraction of the peak per kernel class)")
    ap.add_argument("--workload", choices=["serve14b", "mixed32b", "sweep"], default=None,
                    help="run one of the two other baseline workloads, or a sweep over batch sizes, context lengths and "
                         "portion lengths on the 7B shape, instead (prints its own JSON line)")
    ap.add_argument("--cache-fraction", type=float, default=1.0,
                    help="serve14b: cache capacity as a fraction of what all requests need at once (< 1 forces preemption)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.workload:
        result = run_sweep(args) if args.workload == "sweep" else run_workload(args)
        result["env"] = environment()
        print(json.dumps(result))
        return 0
    result = run_reference(args) if args.impl == "reference" else run_ours(args)
    if "unavailable" not in result:
        result["env"] = environment()
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
