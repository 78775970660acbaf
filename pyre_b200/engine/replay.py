"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no model code of its own: it opens the model folder through
the registry, builds the same ``Model``, ``CacheManager`` and ``Stepper`` that generation
uses, and calls ``Stepper.step`` once per line of its input.

Input, one JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["b"]}

``entries``: per request its next tokens and the places among them whose logits are
wanted; all entries of a line are one batch.  An id seen for the first time begins a
request.  ``end``: requests that are finished after this step; their pages and state slot
go back to the pools.  For a step with wanted places the fp32 logits ``[wanted, vocab]``
are written little-endian to ``<out>/<step>.f32``, in the order of the entries and of
``want``.  After every step a line ``done <step>`` goes to standard output.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from ..cache import CacheManager
from ..models.model import Model, load_model
from .step import StepEntry, Stepper

DEFAULT_PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 64
TOKEN_QUANTUM = 64      # --max-tokens counts each live request rounded up to a multiple of this (or of the page size)


def pages_for_max_tokens(max_tokens: int, page_size: int, max_requests: int = MAX_LIVE_REQUESTS) -> int:
    """Pages that hold live requests of ``max_tokens`` tokens in all, each request's count rounded up to a
    multiple of 64 (or of the page size, if that is larger).  When the page size divides that quantum the
    answer is exact.  Otherwise (pages of 24 or 48 tokens, say) every request but one may need one page more
    than its share of the sum, so that many pages are added."""
    quantum = max(TOKEN_QUANTUM, page_size)
    pages = max(1, -(-int(max_tokens) // page_size))
    if quantum % page_size:
        pages += max(0, min(max_requests, int(max_tokens) // quantum) - 1)
    return pages


def build_runtime(model_dir, dtype, max_tokens: int, page_size: int = DEFAULT_PAGE_SIZE,
                  device: str = "cuda:0", max_requests: int = MAX_LIVE_REQUESTS, poison: bool = False):
    """Model, cache manager and stepper for a model folder: the pieces every entry point shares."""
    if not torch.cuda.is_available():
        raise RuntimeError("pyre_b200 needs a CUDA device (sm_100a); there is no CPU path")
    model, _config = load_model(model_dir, device, dtype)
    cache, stepper = runtime_for_model(model, max_tokens, page_size, max_requests, poison)
    return model, cache, stepper


def runtime_for_model(model: Model, max_tokens: int, page_size: int = DEFAULT_PAGE_SIZE,
                      max_requests: int = MAX_LIVE_REQUESTS, poison: bool = False, cuda_graphs: bool = True):
    """Cache manager and stepper for a model that already has its weights."""
    num_pages = pages_for_max_tokens(max_tokens, page_size, max_requests)
    cache = CacheManager(model.kv_groups, model.state_groups, page_size, num_pages, max_requests, model.dtype,
                         model.device)
    cache.set_poison(poison)
    stepper = Stepper(model, cache, max_positions=model.spec.max_positions or None, cuda_graphs=cuda_graphs)
    return cache, stepper


class TraceError(ValueError):
    """A line of the trace that cannot be run: not JSON, a field missing or of the wrong kind, a request
    ended that is not live, a wanted place outside the entry's tokens, no pages left."""


def _parse_step(line: str, number: int):
    try:
        rec = json.loads(line)
    except json.JSONDecodeError as e:
        raise TraceError(f"line {number}: not JSON ({e.msg} at column {e.colno})") from None
    if not isinstance(rec, dict) or "step" not in rec:
        raise TraceError(f"line {number}: a step is an object with a \"step\" field")
    entries = rec.get("entries", [])
    end = rec.get("end", [])
    if not isinstance(entries, list) or not isinstance(end, list):
        raise TraceError(f"line {number} (step {rec['step']}): \"entries\" and \"end\" are lists")
    for e in entries:
        if not isinstance(e, dict) or "id" not in e or not isinstance(e.get("tokens"), list) \
                or not isinstance(e.get("want", []), list):
            raise TraceError(f"line {number} (step {rec['step']}): an entry is an object with \"id\", a list "
                             f"\"tokens\" and an optional list \"want\"")
        if not all(isinstance(t, int) and not isinstance(t, bool) for t in list(e["tokens"]) + list(e.get("want", []))):
            raise TraceError(f"line {number} (step {rec['step']}): tokens and wanted places are integers")
    return rec["step"], entries, end


def replay(stepper: Stepper, lines, out_dir: Path, done=print) -> None:
    cache = stepper.cache
    out_dir.mkdir(parents=True, exist_ok=True)
    for number, line in enumerate(lines, 1):
        line = line.strip()
        if not line:
            continue
        step, raw_entries, end = _parse_step(line, number)
        try:
            entries = []
            for e in raw_entries:
                rid = e["id"]
                if rid not in cache.lengths:
                    cache.begin(rid)
                entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
            if entries:
                logits = stepper.step(entries)
                if logits.shape[0]:
                    logits.to("cpu").numpy().astype("<f4", copy=False).tofile(out_dir / f"{step}.f32")
            for rid in end:
                cache.end(rid)
        except (ValueError, MemoryError) as e:     # the stepper's and the cache manager's refusals
            raise TraceError(f"line {number} (step {step}): {e}") from e
        done(f"done {step}")
    if torch.device(stepper.device).type == "cuda":
        torch.cuda.synchronize(stepper.device)
    stepper.check_device_errors()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=DEFAULT_PAGE_SIZE, help="tokens per cache page (any size the engine takes)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--poison-freed-pages", action="store_true",
                    help="debug: fill pages with NaN when they go back to the pool")
    args = ap.parse_args(argv)
    if args.page_size <= 0:
        ap.error("--page-size must be positive")
    _, _, stepper = build_runtime(args.model, args.dtype, args.max_tokens, args.page_size, args.device,
                                  poison=args.poison_freed_pages)

    def done(msg):
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    try:
        replay(stepper, sys.stdin, Path(args.out), done)
    except TraceError as e:
        print(f"trace_run: {e}", file=sys.stderr)
        return 1
    return 0
