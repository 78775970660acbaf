"""Command line, in the manner of the reference's scripts: argparse, ``--model`` naming a
model folder, ``--device``, ``--dtype``, ``--max-new-tokens``, ``--out`` for a JSON result
file (scripts/serve.py:16-21, bench/bench_pyre.py:52-59, bench/bench_batch.py:49-54,
scripts/diagnose_parity.py:77-83).  Token ids in, token ids out.

    python -m pyre_b200 generate --model DIR --prompt-ids 5,17,3 --max-new-tokens 16
    python -m pyre_b200 random-model --config config.json --seed 0 --out DIR
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


SIZES = ("Sizes: a head size must be a multiple of 16 up to 256 (others are refused when the model is built).  "
         "In bfloat16, head sizes up to 128 run on the tensor-core attention kernels, larger ones on the exact "
         "fp32-arithmetic kernel, as every float32 run does (slower).  A bfloat16 product whose inner size is no "
         "multiple of 8 (a hidden or feed-forward size like 92) goes to a library product; every other product and "
         "every size of the supported checkpoints runs on the package's own kernels.  Pages of the tcgen05 prompt "
         "attention are powers of two from 4 tokens; other page sizes use the mma.sync kernels.")


def _parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_generate(args) -> int:
    import torch

    from .config import EngineConfig
    from .engine.engine import Engine
    from .sampling import SamplingParams

    prompts = [_parse_ids(p) for p in args.prompt_ids or []]
    if args.prompt_ids_file:
        for line in Path(args.prompt_ids_file).read_text().splitlines():
            if line.strip():
                prompts.append(_parse_ids(line))
    if not prompts:
        print("no prompts: give --prompt-ids or --prompt-ids-file", file=sys.stderr)
        return 2
    ec = EngineConfig(dtype=args.dtype, device=args.device, page_size=args.page_size, num_pages=args.num_pages,
                      cache_memory_fraction=args.cache_memory_fraction, lookahead=not args.no_lookahead,
                      max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_batched_tokens,
                      prefill_chunk=args.prefill_chunk, record_steps=bool(args.step_log))
    print(f"loading {args.model} on {args.device} ...", file=sys.stderr)
    engine = Engine(args.model, ec)
    params = [SamplingParams(temperature=args.temperature, seed=args.seed + i, max_new_tokens=args.max_new_tokens,
                             eos_id=args.eos_id) for i in range(len(prompts))]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_new = sum(len(o.token_ids) for o in outs)
    result = {"model": str(args.model), "dtype": args.dtype, "seconds": dt, "new_tokens": n_new,
              "tokens_per_second": n_new / dt if dt > 0 else None, "stats": engine.stats(),
              "outputs": [{"seq_id": o.seq_id, "prompt_ids": o.prompt_ids, "token_ids": o.token_ids,
                           "finish_reason": o.finish_reason} for o in outs]}
    for o in outs:
        print(" ".join(str(t) for t in o.token_ids))
    if args.step_log:
        Path(args.step_log).parent.mkdir(parents=True, exist_ok=True)
        Path(args.step_log).write_text("".join(json.dumps(rec) + "\n" for rec in engine.step_log))
        print(f"wrote {args.step_log} ({len(engine.step_log)} steps)", file=sys.stderr)
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps(result, indent=2))
        print(f"wrote {args.out}", file=sys.stderr)
    return 0


def cmd_random_model(args) -> int:
    import torch

    from .config import config_from_dict
    from .weights import write_random_model

    raw = json.loads(Path(args.config).read_text())
    cfg = config_from_dict(raw)
    store = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.store_dtype]
    out = write_random_model(args.out, cfg, args.seed, store)
    print(f"wrote {out}/config.json and {out}/model.safetensors (seed {args.seed})")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pyre_b200", description=__doc__.split("\n\n")[0], epilog=SIZES)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids", epilog=SIZES)
    g.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    g.add_argument("--device", default="cuda:0")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("--prompt-ids", action="append", help="token ids of one prompt, e.g. 5,17,3 (repeatable)")
    g.add_argument("--prompt-ids-file", help="file with one prompt per line")
    g.add_argument("--max-new-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    g.add_argument("--seed", type=int, default=0, help="sampling seed of the first prompt; prompt i uses seed + i")
    g.add_argument("--eos-id", type=int, default=None)
    g.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    g.add_argument("--num-pages", type=int, default=None, help="pages of the cache pool")
    g.add_argument("--no-lookahead", action="store_true",
                   help="read every step's ids before the next step is started (the strictly sequential loop)")
    g.add_argument("--cache-memory-fraction", type=float, default=None,
                   help="without --num-pages: size the cache to this fraction of the device memory left after loading")
    g.add_argument("--max-num-seqs", type=int, default=64, help="most requests live at once")
    g.add_argument("--max-batched-tokens", type=int, default=2048, help="token budget of one step")
    g.add_argument("--prefill-chunk", type=int, default=2048, help="most prompt tokens of a request per step")
    g.add_argument("--out", default=None, help="write a JSON result file")
    g.add_argument("--step-log", default=None,
                   help="write one JSON line per step: tokens, requests, pages free, preemptions, host time")
    g.set_defaults(func=cmd_generate)

    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json of a registered architecture")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--store-dtype", choices=["float32", "bfloat16"], default="float32")
    r.set_defaults(func=cmd_random_model)

    args = ap.parse_args(argv)
    return args.func(args)


if __name__ == "__main__":
    sys.exit(main())
