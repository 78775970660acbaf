"""Small, fixed workloads for profilers (``ncu``): a few decode steps or one prompt portion
of a Qwen2.5-7B-shaped model with few layers and random weights, every kernel launched
individually (no CUDA graphs) so that a profiler sees each one.

    python -m pyre_b200.profiling decode  --layers 2 --batch 8 --context 2048 --steps 3
    python -m pyre_b200.profiling prefill --layers 2 --tokens 2048

A few GB on the device at most; ends by itself in seconds.
"""

from __future__ import annotations

import argparse
import sys

SHAPE_7B = dict(architectures=["Qwen2ForCausalLM"], hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                num_attention_heads=28, num_key_value_heads=4, head_dim=128, vocab_size=152064, rope_theta=1e6,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=32768)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("mode", choices=["decode", "prefill"])
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--dtype", default="bfloat16")
    args = ap.parse_args(argv)

    import numpy as np
    import torch

    from .config import config_from_dict
    from .engine.engine import Engine
    from .engine.step import StepEntry
    from .kernels import lib, ops

    cfg = config_from_dict(dict(SHAPE_7B, num_hidden_layers=args.layers))
    tokens = args.batch * (args.context + args.steps + 32) if args.mode == "decode" else 2 * args.tokens + 64
    eng = Engine(config=cfg, seed=0, dtype=args.dtype, max_cache_tokens=tokens, max_num_seqs=max(args.batch, 2),
                 max_num_batched_tokens=max(args.tokens, args.context), prefill_chunk=max(args.tokens, args.context),
                 cuda_graphs=False)
    rng = np.random.default_rng(0)
    st, cache = eng.stepper, eng.cache
    # the measured region is bracketed by cudaProfilerStart/Stop: with `ncu --profile-from-start off`
    # only its kernels are captured
    if args.mode == "prefill":
        for i in range(2):
            cache.begin(i)
            if i == 1:
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
            logits = st.step([StepEntry(i, rng.integers(0, cfg.vocab_size, args.tokens).tolist(), [args.tokens - 1])])
            ops.sample(logits)
            torch.cuda.synchronize()
            print(f"prefill {i}: launches so far {lib.launch_count}", file=sys.stderr)
        torch.cuda.profiler.stop()
    else:
        reqs = list(range(args.batch))
        for r in reqs:
            cache.begin(r)
            st.step([StepEntry(r, rng.integers(0, cfg.vocab_size, args.context).tolist(), [])])
        torch.cuda.synchronize()
        print(f"prompts cached: launches so far {lib.launch_count}", file=sys.stderr)
        for k in range(args.steps):
            if k == args.steps - 1:
                torch.cuda.synchronize()
                torch.cuda.profiler.start()
            logits = st.step([StepEntry(r, [int(rng.integers(0, cfg.vocab_size))], [0]) for r in reqs])
            ops.sample(logits)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(f"decoded {args.steps} steps: launches so far {lib.launch_count}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
