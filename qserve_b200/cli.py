"""Command line of the hybrid-decoder engine.

  python -m qserve_b200.cli generate --model DIR --prompt 5,17,3 [--prompt ...] [--max-new-tokens N] [--temperature T] [--top-k K] [--top-p P]
  python -m qserve_b200.cli trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N      (steps on standard input)

`--model` is a folder with config.json (its "architecture" picks the model class, qserve_b200.modelcfg.ARCHITECTURES) and
model.safetensors.  The shared library is built on first use if it is missing (nvcc, sm_100a).
"""
from __future__ import annotations

import argparse
import sys


def _engine(args, max_tokens: int):
    from .build import ensure_built

    ensure_built()
    import torch

    from .engine import Engine

    if not torch.cuda.is_available():
        print("qserve_b200 needs a CUDA device (there is no CPU path)", file=sys.stderr)
        raise SystemExit(4)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    return Engine.from_dir(args.model, dtype, max_tokens=max_tokens, max_seqs=args.max_seqs, page_size=args.page_size, use_graphs=not args.no_graphs)


def _common(p):
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    p.add_argument("--max-seqs", type=int, default=4, help="state slots = most live sequences")
    p.add_argument("--page-size", type=int, default=64)
    p.add_argument("--no-graphs", action="store_true", help="launch decode-only steps eagerly instead of replaying a captured CUDA graph")


def trace_main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trace_run", description="replay a trace of token batches through the engine and write logits")
    _common(p)
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True, help="positions the page pool holds (rounded up to whole pages per sequence)")
    args = p.parse_args(argv)
    engine = _engine(args, args.max_tokens)
    from .engine import replay_trace

    replay_trace(engine, sys.stdin, args.out)
    return 0


def generate_main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="generate")
    _common(p)
    p.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    p.add_argument("--max-new-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--max-tokens", type=int, default=0, help="page pool size in positions (default: enough for all prompts)")
    args = p.parse_args(argv)
    from .engine import SamplingParams

    prompts = [[int(t) for t in s.split(",") if t.strip()] for s in args.prompt]
    need = sum(-(-(len(q) + args.max_new_tokens) // args.page_size) * args.page_size for q in prompts)
    engine = _engine(args, args.max_tokens or need)
    sp = SamplingParams(args.temperature, args.top_k, args.top_p, args.max_new_tokens)
    for out in engine.generate(prompts, [sp] * len(prompts)):
        print(",".join(str(t) for t in out))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in ("generate", "trace"):
        print(__doc__, file=sys.stderr)
        return 2
    return trace_main(argv[1:]) if argv[0] == "trace" else generate_main(argv[1:])


if __name__ == "__main__":
    raise SystemExit(main())
