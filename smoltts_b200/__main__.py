"""Command line of the package: ``python -m smoltts_b200 <command> ...``.

  generate   token ids in, token ids out, for any registered language model (continuous batching, the library's sampler)
  trace      replay a schedule of steps (JSON lines on standard input) through a model's engine and write the logits
  convert    trainer checkpoint -> exported DualAR checkpoint (same as ``python -m smoltts_b200.convert``)
  build      compile the CUDA libraries in-tree
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _dtype(name: str):
    import torch

    return {"bfloat16": torch.bfloat16, "float32": torch.float32}[name]


def cmd_generate(a) -> int:
    from .registry import load_model
    from .serving import TokenBatcher

    prompts = [[int(t) for t in p.split(",")] for p in a.prompt]
    longest = max(len(p) for p in prompts) + a.max_new_tokens
    model = load_model(a.model, dtype=_dtype(a.dtype), max_tokens=a.max_tokens or 4 * (longest + 64), max_seqs=a.max_seqs)
    batcher = TokenBatcher(model, temp=a.temp, top_k=a.top_k, top_p=a.top_p, min_p=a.min_p, seed=a.seed, eos_id=a.eos)
    for p, out in zip(prompts, batcher.generate(prompts, a.max_new_tokens)):
        print(json.dumps({"prompt": p, "tokens": out}))
    return 0


def cmd_trace(a) -> int:
    """Standard input: one JSON object a line, {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}.  For a step
    with wanted places, writes <out>/<step>.f32 (little-endian fp32 [wanted, vocab], entries' order); prints 'done <step>'."""
    import torch

    from .registry import load_model
    from .serving import TokenBatcher

    try:
        model = load_model(a.model, dtype=_dtype(a.dtype), max_tokens=a.max_tokens, max_seqs=a.max_seqs)
    except TypeError:
        print("this design's engine does not take explicit-token steps", file=sys.stderr)
        return 4
    batcher = TokenBatcher(model)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in step["entries"]]
        logits = batcher.feed(entries, end=step.get("end", []))
        if logits.shape[0]:
            data = logits.to(torch.float32).cpu().contiguous().numpy()
            tmp = os.path.join(a.out, f".{step['step']}.part")
            data.astype("<f4").tofile(tmp)
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        else:
            torch.cuda.synchronize()
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    model.check_device_errors()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m smoltts_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate token ids with a language model")
    g.add_argument("--model", required=True)
    g.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("--temp", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--eos", type=int, default=None)
    g.add_argument("--max-tokens", type=int, default=0, help="positions of the key/value pool (default: fits the prompts)")
    g.add_argument("--max-seqs", type=int, default=4)
    g.set_defaults(fn=cmd_generate)
    t = sub.add_parser("trace", help="replay a step schedule and write logits")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True, help="positions live requests hold at any time (rounded up to pages)")
    t.add_argument("--max-seqs", type=int, default=4)
    t.set_defaults(fn=cmd_trace)
    c = sub.add_parser("convert", help="trainer checkpoint -> exported checkpoint")
    c.add_argument("rest", nargs=argparse.REMAINDER)
    b = sub.add_parser("build", help="compile the CUDA libraries")
    b.add_argument("--only", choices=["core", "lm"], default=None)
    a = ap.parse_args(argv)
    if a.cmd == "convert":
        from . import convert

        return convert.main(a.rest) or 0
    if a.cmd == "build":
        from . import build

        for tgt in build.TARGETS:
            if a.only in (None, tgt):
                print(build.build(target=tgt))
        return 0
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
