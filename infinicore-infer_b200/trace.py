"""Trace replay: feed given token ids through the model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as ONE call of the engine's step function, the same one that
generation uses: same model, cache and kernels.  For a step in which something is wanted the
logits of the wanted places are written to ``<out>/<step>.f32`` as little-endian float32
``[wanted, vocab]``, in the order of the entries and of ``want``.  After every step the
program prints ``done <step>`` and flushes.  Nothing is sampled.

The reference's nearest instrument is ``perplexity()``, which pushes whole sequences through
``forwardBatch`` and reads every row's logits (scripts/jiuge.py:588-639).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_SIZE = 16       # divides 64, so a pool of N tokens holds every request rounded up to 64


def replay(engine, records, out_dir=None, on_done=None):
    """Run trace records (dicts as described above) through ``engine.step``.

    Returns ``{step: float32 array [wanted, vocab]}`` for the steps in which something was
    wanted; with ``out_dir`` each array is also written to ``<out_dir>/<step>.f32``.
    ``on_done(step)`` is called after each step.
    """
    import torch
    from .engine import StepEntry
    results = {}
    for rec in records:
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", ())]
        logits = engine.step(entries)
        if logits.shape[0]:
            data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
            results[step] = data
            if out_dir is not None:
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                with open(tmp, "wb") as f:
                    f.write(data.tobytes())
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        engine.check()
        for rid in rec.get("end", ()):
            if engine.cache.is_live(rid):
                engine.end(rid)
        if on_done is not None:
            on_done(step)
    return results


def _records(stream):
    for line in stream:
        line = line.strip()
        if line:
            yield json.loads(line)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    ap.add_argument("--no-graphs", action="store_true", help="run decode steps without CUDA graphs")
    args = ap.parse_args(argv)

    import torch
    from .engine import Engine

    os.makedirs(args.out, exist_ok=True)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    cache_tokens = max(64, (args.max_tokens + 63) // 64 * 64)
    print(f"[trace_run] loading {args.model} in {args.dtype}", file=sys.stderr, flush=True)
    engine = Engine.from_folder(args.model, dtype=dtype, device="cuda:0", cache_tokens=cache_tokens,
                                page_size=args.page_size, max_requests=16,
                                max_step_tokens=cache_tokens, use_graphs=not args.no_graphs)
    print("[trace_run] ready", file=sys.stderr, flush=True)
    replay(engine, _records(sys.stdin), args.out, on_done=lambda s: print(f"done {s}", flush=True))
    return 0


if __name__ == "__main__":
    sys.exit(main())
