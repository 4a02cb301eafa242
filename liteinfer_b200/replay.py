"""Trace replay: feeds given token ids through the model step by step and writes logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It samples nothing and owns no model code: it builds the same `ModelRunner`
that generation uses (same loader, cache manager, step function and kernels) and
calls `step` once per line of its input.  Each input line is one JSON object:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a line are one batch.  `want` lists the places among an entry's
tokens whose logits are asked for; for a step that wants any, the logits are
written to `<out>/<step>.f32` as little-endian float32 [wanted, vocab], in the
order of the entries and of `want`.  `end` lists requests that are finished
after the step; their pages and state slots go back to the pool.  After every
step a line `done <step>` is printed and flushed.  The cache pool is sized for
`--max-tokens` tokens (each request's count rounded up to a multiple of 64), so
pages are reused as requests come and go.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch


def _parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    parser.add_argument("--max-requests", type=int, default=8, help="most requests live at a time")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false",
                        help="launch every step kernel by kernel (by default steps are replayed from CUDA graphs, "
                             "as the engine does when it serves)")
    return parser.parse_args(argv)


def main(argv=None) -> int:
    args = _parse_args(argv)
    if args.max_tokens < 1:
        print("trace_run: --max-tokens must be >= 1", file=sys.stderr)
        return 2
    if args.page_size < 1 or 64 % args.page_size:
        print("trace_run: --page-size must divide 64", file=sys.stderr)
        return 2
    from liteinfer_b200.config.engine_config import parse_dtype
    from liteinfer_b200.engine.loading import build_runner
    from liteinfer_b200.engine.runner import StepEntry

    dtype = parse_dtype(args.dtype)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    num_pages = -(-args.max_tokens // args.page_size)
    print(f"[trace_run] loading {args.model} ({args.dtype}); cache of {num_pages} pages x {args.page_size} tokens",
          file=sys.stderr, flush=True)
    runner = build_runner(args.model, dtype, args.device, args.page_size, num_pages, args.max_requests)
    if args.cuda_graphs and args.device.startswith("cuda"):
        runner.enable_decode_graphs(args.max_requests, num_pages * args.page_size)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(str(e["id"]), [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])])
                   for e in record.get("entries", [])]
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                array = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                np.ascontiguousarray(array).tofile(out_dir / f"{step}.f32")
        for request_id in record.get("end", []):
            runner.release(str(request_id))
        if args.device.startswith("cuda"):
            torch.cuda.synchronize()
        print(f"done {step}", flush=True)
    runner.check_kernels()
    return 0


if __name__ == "__main__":
    sys.exit(main())
