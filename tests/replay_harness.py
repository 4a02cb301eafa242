"""Builds replay traces (the four ways of cutting the same requests) and runs them.

A *request* is a list of token ids (prompt and forced continuation alike: replay
never samples).  A *trace* is a list of steps in the format of `bin/trace_run`.
`expected_logits` computes, with the plain implementation, the logits every
wanted place must have.
"""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

import plain_llama

ROOT = Path(__file__).resolve().parent.parent


def _round64(n: int) -> int:
    return -(-n // 64) * 64


class Trace:
    def __init__(self) -> None:
        self.steps: list[dict] = []
        self.wanted: list[list[tuple[str, int]]] = []   # per step: (request, absolute position) of each wanted row
        self._held: dict[str, int] = {}
        self.max_tokens = 0
        self.max_live = 0

    def add(self, entries: list[tuple[str, list[int], list[int]]], end: list[str] = ()) -> None:
        """entries: (request id, tokens, wanted places among them)."""
        wanted = []
        for request_id, tokens, want in entries:
            start = self._held.get(request_id, 0)
            self._held[request_id] = start + len(tokens)
            wanted.extend((request_id, start + w) for w in want)
        self.max_tokens = max(self.max_tokens, sum(_round64(n) for n in self._held.values()))
        self.max_live = max(self.max_live, len(self._held))
        self.steps.append({"step": len(self.steps),
                           "entries": [{"id": r, "tokens": list(t), "want": list(w)} for r, t, w in entries],
                           "end": list(end)})
        self.wanted.append(wanted)
        for request_id in end:
            del self._held[request_id]


def whole(trace: Trace, requests: dict[str, list[int]], tag: str = "w") -> None:
    """Each request alone and whole, logits wanted everywhere."""
    for name, tokens in requests.items():
        rid = f"{tag}-{name}"
        trace.add([(rid, tokens, list(range(len(tokens))))], end=[rid])


def tail_decoded(trace: Trace, requests: dict[str, list[int]], tail: int = 32, tag: str = "t") -> None:
    """Most of a request in one step, its last `tail` tokens one by one."""
    for name, tokens in requests.items():
        rid = f"{tag}-{name}"
        head = max(1, len(tokens) - tail)
        trace.add([(rid, tokens[:head], [head - 1])])
        for i in range(head, len(tokens)):
            trace.add([(rid, tokens[i:i + 1], [0])], end=[rid] if i == len(tokens) - 1 else [])
        if head == len(tokens):
            trace.add([], end=[rid])


def portions(trace: Trace, requests: dict[str, list[int]], sizes=(7, 2, 24, 3, 33, 2, 17, 5), tag: str = "p") -> None:
    """Portions of changing size, down to two tokens; logits wanted everywhere."""
    for name, tokens in requests.items():
        rid = f"{tag}-{name}"
        at, k = 0, 0
        while at < len(tokens):
            n = min(sizes[k % len(sizes)], len(tokens) - at)
            k += 1
            last = at + n == len(tokens)
            trace.add([(rid, tokens[at:at + n], list(range(n)))], end=[rid] if last else [])
            at += n


def mixed(trace: Trace, requests: dict[str, list[int]], chunk: int = 24, live: int = 4, decode_tail: int = 12,
          tag: str = "m") -> None:
    """Up to `live` requests at a time: portions of some beside single tokens of others.

    A request is fed in portions of `chunk` until `decode_tail` tokens are left,
    then one token a step.  New requests start as soon as a seat is free, so the
    pages of finished requests are handed to the newcomers.
    """
    waiting = [(f"{tag}-{name}", tokens) for name, tokens in requests.items()]
    running: list[list] = []   # [rid, tokens, at]
    while waiting or running:
        while waiting and len(running) < live:
            rid, tokens = waiting.pop(0)
            running.append([rid, tokens, 0])
        entries, ended = [], []
        for slot in running:
            rid, tokens, at = slot
            prompt_end = max(1, len(tokens) - decode_tail)
            n = min(chunk, prompt_end - at) if at < prompt_end else 1
            # Stagger the requests so that portions meet single tokens of the others.
            if at == 0 and len(entries) % 2 == 1 and n > 2:
                n = max(2, n // 3)
            want = [n - 1] if at + n >= prompt_end else ([0] if n > 3 else [])
            entries.append((rid, tokens[at:at + n], want))
            slot[2] = at + n
            if slot[2] == len(tokens):
                ended.append(rid)
        trace.add(entries, end=ended)
        running = [s for s in running if s[2] < len(s[1])]


def expected_logits(model_dir: Path, requests: dict[str, list[int]], dtype=torch.float32, device="cpu"):
    """{request name: logits [len, vocab] float32} from the plain implementation."""
    config, weights = plain_llama.read_model(model_dir)
    return {name: plain_llama.forward(config, weights, tokens, dtype, device).float().cpu()
            for name, tokens in requests.items()}


def gather_expected(trace: Trace, expected: dict[str, torch.Tensor]) -> list[torch.Tensor | None]:
    """Per step, the rows the step must produce (request ids are '<tag>-<name>')."""
    out = []
    for wanted in trace.wanted:
        if not wanted:
            out.append(None)
            continue
        out.append(torch.stack([expected[rid.split("-", 1)[1]][pos] for rid, pos in wanted]))
    return out


def run_in_process(runner, trace: Trace) -> list[torch.Tensor | None]:
    from liteinfer_b200.engine.runner import StepEntry

    results = []
    for step in trace.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]]
        logits = runner.step(entries) if entries else None
        results.append(logits.float().cpu() if logits is not None and logits.shape[0] else None)
        for rid in step["end"]:
            runner.release(rid)
        runner.cache.check_invariants()
    return results


def run_program(trace: Trace, model_dir: Path, dtype: str, out_dir: Path, vocab: int, page_size: int | None = None,
                timeout: int = 600) -> list[torch.Tensor | None]:
    """Runs bin/trace_run as a child process, feeding one step at a time and waiting for `done`."""
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(trace.max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
    try:
        for step in trace.steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {step['step']}", f"trace_run said {line!r} at step {step['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    results = []
    for step, wanted in zip(trace.steps, trace.wanted):
        path = out_dir / f"{step['step']}.f32"
        if not wanted:
            assert not path.exists()
            results.append(None)
            continue
        data = np.fromfile(path, dtype="<f4")
        assert data.size == len(wanted) * vocab, f"step {step['step']}: {data.size} floats for {len(wanted)} rows"
        results.append(torch.from_numpy(data.reshape(len(wanted), vocab).copy()))
    return results


def worst_error(results, expected) -> tuple[float, int]:
    """(largest absolute difference, step where it occurs)."""
    worst, where = 0.0, -1
    for i, (got, want) in enumerate(zip(results, expected)):
        if want is None:
            assert got is None
            continue
        assert got is not None and got.shape == want.shape, f"step {i}: shape {None if got is None else got.shape}"
        assert torch.isfinite(got).all(), f"step {i}: non-finite logits"
        err = float((got - want).abs().max())
        if err > worst:
            worst, where = err, i
    return worst, where
