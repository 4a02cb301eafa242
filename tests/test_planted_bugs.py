"""The replay tests must fail when the engine is wrong: each classic fault of a paged, batched step function is
planted in turn, the mixed trace of tests/replay_harness.py is run on the CPU stand-ins, and the worst difference
from the plain implementation must exceed the tolerance that the clean run stays under.

The reference's own builders planted these faults by hand (docs/milestones.md:29: a context one short, a shifted
query_start_loc, a rotary position off by one) and poison what must not be read
(tests/unit/test_paged_decode.py:133-149); here the planting is the test.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import replay_harness as rh
import tiny_configs

TOLERANCE = 2e-5        # what test_replay_cpu.py and test_replay_gpu.py ask of a float32 run


def _run(model_dirs, name="tiny_b", lengths=(9, 40, 64, 100)):
    from liteinfer_b200.engine.loading import build_runner

    config, _, page = tiny_configs.ALL[name]
    requests = {f"r{i}": tiny_configs.prompt(config["vocab_size"], n, i) for i, n in enumerate(lengths)}
    expected = rh.expected_logits(model_dirs[name], requests)
    trace = rh.Trace()
    rh.mixed(trace, requests)
    runner = build_runner(model_dirs[name], torch.float32, "cpu", page, -(-trace.max_tokens // page), 4)
    results = []
    from liteinfer_b200.engine.runner import StepEntry
    for step in trace.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]]
        logits = runner.step(entries)
        results.append(logits.float() if logits.shape[0] else None)
        for rid in step["end"]:
            runner.release(rid)
    worst = 0.0
    for got, want in zip(results, rh.gather_expected(trace, expected)):
        if want is not None:
            # A fault may also produce NaN (a page that was never written): that counts as a difference.
            diff = (got - want).abs()
            worst = max(worst, float(torch.nan_to_num(diff, nan=1e9).max()))
    return worst


def _plant_in_batch(monkeypatch, change):
    """Lets `change(batch, arrays, entries)` damage the batch that the step function has just laid out."""
    from liteinfer_b200.engine import runner as runner_module

    original = runner_module._fill

    def damaged(batch, flat, entries, cache, starts):
        original(batch, flat, entries, cache, starts)
        views = batch.views(flat)
        arrays = {name: getattr(views, name) for name in ("tok", "pos", "seq", "qsl", "ctxl", "slots", "rows", "dseq", "dtok", "pseq")}
        arrays["tables"] = [t.reshape(batch.B, w) for t, w in zip(views.tables, batch.widths) if w]
        change(batch, arrays, entries)

    monkeypatch.setattr(runner_module, "_fill", damaged)


def test_the_clean_run_is_within_tolerance(cpu_kernels, model_dirs):
    assert _run(model_dirs) < TOLERANCE


def test_context_one_short(cpu_kernels, model_dirs, monkeypatch):
    def change(batch, a, entries):
        a["ctxl"][:] = np.maximum(a["ctxl"] - 1, 1)
    _plant_in_batch(monkeypatch, change)
    assert _run(model_dirs) > 100 * TOLERANCE


def test_query_start_loc_shifted(cpu_kernels, model_dirs, monkeypatch):
    def change(batch, a, entries):
        if batch.B > 1:
            a["qsl"][1:batch.B] += 1        # every inner boundary one token late
    _plant_in_batch(monkeypatch, change)
    assert _run(model_dirs) > 100 * TOLERANCE


def test_rotary_position_off_by_one(cpu_kernels, model_dirs, monkeypatch):
    """The queries rotated as if they stood one position further on (keys and the cache as they should be).  A
    shift of queries and keys alike would cancel out in the scores, since the rotation is relative."""
    import torch_kernels

    import liteinfer_b200.ops as ops

    original = torch_kernels.rope_kv_write

    def shifted(qkv, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, heads, kv_heads, head_dim,
                rotary_dim, store=True):
        wrong = qkv.clone()
        original(wrong, positions + 1, seq_of_token, block_table, k_pool, v_pool, inv_freq, heads, kv_heads,
                 head_dim, rotary_dim, store=False)
        original(qkv, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, heads, kv_heads, head_dim,
                 rotary_dim, store=store)
        qkv[:, :heads * head_dim] = wrong[:, :heads * head_dim]

    monkeypatch.setattr(ops, "rope_kv_write", shifted)
    assert _run(model_dirs) > 100 * TOLERANCE


def test_block_table_entry_swapped_between_two_requests(cpu_kernels, model_dirs, monkeypatch):
    def change(batch, a, entries):
        for table in a["tables"]:
            if batch.B > 1 and table[0, 0] >= 0 and table[1, 0] >= 0:
                table[0, 0], table[1, 0] = int(table[1, 0]), int(table[0, 0])
    _plant_in_batch(monkeypatch, change)
    assert _run(model_dirs) > 100 * TOLERANCE


def test_block_table_row_kept_from_an_earlier_step(cpu_kernels, model_dirs, monkeypatch):
    """A copy of a request's block table that is not refreshed when the request takes more pages (what the
    graphs' staged batches guard against with the cache manager's table versions)."""
    kept: dict[str, list[np.ndarray]] = {}

    def change(batch, a, entries):
        for i, entry in enumerate(entries):
            rows = kept.setdefault(entry.request_id, [table[i].copy() for table in a["tables"]])
            for table, row in zip(a["tables"], rows):
                n = min(len(row), table.shape[1])
                table[i, :] = -1
                table[i, :n] = row[:n]
    _plant_in_batch(monkeypatch, change)
    assert _run(model_dirs) > 100 * TOLERANCE


def test_a_page_given_back_too_early(cpu_kernels, model_dirs, monkeypatch):
    """The allocator hands a live request's first page to the next newcomer as well (and, its bookkeeping being
    what is broken, does not notice when the page comes back twice): two requests then write the same slots."""
    from liteinfer_b200.cache.pages import PageAllocator

    original, original_free = PageAllocator.allocate, PageAllocator.free
    state = {"stolen": None}

    def allocate(self, count):
        pages = original(self, count)
        if type(self) is PageAllocator and state["stolen"] is None and self.num_held > count and count:
            held = [p for p in range(self.num_pages) if self.is_held(p) and p not in pages]
            state["stolen"] = held[0]
            self.free([pages[0]])
            pages[0] = held[0]
        return pages

    def free(self, pages):
        original_free(self, [p for p in pages if self.is_held(p)])

    monkeypatch.setattr(PageAllocator, "allocate", allocate)
    monkeypatch.setattr(PageAllocator, "free", free)
    assert _run(model_dirs) > 100 * TOLERANCE


def test_logit_rows_off_by_one(cpu_kernels, model_dirs, monkeypatch):
    def change(batch, a, entries):
        a["rows"][:] = np.maximum(a["rows"] - 1, 0)
    _plant_in_batch(monkeypatch, change)
    assert _run(model_dirs) > 100 * TOLERANCE
