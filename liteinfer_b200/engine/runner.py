"""The step function: one batch of (request, its next tokens) through the model, from the cache.

`ModelRunner.step` takes any mix of entries — a whole prompt, a portion of
one cut anywhere, a single decoded token — runs exactly the tokens it is given
as one batch, and returns logits only at the places asked for.  What the
requests computed earlier is read from the cache; what this step computes is
written there.  The cache changes only if the step succeeds.

The reference's `ModelRunner.execute` (liteinfer/engine/model_runner.py:137-172)
has the same contract on `Sequence` objects and returns one row per sequence;
here the batch is plain token ids so that the scheduler's engine and the
trace-replay program drive the very same function, and rows are computed only
where `want` asks.

A step that holds only single decoded tokens, each wanting its logits, can be
replayed from a CUDA graph (one graph per batch width, captured on first use,
as liteinfer/engine/cuda_graphs.py:105-260 does): the batch is then written
into buffers of fixed size and place, and the kernels read their bounds from
those buffers.  Every other step of moderate size (portions of prompts, alone
or beside decoded tokens) is replayed from a graph too, one per padded shape:
the step's tokens, sequences and wanted rows are rounded up to the next size of
a ladder, the places of padding belong to no sequence (kernels skip them), and
only the real rows are returned.  A step launched kernel by kernel costs the
host a few milliseconds, more than the device needs for a short prompt.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from liteinfer_b200.cache.manager import CacheManager
from liteinfer_b200.ops import kernels
from liteinfer_b200.parts.context import AttentionPlan, StepContext
from liteinfer_b200.parts.model import Model

_MAX_GRAPHS = 128   # liteinfer/engine/cuda_graphs.py:68


def ops_scatter(tokens, dst, src, source):
    from liteinfer_b200 import ops      # through the module, so that a stand-in kernel is found
    return ops.scatter_tokens(tokens, dst, src, source)


def ops_stage(device, host, tokens, dst, src, source) -> bool:
    from liteinfer_b200 import ops
    return ops.stage_batch(device, host, tokens, dst, src, source)


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them whose logits are wanted.

    `late` (an entry of one token only): the token's value is not on the host yet; it is element `late` of the
    tensor of sampled tokens that `ModelRunner.step` is given as `late_source`, and is copied from there on the
    device.  `tokens` then holds a stand-in that is never looked at."""

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)
    late: int | None = None


class _Views:
    """The arrays of one staged batch (slices of one buffer, numpy or torch)."""

    __slots__ = ("tok", "pos", "seq", "qsl", "ctxl", "slots", "rows", "dseq", "dtok", "pseq", "late_dst", "late_src",
                 "tables")
    NAMES = __slots__[:-1]

    def __iter__(self):      # tok, pos, seq, qsl, ctxl, slots, rows, dseq, dtok, pseq, late_dst, late_src, *tables
        for name in self.NAMES:
            yield getattr(self, name)
        yield from self.tables


class _Batch:
    """Where each array of a step lies in the one int32 staging buffer."""

    def __init__(self, B: int, T: int, R: int, widths: list[int], n_decode: int, n_prefill: int) -> None:
        self.B, self.T, self.R, self.widths = B, T, R, widths
        self.n_decode, self.n_prefill = n_decode, n_prefill
        sizes = [T, T, T, B + 1, B, B, R, n_decode, n_decode, n_prefill, B, B] + [B * w for w in widths]
        # Every array starts on a 16-byte boundary.
        self.sizes = sizes
        self.offsets = []
        at = 0
        for n in sizes:
            self.offsets.append(at)
            at += -(-n // 4) * 4
        self.total = max(at, 4)

    def views(self, flat) -> _Views:
        """The arrays as slices of `flat` (a numpy array or a tensor)."""
        slices = [flat[o:o + n] for o, n in zip(self.offsets, self.sizes)]
        v = _Views()
        for name, array in zip(_Views.NAMES, slices):
            setattr(v, name, array)
        v.tables = slices[len(_Views.NAMES):]
        return v


def _fill(batch: _Batch, flat: np.ndarray, entries: list[StepEntry], cache: CacheManager,
          starts: list[int]) -> None:
    tok, pos, seq, qsl, ctxl, slots, rows, dseq, dtok, pseq, late_dst, late_src, *tables = batch.views(flat)
    cursor = row_cursor = nd = npf = late = 0
    qsl[0] = 0
    late_dst[:] = -1
    for i, entry in enumerate(entries):
        n = len(entry.tokens)
        if entry.late is None:
            tok[cursor:cursor + n] = entry.tokens
        else:
            tok[cursor] = 0
            late_dst[late], late_src[late] = cursor, entry.late
            late += 1
        pos[cursor:cursor + n] = np.arange(starts[i], starts[i] + n, dtype=np.int32)
        seq[cursor:cursor + n] = i
        for place in entry.want:
            rows[row_cursor] = cursor + place
            row_cursor += 1
        if n == 1:
            dseq[nd], dtok[nd] = i, cursor
            nd += 1
        else:
            pseq[npf] = i
            npf += 1
        cursor += n
        qsl[i + 1] = cursor
        ctxl[i] = starts[i] + n
        slots[i] = cache.state_slot(entry.request_id)
    for g, width in enumerate(batch.widths):
        if not width:
            continue
        table = tables[g].reshape(batch.B, width)
        table.fill(-1)
        for i, entry in enumerate(entries):
            blocks = cache.block_table(g, entry.request_id)
            table[i, :len(blocks)] = blocks


def _context(batch: _Batch, dev: torch.Tensor, device, counts, totals, decode_splits, decode_bound) -> StepContext:
    tok, pos, seq, qsl, ctxl, slots, rows, dseq, dtok, pseq, _, _, *tables = batch.views(dev)
    B = batch.B
    tables = [t.view(B, w) if w else torch.full((B, 1), -1, dtype=torch.int32, device=device)
              for t, w in zip(tables, batch.widths)]
    prefill_lens = [c for c in counts if c > 1]
    plan = AttentionPlan(
        num_decode=batch.n_decode, decode_seqs=dseq, decode_tokens=dtok, num_prefill=batch.n_prefill,
        prefill_seqs=pseq, max_prefill_query_len=max(prefill_lens, default=0), max_decode_context_len=decode_bound)
    return StepContext(
        num_tokens=batch.T, num_seqs=B, token_ids=tok, positions=pos, seq_of_token=seq, query_start_loc=qsl,
        context_lens=ctxl, block_tables=tables, state_slots=slots, logit_rows=rows, num_logit_rows=batch.R,
        max_query_len=max(counts), max_context_len=max(totals), query_lens=tuple(counts),
        host_context_lens=tuple(totals), decode_splits=decode_splits, plan=plan)


class _DecodeGraph:
    """One captured decode forward for exactly `width` sequences."""

    def __init__(self, runner: ModelRunner, width: int, max_model_len: int) -> None:
        cache = runner.cache
        pages = -(-max_model_len // cache.page_size)
        self.batch = _Batch(width, width, width, [pages] * len(cache.groups), width, 0)
        self.device_buffer = torch.zeros(self.batch.total, dtype=torch.int32, device=runner.device)
        counts, totals = [1] * width, [max_model_len] * width
        self.ctx = _context(self.batch, self.device_buffer, runner.device, counts, totals, runner.decode_splits,
                            max_model_len)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.launches = 0
        # The batch is staged in one pinned buffer that keeps its contents from step to step: the rows of a
        # request (its block tables, its state slot) are rewritten only when the cache manager says they changed,
        # what is the same for every batch of this width is written once, and a step writes tokens and lengths.
        self.host = torch.zeros(self.batch.total, dtype=torch.int32, pin_memory=True)
        self.views = self.batch.views(self.host.numpy())
        self.copied = torch.cuda.Event()       # recorded behind the copy of `host` to the device
        self.row_keys: list[tuple[str, int] | None] = [None] * width
        self._write_fixed_parts()

    def _write_fixed_parts(self) -> None:
        """What is the same for every batch of this width: sequence i brings token i and wants its logits."""
        tok, pos, seq, qsl, ctxl, slots, rows, dseq, dtok, pseq, late_dst, late_src, *tables = self.views
        width = self.batch.B
        late_dst[:] = -1
        seq[:] = np.arange(width, dtype=np.int32)
        qsl[:] = np.arange(width + 1, dtype=np.int32)
        rows[:] = seq
        dseq[:] = seq
        dtok[:] = seq
        for table in tables:
            table.fill(-1)
        self.row_keys = [None] * width

    def stage_padding(self) -> None:
        """A batch that is all padding: no token belongs to a sequence, no sequence brings a token or holds a
        context, the attention launches find no work.  Kernels run on it and touch neither pages nor state."""
        _write_padding(self.views)

    def after_capture(self) -> None:
        self._write_fixed_parts()

    def stage(self, entries: list[StepEntry], cache: CacheManager, starts: list[int]) -> None:
        """Writes this step's batch (every entry one token, logits wanted) into the pinned buffer."""
        self.copied.synchronize()              # the device has read the batch before this one
        tok, pos, seq, qsl, ctxl, slots, rows, dseq, dtok, pseq, late_dst, late_src, *tables = self.views
        tok[:] = [entry.tokens[0] if entry.late is None else 0 for entry in entries]
        late_dst[:] = [-1 if entry.late is None else i for i, entry in enumerate(entries)]     # token row i is sequence i
        late_src[:] = [entry.late or 0 for entry in entries]
        pos[:] = starts
        np.add(pos, 1, out=ctxl)
        for i, entry in enumerate(entries):
            key = (entry.request_id, cache.table_version(entry.request_id))
            if self.row_keys[i] == key:
                continue
            self.row_keys[i] = key
            slots[i] = cache.state_slot(entry.request_id)
            for g, width in enumerate(self.batch.widths):
                blocks = cache.block_table(g, entry.request_id)
                row = tables[g][i * width:(i + 1) * width]
                row[:len(blocks)] = blocks
                row[len(blocks):] = -1

    def capture(self, runner: ModelRunner) -> None:
        """One eager pass on a side stream, then the capture, both on a batch that is all padding: a live batch
        would be run twice more than it should (harmless for keys and values, which are written to the same
        places each time, but a part that updates a request's state in place would apply its step three times).
        The graph is kept only if the capture succeeded."""
        self.copied.synchronize()
        self.stage_padding()
        self.device_buffer.copy_(self.host, non_blocking=True)
        stream = torch.cuda.Stream(device=runner.device)
        stream.wait_stream(torch.cuda.current_stream(runner.device))
        with torch.cuda.stream(stream), kernels.on_current_stream():
            runner.model.forward(self.ctx, runner.layer_caches)
        torch.cuda.current_stream(runner.device).wait_stream(stream)
        torch.cuda.synchronize(runner.device)
        before = kernels.launch_count
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, pool=runner.graph_pool), kernels.on_current_stream():
            logits = runner.model.forward(self.ctx, runner.layer_caches)
        self.launches = kernels.launch_count - before
        self.graph, self.logits = graph, logits
        self.after_capture()


def _write_padding(views) -> None:
    tok, pos, seq, qsl, ctxl, slots, rows, dseq, dtok, pseq, late_dst, late_src, *tables = views
    for array in (tok, pos, qsl, ctxl, slots, rows, dtok, late_src):
        array[:] = 0
    for array in (seq, dseq, pseq, late_dst, *tables):
        array[:] = -1


def _pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def _token_bucket(n: int) -> int:
    """The padded number of tokens of a step: steps of 16 up to 128, then of an eighth of the next power of two."""
    step = 16 if n <= 128 else _pow2(n) // 8
    return -(-n // step) * step


class _PaddedGraph:
    """One captured forward for any step that fits a padded shape: up to `tokens` tokens in up to `seqs` sequences,
    of which up to `prefill` bring more than one token, with up to `rows` wanted rows."""

    def __init__(self, runner: ModelRunner, tokens: int, seqs: int, decode: bool, prefill: int, rows: int,
                 max_model_len: int) -> None:
        cache = runner.cache
        pages = -(-max_model_len // cache.page_size)
        n_decode = seqs if decode else 0
        self.batch = batch = _Batch(seqs, tokens, rows, [pages] * len(cache.groups), n_decode, prefill)
        self.device_buffer = torch.zeros(batch.total, dtype=torch.int32, device=runner.device)
        tok, pos, seq, qsl, ctxl, slots, wanted, dseq, dtok, pseq, _, _, *tables = batch.views(self.device_buffer)
        tables = [t.view(seqs, w) for t, w in zip(tables, batch.widths)]
        # The kernels' launch bounds are those of the padded shape; what a step really holds is in the buffers.
        plan = AttentionPlan(num_decode=n_decode, decode_seqs=dseq, decode_tokens=dtok, num_prefill=prefill,
                             prefill_seqs=pseq, max_prefill_query_len=tokens if prefill else 0,
                             max_decode_context_len=max_model_len)
        self.ctx = StepContext(
            num_tokens=tokens, num_seqs=seqs, token_ids=tok, positions=pos, seq_of_token=seq, query_start_loc=qsl,
            context_lens=ctxl, block_tables=tables, state_slots=slots, logit_rows=wanted, num_logit_rows=rows,
            max_query_len=tokens if prefill else 1, max_context_len=max_model_len,
            decode_splits=runner.decode_splits, plan=plan)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.launches = 0
        self.host = torch.zeros(batch.total, dtype=torch.int32, pin_memory=True)
        self.views = batch.views(self.host.numpy())
        self.copied = torch.cuda.Event()

    def stage(self, entries: list[StepEntry], cache: CacheManager, starts: list[int]) -> int:
        """Writes this step's batch and the padding around it into the pinned buffer; returns the wanted rows."""
        self.copied.synchronize()
        _fill(self.batch, self.host.numpy(), entries, cache, starts)
        tok, pos, seq, qsl, ctxl, slots, wanted, dseq, dtok, pseq, *_ = self.views
        B = len(entries)
        T = int(qsl[B])
        R = sum(len(e.want) for e in entries)
        n_decode = sum(1 for e in entries if len(e.tokens) == 1)
        tok[T:] = 0
        pos[T:] = 0
        seq[T:] = -1            # a token of padding belongs to no sequence: nothing is stored for it
        qsl[B + 1:] = T         # a sequence of padding brings no token
        ctxl[B:] = 0
        slots[B:] = 0
        wanted[R:] = 0
        dseq[n_decode:] = -1    # the attention launches skip these places
        dtok[n_decode:] = 0
        pseq[B - n_decode:] = -1
        return R

    def stage_padding(self) -> None:
        _write_padding(self.views)

    def after_capture(self) -> None:
        pass        # `stage` writes the whole batch every step

    capture = _DecodeGraph.capture


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, decode_splits: int | None = None) -> None:
        self.model, self.cache = model, cache
        self.device = model.device
        self.decode_splits = decode_splits
        self.layer_caches = cache.layer_caches()
        self._pinned = self.device.type == "cuda"
        self.num_steps = 0
        self._graphs: dict[int, _DecodeGraph] = {}
        self._padded_graphs: dict[tuple, _PaddedGraph] = {}
        self._graph_limits: tuple[int, int] | None = None
        self._padded_limit = 0      # most tokens of a step that is replayed from a padded graph
        self.graph_pool = None
        self.graph_launches = 0     # launches of this package's kernels replayed from graphs
        self.graph_replays = 0

    # ---------------------------------------------------------------- batch
    def _validate(self, entries: list[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen: set[str] = set()
        vocab = self.model.spec.vocab_size
        for entry in entries:
            if entry.request_id in seen:
                raise ValueError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            n = len(entry.tokens)
            if n < 1:
                raise ValueError(f"request {entry.request_id!r} brings no tokens")
            if entry.late is not None:
                if n != 1 or entry.late < 0:
                    raise ValueError(f"request {entry.request_id!r}: a token read on the device is one token")
            elif min(entry.tokens) < 0 or max(entry.tokens) >= vocab:
                raise ValueError(f"request {entry.request_id!r} has a token id outside [0, {vocab})")
            for place in entry.want:
                if not 0 <= place < n:
                    raise ValueError(f"request {entry.request_id!r} wants logits at {place}, but brings {n} tokens")

    def _stage(self, batch: _Batch, dev: torch.Tensor, host: torch.Tensor, entries: list[StepEntry], late_source) -> None:
        """The staged batch from its pinned buffer to the device and the late tokens into it: one kernel that reads
        the pinned buffer in place where the batch is small, else a copy and the scatter."""
        late = any(e.late is not None for e in entries)
        if late and late_source is None:
            raise ValueError("an entry's token is to be read on the device, but no tensor of sampled tokens was given")
        if dev.is_cuda:
            v = batch.views(dev)
            if ops_stage(dev, host, v.tok, v.late_dst, v.late_src, late_source if late else None):
                return
        dev.copy_(host, non_blocking=True)
        self._place_late_tokens(batch, dev, entries, late_source)

    @staticmethod
    def _place_late_tokens(batch: _Batch, dev: torch.Tensor, entries: list[StepEntry], late_source) -> None:
        """Tokens that were sampled on the device and never read: from `late_source` into the batch, on the device."""
        if not any(e.late is not None for e in entries):
            return
        if late_source is None:
            raise ValueError("an entry's token is to be read on the device, but no tensor of sampled tokens was given")
        v = batch.views(dev)
        ops_scatter(v.tok, v.late_dst, v.late_src, late_source)

    def build_context(self, entries: list[StepEntry], late_source: torch.Tensor | None = None) -> StepContext:
        """The batch as device tensors (one staging buffer, one host-to-device copy)."""
        cache = self.cache
        starts = [cache.length(e.request_id) for e in entries]
        counts = [len(e.tokens) for e in entries]
        totals = [s + c for s, c in zip(starts, counts)]
        widths = [max(len(cache.block_table(g, e.request_id)) for e in entries) for g in range(len(cache.groups))]
        n_decode = sum(1 for c in counts if c == 1)
        batch = _Batch(len(entries), sum(counts), sum(len(e.want) for e in entries), widths, n_decode,
                       len(entries) - n_decode)
        host = torch.empty(batch.total, dtype=torch.int32, pin_memory=self._pinned)
        _fill(batch, host.numpy(), entries, cache, starts)
        dev = host.to(self.device, non_blocking=True)
        self._place_late_tokens(batch, dev, entries, late_source)
        decode_bound = max((t for t, c in zip(totals, counts) if c == 1), default=0)
        return _context(batch, dev, self.device, counts, totals, self.decode_splits, decode_bound)

    # --------------------------------------------------------------- graphs
    def enable_decode_graphs(self, max_num_seqs: int, max_model_len: int, max_padded_tokens: int = 2048) -> None:
        """Replay steps from CUDA graphs: steps of single decoded tokens from a graph of their exact width, other
        steps of at most `max_padded_tokens` tokens from a graph of their padded shape (0: those run kernel by
        kernel; larger steps always do, their time on the device dwarfs the host's)."""
        if self.device.type != "cuda":
            raise ValueError("CUDA graphs need a CUDA device")
        if not self.model.graph_safe:
            return          # a part works on the host inside forward: every step launches kernel by kernel
        self._graph_limits = (max_num_seqs, max_model_len)
        self._padded_limit = max_padded_tokens
        self.graph_pool = torch.cuda.graph_pool_handle()

    def _graph_for(self, entries: list[StepEntry], totals: list[int]) -> _DecodeGraph | None:
        if self._graph_limits is None:
            return None
        max_seqs, max_len = self._graph_limits
        width = len(entries)
        if width > max_seqs or max(totals) > max_len:
            return None
        if any(len(e.tokens) != 1 or tuple(e.want) != (0,) for e in entries):
            return None
        graph = self._graphs.get(width)
        if graph is None:
            if len(self._graphs) >= _MAX_GRAPHS:
                return None
            graph = self._graphs[width] = _DecodeGraph(self, width, max_len)
        return graph

    def _padded_graph_for(self, entries: list[StepEntry], totals: list[int]) -> _PaddedGraph | None:
        if self._graph_limits is None or not self._padded_limit:
            return None
        max_seqs, max_len = self._graph_limits
        tokens = sum(len(e.tokens) for e in entries)
        if len(entries) > max_seqs or max(totals) > max_len or tokens > self._padded_limit:
            return None
        seqs = min(_pow2(len(entries)), max(max_seqs, 1))
        n_decode = sum(1 for e in entries if len(e.tokens) == 1)
        prefill = min(_pow2(len(entries) - n_decode), seqs) if n_decode < len(entries) else 0
        wanted = sum(len(e.want) for e in entries)
        rows = seqs if wanted <= seqs else _token_bucket(wanted)
        key = (_token_bucket(tokens), seqs, n_decode > 0, prefill, rows)
        graph = self._padded_graphs.get(key)
        if graph is None:
            if len(self._padded_graphs) >= _MAX_GRAPHS:      # the decode graphs have a table of their own
                return None
            graph = self._padded_graphs[key] = _PaddedGraph(self, *key, max_len)
        return graph

    def _replay(self, graph: _DecodeGraph | _PaddedGraph, entries: list[StepEntry],
                late_source: torch.Tensor | None = None, borrow: bool = False) -> torch.Tensor:
        if graph.graph is None:
            try:
                graph.capture(self)
            except BaseException:
                # A graph whose capture failed (out of memory, say) must not be found again by the next step.
                self._graphs = {k: g for k, g in self._graphs.items() if g is not graph}
                self._padded_graphs = {k: g for k, g in self._padded_graphs.items() if g is not graph}
                raise
        starts = [self.cache.length(e.request_id) for e in entries]
        wanted = graph.stage(entries, self.cache, starts)
        self._stage(graph.batch, graph.device_buffer, graph.host, entries, late_source)
        graph.copied.record()
        graph.graph.replay()
        self.graph_launches += graph.launches
        self.graph_replays += 1
        logits = graph.logits if wanted is None else graph.logits[:wanted]
        return logits if borrow else logits.clone()

    # ----------------------------------------------------------------- step
    def step(self, entries: list[StepEntry], late_source: torch.Tensor | None = None,
             borrow: bool = False) -> torch.Tensor:
        """Logits [number of wanted places, vocab], in the order of `entries` and of each entry's `want`.
        `late_source` (int32, on the device): where the tokens of entries marked `late` are read from.
        `borrow`: the caller is done with the logits (on this stream) before it calls `step` again, so a step that a
        graph replays may return the graph's own buffer instead of a copy of it."""
        self._validate(entries)
        ids = [e.request_id for e in entries]
        totals = [self.cache.length(e.request_id) + len(e.tokens) for e in entries]
        self.cache.reserve(ids, totals)   # raises before anything changes
        try:
            graph = self._graph_for(entries, totals) or self._padded_graph_for(entries, totals)
            if graph is not None:
                logits = self._replay(graph, entries, late_source, borrow)
            else:
                context = self.build_context(entries, late_source)
                with kernels.on_current_stream():
                    logits = self.model.forward(context, self.layer_caches)
        except BaseException:
            self.cache.rollback(ids)
            raise
        for request_id, total in zip(ids, totals):
            self.cache.commit(request_id, total)
        self.num_steps += 1
        return logits

    def check_kernels(self) -> None:
        """Raises if a kernel has flagged a fault since the last check: a bounded wait inside a tcgen05 or TMA
        kernel that gave up, or a token id outside the embedding table (the results since the last check are then
        not to be trusted).  Reads two integers from the device, so callers do it where they synchronise anyway."""
        if self.device.type != "cuda":
            return
        from liteinfer_b200 import ops

        where, bad_token = ops.error_flags(self.device)
        if where:
            raise RuntimeError(f"a tcgen05 kernel stopped waiting on its pipeline (wait number {where}); "
                               "its output is unreliable")
        if bad_token:
            raise RuntimeError("a token id outside the vocabulary reached the embedding kernel")

    def release(self, request_id: str) -> None:
        """The request is finished: what it holds is given back."""
        self.cache.release(request_id)
