"""Slot addressing: block tables turned into the flat token slots of a pool.

The CUDA kernels read block tables directly (one int32 per page).  Host code that
wants a token's place as one number, and the plain-PyTorch stand-ins of the
tests, use these three helpers, which keep the names and meanings of
liteinfer/cache/block_pool.py:131-223:

    slot = page * page_size + position % page_size

is the index of a token in a pool seen as pages * page_size token slots per KV
head (the pool here is [pages, kv_heads, page_size, head_dim], so the token lies
at `pool[slot // page_size, :, slot % page_size]`).  Everything is computed on the host from the Python block tables
and lengths: nothing waits on the device, and one transfer moves the result.
A page that was given back (-1 in a block table) yields slot -1.
"""

from __future__ import annotations

from typing import NamedTuple, Sequence

import numpy as np
import torch

__all__ = ["PackedAddresses", "newest_slots", "packed_addresses", "slot_table"]


def _slots(table: Sequence[int], positions: np.ndarray, page_size: int) -> np.ndarray:
    pages = np.asarray(table, dtype=np.int64)[positions // page_size]
    return np.where(pages >= 0, pages * page_size + positions % page_size, -1)


def slot_table(block_tables: Sequence[Sequence[int]], totals: Sequence[int], page_size: int,
               device: torch.device | str = "cpu") -> torch.Tensor:
    """[B, max(totals)] int64, left-aligned: column p of row i is the slot of position p of sequence i;
    columns at and past a sequence's total hold -1 and are never to be read."""
    out = np.full((len(block_tables), max(totals, default=0)), -1, dtype=np.int64)
    for i, (table, total) in enumerate(zip(block_tables, totals, strict=True)):
        out[i, :total] = _slots(table, np.arange(total), page_size)
    return torch.from_numpy(out).to(device)


def newest_slots(block_tables: Sequence[Sequence[int]], positions: Sequence[int], page_size: int,
                 device: torch.device | str = "cpu") -> torch.Tensor:
    """[1, B] int64: the slot of one position per sequence, where a decode step writes."""
    slots = [int(_slots(table, np.asarray([position]), page_size)[0])
             for table, position in zip(block_tables, positions, strict=True)]
    return torch.tensor([slots], dtype=torch.int64, device=device)


class PackedAddresses(NamedTuple):
    slots: torch.Tensor            # [1, total] slot of every token of the step: where the pass writes
    positions: torch.Tensor        # [1, total] logical position of every token: what the rotary encoding reads
    query_start_loc: torch.Tensor  # [B + 1] int32 prefix sums of the counts
    slot_table: torch.Tensor       # [B, max context] slots of each sequence's whole context: what attention reads
    context_lens: torch.Tensor     # [B] int32 tokens each sequence holds once the step is written


def packed_addresses(block_tables: Sequence[Sequence[int]], starts: Sequence[int], counts: Sequence[int],
                     page_size: int, device: torch.device | str = "cpu") -> PackedAddresses:
    """Every address of a step in which sequence i brings its positions [starts[i], starts[i] + counts[i])."""
    totals = [s + c for s, c in zip(starts, counts, strict=True)]
    positions = np.concatenate([np.arange(s, t) for s, t in zip(starts, totals)]) if totals else np.zeros(0, np.int64)
    slots = np.concatenate([_slots(table, np.arange(s, t), page_size)
                            for table, s, t in zip(block_tables, starts, totals, strict=True)]) if totals else positions
    starts_of = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return PackedAddresses(
        slots=torch.from_numpy(slots.astype(np.int64)).unsqueeze(0).to(device),
        positions=torch.from_numpy(positions.astype(np.int64)).unsqueeze(0).to(device),
        query_start_loc=torch.from_numpy(starts_of).to(device),
        slot_table=slot_table(block_tables, totals, page_size, device),
        context_lens=torch.tensor(totals, dtype=torch.int32, device=device))
