"""User-facing result types (liteinfer/outputs.py:8-33)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass
class RequestOutput:
    """A completed generation."""

    request_id: str
    prompt: str
    text: str
    token_ids: list[int]
    finish_reason: str  # "stop" | "length" | "abort"


@dataclass
class StreamEvent:
    """One streaming event; `text` and `output_token_ids` are cumulative, the last event is finished."""

    request_id: str
    prompt: str
    output_token_ids: list[int]
    text: str
    is_finished: bool
    finish_reason: str | None
