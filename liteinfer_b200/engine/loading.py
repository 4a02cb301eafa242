"""From a model folder to a `ModelRunner`.

`make_runner` puts a loaded model together with a cache manager of a given size and a step function; the engine
core calls it once it has worked out how many pages memory affords, and `build_runner` (the trace-replay program,
tests and tools, which name the number of pages themselves) loads the model first.
"""

from __future__ import annotations

from pathlib import Path

import torch

from liteinfer_b200.cache.manager import CacheManager
from liteinfer_b200.engine.runner import ModelRunner
from liteinfer_b200.weights.loader import load_model


def resolve_model_path(model: str | Path) -> Path:
    """A local folder only (liteinfer/hub.py:26-28 returns a local directory as it is;
    its download branch needs a network and is not built)."""
    path = Path(model)
    if not path.is_dir():
        raise FileNotFoundError(f"model folder {model!r} does not exist (models are read from local folders only)")
    return path


def make_runner(model, dtype: torch.dtype, device: torch.device | str, page_size: int, num_pages: int,
                max_requests: int, decode_splits: int | None = None) -> ModelRunner:
    cache = CacheManager(model.cache_needs(), model.schedule, page_size, num_pages, max_requests, dtype,
                         torch.device(device))
    return ModelRunner(model, cache, decode_splits)


def build_runner(model_dir: str | Path, dtype: torch.dtype, device: torch.device | str, page_size: int,
                 num_pages: int, max_requests: int, decode_splits: int | None = None) -> ModelRunner:
    device = torch.device(device)
    model, _ = load_model(resolve_model_path(model_dir), dtype, device)
    return make_runner(model, dtype, device, page_size, num_pages, max_requests, decode_splits)
