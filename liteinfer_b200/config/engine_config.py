"""Engine configuration: the knobs of liteinfer's `EngineConfig`, with its names and meanings.

Reference: liteinfer/config.py:13-103.  Fields that chose between attention
back ends are accepted for compatibility but only name this engine's one path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
}


def parse_dtype(dtype: str | torch.dtype) -> torch.dtype:
    """bfloat16 (the serving precision) or float32 (true 32-bit everywhere)."""
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {dtype} is not supported; use bfloat16 or float32")
        return dtype
    try:
        return _DTYPES[str(dtype).lower().replace("torch.", "")]
    except KeyError:
        raise ValueError(f"dtype {dtype!r} is not supported; use bfloat16 or float32") from None


@dataclass
class EngineConfig:
    model: str

    dtype: torch.dtype | str = torch.bfloat16
    device: str = "auto"

    max_num_seqs: int = 32
    max_model_len: int = 4096

    # Tokens one step may compute across all its sequences; a prompt larger than
    # what is left of it is cut into portions.  None: `max_num_seqs * max_model_len`,
    # which never cuts (liteinfer/config.py:23-28,92-97).
    max_num_batched_tokens: int | None = None

    # Seeds requests whose SamplingParams carry no seed of their own.
    seed: int = 42

    # Only this engine's paged kernels exist; None or "paged" name them.
    attn_implementation: str | None = None

    max_waiting_seqs: int = 1024

    # Replay decode steps from CUDA graphs.  None: wherever the device is CUDA.
    enable_cuda_graphs: bool | None = None

    # Programs that share one sequence's key loop in decode attention; None lets
    # the engine choose from the batch width and the context.
    paged_decode_splits: int | None = None

    collect_stats: bool = True

    # Launch a step before the tokens of the step before it have been read (they are copied into the batch on the
    # device), so that planning and the stop rules run beside the device's work.  None: on.  False: every step's
    # tokens are read before the next launch.
    async_scheduling: bool | None = None

    block_size: int = 16
    gpu_memory_utilization: float = 0.85
    num_gpu_blocks: int | None = None

    def __post_init__(self) -> None:
        self.dtype = parse_dtype(self.dtype)
        at_least_one = ("max_num_seqs", "max_model_len", "block_size", "max_waiting_seqs")
        optional_at_least_one = ("paged_decode_splits", "num_gpu_blocks")
        for name in at_least_one + optional_at_least_one:
            value = getattr(self, name)
            if value is None and name in optional_at_least_one:
                continue
            if value < 1:
                raise ValueError(f"{name}={value}: it counts something and must be at least 1")
        if self.max_num_batched_tokens is not None and self.max_num_batched_tokens < self.max_num_seqs:
            # A step must have room for one token of every seated request, or decoding requests would starve a prompt.
            raise ValueError(f"max_num_batched_tokens={self.max_num_batched_tokens} is below max_num_seqs="
                             f"{self.max_num_seqs}: a step could not decode every seated request")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError(f"gpu_memory_utilization={self.gpu_memory_utilization}: a share of the device's memory in (0, 1]")
        if self.attn_implementation not in (None, "paged"):
            raise ValueError(f"attn_implementation={self.attn_implementation!r}: this engine has one attention path, "
                             "'paged' (its own kernels over the paged cache)")

    @property
    def token_budget(self) -> int:
        """Tokens a step may compute: `max_num_batched_tokens`, or when that is None as many as the seats could
        ever bring (which cuts no prompt)."""
        if self.max_num_batched_tokens is None:
            return self.max_num_seqs * self.max_model_len
        return self.max_num_batched_tokens

    def resolved_device(self) -> torch.device:
        if self.device == "auto":
            return torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
        device = torch.device(self.device)
        if device.type == "cuda" and device.index is None:      # "cuda" and "cuda:0" compare and hash apart
            device = torch.device("cuda", torch.cuda.current_device() if torch.cuda.is_available() else 0)
        return device
