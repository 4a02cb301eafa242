"""Reads a model folder: config.json chooses the architecture, safetensors are bound by tensor name.

liteinfer/models/loader.py:42-86 streams every `*.safetensors` shard and copies
each tensor into the same-named parameter, converting to the engine's dtype;
missing names raise, a tied head may be absent (:79-82).  Here the parts say
which names and shapes they read (`Model.tensor_specs`), and every mismatch —
missing names, unexpected names, wrong shapes — is reported in one
`WeightsError`.
"""

from __future__ import annotations

from pathlib import Path

import torch
from safetensors import safe_open

from liteinfer_b200.config.registry import resolve_model_dir
from liteinfer_b200.parts.model import Model

# Buffers that old checkpoints store although they are recomputed from the configuration.
_IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightsError(RuntimeError):
    """The checkpoint does not hold the tensors the model reads."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape) -> None:
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights under {model_dir} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{name} is {list(got)}, expected {list(want)}" for name, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def _target_dtype(kind: str, engine_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if kind == "f32":
        return torch.float32
    return engine_dtype


def safetensor_shards(model_dir: Path) -> list[Path]:
    shards = sorted(Path(model_dir).glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"no *.safetensors files under {model_dir}")
    return shards


def load_model(model_dir: str | Path, dtype: torch.dtype, device: torch.device | str):
    """(Model with its tensors bound on `device`, typed configuration) for a model folder."""
    model_dir = Path(model_dir)
    device = torch.device(device)
    arch, config = resolve_model_dir(model_dir)
    spec = arch.build_spec(config)
    model = Model(spec, dtype, device)
    expected = model.tensor_specs()
    tied = dict(spec.tied)

    tensors: dict[str, torch.Tensor] = {}
    unexpected: list[str] = []
    wrong_shape: list[tuple[str, tuple, tuple]] = []
    for shard in safetensor_shards(model_dir):
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for name in f.keys():  # noqa: SIM118
                want = expected.get(name)
                if want is None or name in tied:
                    # A tied head stored beside the embedding is not read (loader.py:64-69 likewise).
                    if name not in tied and not name.endswith(_IGNORED_SUFFIXES):
                        unexpected.append(name)
                    continue
                got = tuple(f.get_slice(name).get_shape())
                if got != tuple(want.shape):
                    wrong_shape.append((name, got, tuple(want.shape)))
                    continue
                tensors[name] = f.get_tensor(name).to(device=device, dtype=_target_dtype(want.kind, dtype))

    for name, source in tied.items():
        if source in tensors:
            tensors[name] = tensors[source]
    missing = [name for name in expected if name not in tensors
               and not any(name == w[0] for w in wrong_shape)]
    if missing or unexpected or wrong_shape:
        raise WeightsError(model_dir, missing, sorted(unexpected), wrong_shape)
    model.bind(tensors)
    return model, config
