"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

Every tensor the architecture's parts read is drawn with a CPU generator seeded
once, in the fixed order of `Model.tensor_specs()`: "normal" tensors from
N(0, 0.02), "ones_normal" (norm weights) from 1 + N(0, 0.01), "zeros" as zeros,
a tensor whose spec brings its own init function from that function (given the
same generator), integer tables uniformly; each is drawn in float32 and then stored in `dtype`.
Names that alias another tensor (a tied head) are not written, as in a real
checkpoint.  The folder is what any other loader of this architecture reads.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any

import torch
from safetensors.torch import save_file

from liteinfer_b200.config.registry import resolve
from liteinfer_b200.parts.model import Model


def random_tensors(raw_config: dict[str, Any], seed: int, dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    arch, config = resolve(raw_config)
    spec = arch.build_spec(config)
    model = Model(spec, dtype, torch.device("cpu"))
    generator = torch.Generator(device="cpu").manual_seed(int(seed))
    tensors: dict[str, torch.Tensor] = {}
    for name, want in model.tensor_specs().items():
        if name in spec.tied:
            continue
        if want.kind == "int":
            tensors[name] = torch.randint(0, 2 ** 15, want.shape, generator=generator, dtype=torch.int32)
            continue
        if callable(want.init):
            value = torch.as_tensor(want.init(tuple(want.shape), generator), dtype=torch.float32)
            if tuple(value.shape) != tuple(want.shape):
                raise ValueError(f"the init function of {name!r} returned shape {tuple(value.shape)}, not {tuple(want.shape)}")
        elif want.init == "zeros":
            value = torch.zeros(want.shape, dtype=torch.float32)
        elif want.init == "ones_normal":
            value = 1.0 + 0.01 * torch.randn(want.shape, generator=generator, dtype=torch.float32)
        else:
            value = 0.02 * torch.randn(want.shape, generator=generator, dtype=torch.float32)
        tensors[name] = value if want.kind == "f32" else value.to(dtype)
    return tensors


def write_random_model(raw_config: dict[str, Any], out_dir: str | Path, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Create `out_dir` with config.json and model.safetensors; returns the folder."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    arch, config = resolve(raw_config)
    config_json = config.to_dict() if hasattr(config, "to_dict") else dict(raw_config)
    config_json.setdefault("architectures", [arch.name])
    config_json["torch_dtype"] = str(dtype).replace("torch.", "")
    (out_dir / "config.json").write_text(json.dumps(config_json, indent=2) + "\n")
    save_file(random_tensors(raw_config, seed, dtype), str(out_dir / "model.safetensors"))
    return out_dir
