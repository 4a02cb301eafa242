"""The one registry from an architecture's name (config.json `architectures[0]`) to its model.

An architecture is two things: a typed configuration class with
`from_dict(config.json contents)`, and a function from that configuration to a
`ModelSpec` (which parts, which sizes, which order, which tensor names).  The
reference keeps the same table as `_DISPATCH` (liteinfer/models/loader.py:26-28)
and refuses unknown names listing the known ones (loader.py:96-98).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from liteinfer_b200.config.model_config import ConfigError, read_config_json
from liteinfer_b200.parts.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                       # has from_dict(dict) and to_dict()
    build_spec: Callable[[Any], ModelSpec]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build_spec: Callable[[Any], ModelSpec],
                          replace: bool = False) -> None:
    if name in ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def _builtins() -> None:
    import liteinfer_b200.architectures.llama  # noqa: F401  (registers LlamaForCausalLM)


def architecture_name(raw: dict[str, Any], where: str = "config.json") -> str:
    architectures = raw.get("architectures") or []
    if not architectures:
        raise ConfigError(f"{where} has no 'architectures' field")
    return str(architectures[0])


def resolve(raw: dict[str, Any], where: str = "config.json") -> tuple[Architecture, Any]:
    """(architecture, typed configuration) for the contents of a config.json."""
    _builtins()
    name = architecture_name(raw, where)
    if name not in ARCHITECTURES:
        raise ConfigError(f"unsupported architecture {name!r}; known: {sorted(ARCHITECTURES)}")
    arch = ARCHITECTURES[name]
    return arch, arch.config_class.from_dict(raw)


def resolve_model_dir(model_dir: str | Path) -> tuple[Architecture, Any]:
    return resolve(read_config_json(model_dir), f"config.json under {model_dir}")
