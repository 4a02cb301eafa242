"""Shared fixtures: tiny random model folders (in a temporary folder) and the CPU stand-in kernels."""

from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
for p in (str(ROOT), str(HERE)):
    if p not in sys.path:
        sys.path.insert(0, p)

import tiny_configs  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); skipped where there is none")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory) -> dict[str, Path]:
    """{"tiny_a": folder, ...}: written by the random-weights mode, bfloat16 tensors."""
    from liteinfer_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("models")
    return {name: write_random_model(cfg, base / name, seed) for name, (cfg, seed, _) in tiny_configs.ALL.items()}


@pytest.fixture
def cpu_kernels(monkeypatch):
    """Stands plain torch functions in for the CUDA kernels, for tests of host logic on a CPU."""
    import torch_kernels

    import liteinfer_b200.ops as ops

    for name in torch_kernels.ALL:
        monkeypatch.setattr(ops, name, getattr(torch_kernels, name))
    return torch_kernels
