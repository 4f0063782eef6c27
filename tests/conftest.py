"""Test configuration: the `gpu` marker, import paths, and helpers shared by the tests."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (config.json + model.safetensors, bfloat16-stored random weights) of
    the tiny configurations, made in a temporary folder."""
    from tiny_configs import ALL, SEEDS

    from emberserve_b200.weights.loader import write_random_model

    root = tmp_path_factory.mktemp("models")
    return {name: write_random_model(cfg, root / name, SEEDS[name]) for name, cfg in ALL.items()}
