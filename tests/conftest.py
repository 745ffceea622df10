import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_npz(name):
    with np.load(GOLDEN / name) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def triton_ops():
    return {k: torch.from_numpy(v) for k, v in load_npz("triton_ops.npz").items()}


@pytest.fixture(scope="session")
def hf_llada():
    raw = load_npz("hf_llada.npz")
    meta = json.loads(bytes(raw.pop("meta")).decode())
    weights = {k[3:]: torch.from_numpy(v) for k, v in raw.items() if k.startswith("w::")}
    arrays = {k: v for k, v in raw.items() if not k.startswith("w::")}
    return meta, weights, arrays


def _hf_fixture(name):
    raw = load_npz(name)
    meta = json.loads(bytes(raw.pop("meta")).decode())
    weights = {k[3:]: torch.from_numpy(v) for k, v in raw.items() if k.startswith("w::")}
    arrays = {k: v for k, v in raw.items() if not k.startswith("w::")}
    return meta, weights, arrays


@pytest.fixture(scope="session")
def hf_dream():
    return _hf_fixture("hf_dream.npz")


@pytest.fixture(scope="session")
def hf_llada_dkv():
    return _hf_fixture("hf_llada_dkv.npz")


@pytest.fixture(scope="session")
def hf_dream_dkv():
    return _hf_fixture("hf_dream_dkv.npz")


@pytest.fixture(scope="session")
def layout_cases():
    return json.loads((GOLDEN / "layout.json").read_text())
