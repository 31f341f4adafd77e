"""Shared pytest setup: marker registration, import of the hyphen-named package, fixture loaders."""
import importlib
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pkg(sub: str = ""):
    """Import pre-tjax_b200 or one of its sub-modules (the hyphen rules out a plain import statement)."""
    return importlib.import_module("pre-tjax_b200" + ("." + sub if sub else ""))


def load_golden(name: str):
    with np.load(GOLDEN / name) as z:
        return {k: z[k] for k in z.files}


def tt(a, dtype=None, device="cpu"):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(device)


@pytest.fixture(scope="session")
def ops_golden():
    return load_golden("ops_small.npz")


@pytest.fixture(scope="session")
def tiny_golden():
    return load_golden("tiny_model.npz")


@pytest.fixture(scope="session")
def cfg1_golden():
    return load_golden("cfg1_summary.npz")


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| / max |b| : relative error on the scale of the reference tensor."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    denom = float(b.abs().max())
    return float((a - b).abs().max()) / (denom if denom > 0 else 1.0)


@pytest.fixture(scope="session")
def eval_golden():
    return load_golden("eval_callers.npz")


@pytest.fixture(scope="session")
def packed_golden():
    return load_golden("packed_model.npz")
