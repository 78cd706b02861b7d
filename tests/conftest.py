import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def golden_tokens():
    return json.loads((GOLDEN / "tokens.json").read_text())


@pytest.fixture(scope="session")
def golden_votes():
    return json.loads((GOLDEN / "votes.json").read_text())


@pytest.fixture(scope="session")
def golden_eval():
    return json.loads((GOLDEN / "eval.json").read_text())


@pytest.fixture(scope="session")
def golden_model():
    return dict(np.load(GOLDEN / "model_tiny.npz"))


def tuple_preds(preds):
    return [(g, d, tuple(p) if p is not None else None) for g, d, p in preds]
