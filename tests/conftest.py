import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """name -> dict(score, lengths, k, row_starts|None, expected) from tests/golden/topk_golden.npz."""
    z = np.load(ROOT / "tests" / "golden" / "topk_golden.npz")
    names = sorted({k.split("/")[0] for k in z.files})
    cases = {}
    for n in names:
        cases[n] = dict(
            score=z[f"{n}/score"], lengths=z[f"{n}/lengths"], k=int(z[f"{n}/k"]),
            row_starts=z[f"{n}/row_starts"] if f"{n}/row_starts" in z.files else None,
            expected=z[f"{n}/expected"],
            # 16-bit cases: the raw bits and "bf16" / "f16"; "score" is then their exact fp32 widening
            bits16=z[f"{n}/score_bits16"] if f"{n}/score_bits16" in z.files else None,
            dtype=str(z[f"{n}/dtype"]) if f"{n}/dtype" in z.files else "f32")
    return cases


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build_c()
    return o
