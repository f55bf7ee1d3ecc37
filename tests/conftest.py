import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def ctx():
    """One native context on device 0 for the whole session (GPU tests only)."""
    import strict_b200 as sb
    c = sb.Context(0)
    yield c
    c.dispose()


@pytest.fixture(scope="session")
def parity_log():
    """Appends one JSON line per parity record (logit errors, near-tie divergences with the
    oracle's margin) to $STRICTB200_PARITY_LOG when that is set; always keeps them in memory and
    prints them at the end of the session (visible with -s / -rA)."""
    import json
    records = []
    path = os.environ.get("STRICTB200_PARITY_LOG")

    def log(rec):
        records.append(rec)
        if path:
            with open(path, "a") as f:
                f.write(json.dumps(rec) + "\n")

    yield log
    for r in records:
        print("parity:", json.dumps(r))


@pytest.fixture
def rng():
    return np.random.default_rng(1234)


# tolerances of the benchmark specification
TOL_F32 = dict(max_abs=2e-2, mean_rel=1e-3)   # fp32 / bf16 paths
TOL_FP8 = dict(max_abs=5e-2, mean_rel=5e-3)   # FP8 paths


def logits_close(got, want, max_abs, mean_rel):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    err = np.abs(got - want)
    rel = err.mean() / max(np.abs(want).mean(), 1e-30)
    return err.max() <= max_abs and rel <= mean_rel, float(err.max()), float(rel)
