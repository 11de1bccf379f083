import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    return orc.Oracle(threads=1)


@pytest.fixture(scope="session")
def kats():
    with open(os.path.join(GOLDEN, "reference_kats.json")) as fh:
        return json.load(fh)["cases"]


@pytest.fixture(scope="session")
def seeded():
    return dict(np.load(os.path.join(GOLDEN, "seeded_cases.npz")))


def expected_of(case):
    return np.array(case["expected_bits"], np.uint32).view(np.float32)


def run_kat(impl, case):
    """Runs one reference known-answer case on `impl` (the oracle, the compiled
    reference kernels, or the CUDA builtins: all expose the same method names)."""
    i = case["inputs"]
    f = lambda k: np.array(i[k], np.float32)
    b = case["builtin"]
    if b == "fadd":
        return impl.fadd(f("a"), i["scaleA"], f("b"), i["scaleB"])
    if b == "fmul":
        return impl.fmul(f("a"), f("b"))
    if b == "fdivide":
        return impl.fdivide(f("a"), f("b"))
    if b == "fmulconcat":
        return impl.fmulconcat(f("gradient"), f("local"))
    if b == "fsigmoid":
        return impl.fsigmoid(f("a"))
    if b == "flogloss":
        return impl.flogloss(f("predicted"), f("groundTruth"))
    if b == "fmatmul":
        left = f("left").reshape(i["left_shape"])
        right = f("right").reshape(i["right_shape"])
        return impl.fmatmul(i["tl"], i["tr"], left, right)
    raise KeyError(b)
