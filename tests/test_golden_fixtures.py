"""The committed fixtures (tests/golden/cases.npz, written by tests/golden/make_golden.py) against the oracle built
here: the input recipes still give the same inputs and the oracle still gives the frozen answers. CPU only."""
import importlib.util
import os

import numpy as np
import pytest

import oracle as mo

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod, np.load(os.path.join(GOLDEN, "cases.npz"))


MG, FIX = load()


def test_every_case_has_a_fixture():
    assert sorted(k for k in FIX.files if not k.endswith("__insum")) == sorted(MG.CASES)


@pytest.mark.parametrize("name", sorted(MG.CASES))
def test_oracle_reproduces_fixture(name):
    kind, p = MG.CASES[name]
    ins = MG.inputs(kind, p)
    sums = np.array([float(np.sum(np.asarray(x, dtype=np.float64))) for x in ins])
    assert np.array_equal(sums, FIX[name + "__insum"]), "the input recipe changed"
    got = MG.truth(kind, p, ins)
    want = FIX[name]
    assert got.shape == want.shape
    # f64 arithmetic; only the contraction of a*b+c into one instruction may differ between hosts
    assert mo.normalised_error(got, want) <= 1e-12
