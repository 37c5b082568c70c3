"""The committed fixtures under tests/golden against the oracle and the generators as they are now:
same seeded inputs, same quantised weights, same routing bits, same output bits."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402


@pytest.mark.parametrize("name", make_golden.SHAPES)
def test_oracle_reproduces_committed_fixture(name):
    want = np.load(os.path.join(HERE, "golden", f"block_{name}.npz"))
    got = make_golden.golden_of(name)
    assert str(got["x_sha"]) == str(want["x_sha"]), "the seeded token generator changed"
    assert str(got["router_sha"]) == str(want["router_sha"]), "the seeded router generator changed"
    assert str(got["weights_sha"]) == str(want["weights_sha"]), "the weight generator or a quantiser changed"
    assert np.array_equal(got["idx"], want["idx"]), "routing indices changed"
    assert np.array_equal(got["w_bits"], want["w_bits"]), "routing weights changed"
    assert np.array_equal(got["out_bits"], want["out_bits"]), "block output changed"
