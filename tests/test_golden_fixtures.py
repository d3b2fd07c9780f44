"""The committed fixtures of tests/golden/ (made by tests/golden/make_fixtures.py from the CPU oracle)
against the oracle on CPU and against the CUDA library, through the C ABI, on the GPU box."""
import hashlib
import json
import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from cases import CASES, run_case  # noqa: E402

with open(os.path.join(HERE, "golden", "config_fixtures.json")) as f:
    FIXTURES = json.load(f)


def check(got, want, what):
    if want is None:
        assert got is None, f"{what}: expected 'not smaller'"
        return
    assert got is not None, f"{what}: missing"
    assert got.size == want["bytes"], f"{what}: {got.size} bytes, fixture has {want['bytes']}"
    assert got[:32].tobytes().hex() == want["head"], what
    assert hashlib.sha256(got.tobytes()).hexdigest() == want["sha256"], what


@pytest.mark.parametrize("name", sorted(CASES))
def test_fixture(backend, name):
    folded, stream = run_case(name, backend)
    check(folded, FIXTURES[name]["folded"], name + " folded")
    check(stream, FIXTURES[name]["stream"], name + " stream")
