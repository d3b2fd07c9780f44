"""Writes tests/golden/config_fixtures.json: size, SHA-256 and leading bytes of what the CPU oracle
(oracle/liboracle.so) produces for the seeded cases of cases.py.

    python tests/golden/make_fixtures.py

The fixtures pin both sides against drift: the oracle must keep reproducing them on CPU and the CUDA
library must reproduce them on the GPU.  They come from the oracle, not from a build of the reference
(which needs MLIR/OpenVINO); the reference's own known-answer vectors are in tests/test_golden_vectors.py.
"""
import hashlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

from cases import CASES, run_case  # noqa: E402
from oracle_backend import OracleBackend  # noqa: E402


def digest(a):
    return None if a is None else {"bytes": int(a.size), "sha256": hashlib.sha256(a.tobytes()).hexdigest(),
                                   "head": a[:32].tobytes().hex()}


def main():
    orc = OracleBackend()
    out = {}
    for name in CASES:
        folded, stream = run_case(name, orc)
        out[name] = {"folded": digest(folded), "stream": digest(stream)}
    with open(os.path.join(HERE, "config_fixtures.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")
    print(json.dumps({k: (v["folded"]["bytes"], v["stream"] and v["stream"]["bytes"]) for k, v in out.items()}))


if __name__ == "__main__":
    main()
