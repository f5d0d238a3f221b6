"""The oracle reproduces, on the CPU, what the reference's own code returned on a B200.

tests/golden/reference_parity_{in,out}.bin were written by tests/golden/reference_vectors.py, which
runs the reference's unmodified CUDA sources (oracle/_ref/ref_harness) on a seeded input: generators,
row commitments of int and Fr tensors, a Hyrax opening, prove_matmul, prove_eleMul, combine_claims,
tLookupRange::prove and tLookupRangeMapping::prove."""
import sys
from pathlib import Path

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))

import reference_vectors as rv  # noqa: E402


def test_oracle_equals_the_reference_run():
    p = rv.read_blob(GOLDEN / rv.IN_NAME)
    # the committed inputs are the ones the generator script builds
    q = rv.build_inputs()
    for k, want in q.items():
        if hasattr(want, "shape"):
            assert (p[k].reshape(-1) == want.reshape(-1)).all(), k
        else:
            assert p[k] == want, k
    o = rv.parse_outputs(p, (GOLDEN / rv.OUT_NAME).read_bytes())
    rv.check_oracle(p, o)
