"""Pins the CPU oracle against the reference's OWN emitted CPU code: the unmodified reference
generator (ROperator_Gemm / Conv / Relu / Pool / Reshape / Softmax ::Generate) emitted headers for
the seeded cases, they ran through OpenBLAS, and their outputs are stored in
tests/golden/ref_outputs.npz (made by tests/golden/make_ref_outputs.py). Tolerance: max relative
error 1e-5 with the floor defined in helpers.rel_err (the fp32 bar of the dense-contraction path)."""
from pathlib import Path

import numpy as np
import pytest

from helpers import GOLDEN, rel_err

from oracle import build_ref, run_model

REF = np.load(GOLDEN / "ref_outputs.npz")
CASES = sorted(REF.files)


@pytest.mark.parametrize("case", CASES)
def test_oracle_matches_reference_emitted_code(case):
    m, x = build_ref.all_cases()[case]
    y = run_model.run(m, x)
    assert y.size == REF[case].size
    assert rel_err(y, REF[case]) <= 1e-5


def test_reference_library_reproduces_stored_outputs():
    """Where oracle/_ref was built (the container with the reference checkout, or the files shipped
    with it), running the reference code again must give the stored vectors."""
    from oracle import ref_runner
    if not ref_runner.available():
        pytest.skip("oracle/_ref/libsofie_ref.so not built on this machine")
    for case in ("ref_c1", "ref_conv_grp", "ref_c2_b4"):
        m, x = build_ref.all_cases()[case]
        y = ref_runner.infer(case, x, REF[case].size)
        assert rel_err(y, REF[case]) <= 2e-6  # OpenBLAS may pick another kernel on another CPU
