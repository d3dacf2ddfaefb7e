"""Pins the CPU oracle: it must reproduce every golden vector the reference's own tests hold for
the dense-contraction path (reference: src/SOFIE_core/test/TestCustomModelsFromONNX.cxx:330-391,
693-712,860-967,1028-1115,1966-2045,3028-3044) within the reference's tolerance of 1e-3."""
import numpy as np
import pytest

from helpers import FIXTURE_CASES, OracleBackend, load_fixtures, run_fixture


@pytest.mark.parametrize("name", FIXTURE_CASES)
def test_oracle_reproduces_reference_golden(name):
    manifest, arrays = load_fixtures()
    y = run_fixture(name, manifest, arrays, OracleBackend())
    exp = arrays[f"{name}/expected"]
    assert y.shape == exp.shape
    assert np.abs(y - exp).max() <= manifest[name]["tolerance"]
