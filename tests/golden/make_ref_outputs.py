"""Runs the reference's own emitted CPU code (oracle/_ref, see oracle/build_ref.py) on the seeded
parity cases and stores its outputs in tests/golden/ref_outputs.npz, so that the parity tests can
compare against the reference where the reference checkout does not exist.

Run (in the container that has the reference):  python oracle/build_ref.py && python tests/golden/make_ref_outputs.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref, ref_runner  # noqa: E402
from oracle import run_model  # noqa: E402


def main():
    out = {}
    for name, (m, x) in build_ref.all_cases().items():
        n_out = run_model.run(m, x).size  # the oracle gives the output size
        out[name] = ref_runner.infer(name, x, n_out)
    np.savez_compressed(Path(__file__).resolve().parent / "ref_outputs.npz", **out)
    print({k: v.shape for k, v in out.items()}, ref_runner.blas_config(), ref_runner.threads())


if __name__ == "__main__":
    main()
