"""Extracts the reference's own golden vectors for the dense-contraction path into
tests/golden/reference_fixtures.npz + reference_fixtures.json.

Sources (read as data, in the container that has the reference checkout):
  <ref>/src/SOFIE_core/test/input_models/<Name>.onnx                 weights and attributes
  <ref>/src/SOFIE_core/test/input_models/references/<Name>.ref.hxx   expected outputs
  <ref>/src/SOFIE_core/test/TestCustomModelsFromONNX.cxx             the inputs (all-ones / iota / literals)

It also stores the fixture models themselves, byte for byte, as tests/golden/onnx/<Name>.onnx: they are the test
vectors the reference's own parser tests read, and the C++ parser of this repository is tested on those very bytes.

Run:  python tests/golden/make_golden.py [path of the reference checkout]
      (default: the environment variable SOFIE_REFERENCE_DIR, else a directory `reference` next to this repository)
The tests only read the generated files; they never touch the reference checkout.
"""
from __future__ import annotations

import json
import re
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from sofie_b200 import onnx_wire as ow  # noqa: E402

CASES = ["Linear_16", "Linear_32", "Linear_64", "ConvWithPadding", "ConvWithoutPadding", "ConvWithAutopadSameLower",
         "ConvWithStridesPadding", "ConvWithStridesNoPadding", "MaxPool2d", "MaxPool3d", "AvgPool", "Softmax1d", "Softmax2d",
         "Softmax3d", "Softmax4d", "Einsum_matmul",
         # elementwise family
         "LinearWithSelu", "LinearWithSigmoid", "LinearWithLeakyRelu", "Add", "Sub", "Mul", "Div", "Neg", "Exp", "Log", "Elu",
         "Tanh", "Sqrt", "Reciprocal",
         # broadcasting Add (rank <= 4) and transposed convolutions
         "AddBroadcast1", "AddBroadcast2", "AddBroadcast3", "AddBroadcast4", "AddBroadcast5", "AddBroadcast7",
         "ConvTranspose1d", "ConvTranspose2d", "ConvTransposeBias2d", "ConvTransposeBias2dBatched", "MaxPool1d",
         # general two-operand Einsum (expectations in the test bodies)
         "Einsum_3", "Einsum_4", "Einsum_dotprod",
         # more of the elementwise family and a graph without inputs made of a Constant node. (ConvWithAsymmetricPadding is
         # left out: the reference disables that test of its own, its generator averages unequal pads.)
         "Erf", "Abs", "Cos", "Sin", "Constant"]
# cases whose test computes its expectation from the input (`std::sin(input[i])` and the like) instead of holding a vector
COMPUTED = {"Sin": np.sin, "Cos": np.cos, "Abs": np.abs}
TEST_NAME = {"Linear_16": "Linear16", "Linear_32": "Linear32", "Linear_64": "Linear64"}
FLOAT_RE = re.compile(r"[-+]?(?:\d+\.?\d*|\.\d+)(?:[eE][-+]?\d+)?")


def floats_in_braces(text: str) -> np.ndarray:
    body = text[text.index("{") + 1: text.rindex("}")]
    return np.array([float(v) for v in FLOAT_RE.findall(body)], np.float32)


def expected_output(ref_dir: Path, name: str) -> np.ndarray | None:
    p = ref_dir / f"{name}.ref.hxx"
    if not p.exists():
        return None
    text = p.read_text()
    m = re.search(r"float\s+\w+\[\]\s*=\s*\{[^}]*\}", text, re.S)
    return floats_in_braces(m.group(0))


def test_block(src: str, test: str) -> str:
    i = src.index(f"TEST(ONNX, {test})")
    j = src.find("\nTEST(", i + 5)
    return src[i:j if j > 0 else len(src)]


def test_inputs(block: str, n_elems: list[int]) -> list[np.ndarray]:
    """Inputs as the reference test builds them: fill_n(1.0f), iota from 0, or literal vectors."""
    lits = re.findall(r"std::vector<float>\s+(?:input\w*|[ABC])\s*(?:\(\s*\{|\{)([^}]*)\}", block, re.S)
    if lits:
        return [np.array([float(v) for v in FLOAT_RE.findall(b)], np.float32) for b in lits]
    if "std::iota" in block:
        return [np.arange(n, dtype=np.float32) for n in n_elems]
    if "std::fill_n" in block:
        return [np.ones(n, np.float32) for n in n_elems]
    if not n_elems:
        return []   # a graph without inputs (Constant)
    raise ValueError("cannot find the test input")


def main():
    import os
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SOFIE_REFERENCE_DIR", ROOT.parent / "reference"))
    tdir = ref / "src/SOFIE_core/test"
    (Path(__file__).resolve().parent / "onnx").mkdir(exist_ok=True)
    src = (tdir / "TestCustomModelsFromONNX.cxx").read_text()
    arrays, manifest = {}, {}
    for name in CASES:
        raw = (tdir / "input_models" / f"{name}.onnx").read_bytes()
        (Path(__file__).resolve().parent / "onnx" / f"{name}.onnx").write_bytes(raw)
        m = ow.read_model(raw)
        block = test_block(src, TEST_NAME.get(name, name))
        graph_inputs = [(n, s) for (n, _, s) in m["inputs"] if n not in m["initializers"]]
        ins = test_inputs(block, [int(np.prod(s)) for _, s in graph_inputs])
        exp = expected_output(tdir / "input_models/references", name)
        if exp is None and name in COMPUTED:
            exp = COMPUTED[name](ins[0].astype(np.float64)).astype(np.float32)
        elif exp is None:  # Einsum_matmul keeps its expectation in the test body
            body = re.search(r"correct_output\s*=?\s*\{([^}]*)\}", block).group(1)
            # items are literals or sums of literals ("5 + 12 + 21")
            exp = np.array([sum(float(v) for v in FLOAT_RE.findall(item.replace(" ", "").replace("+", " "))) for item in body.split(",")
                            if item.strip()], np.float32)
        entry = dict(inputs=[], nodes=[], tolerance=1e-3)
        for (iname, shape), arr in zip(graph_inputs, ins):
            arrays[f"{name}/in/{iname}"] = arr.reshape(shape)
            entry["inputs"].append(iname)
        for wname, arr in m["initializers"].items():
            arrays[f"{name}/w/{wname}"] = arr
        for k, n in enumerate(m["nodes"]):
            attrs = {}
            for a, v in n["attrs"].items():
                if isinstance(v, tuple):      # a tensor attribute (Constant): (name, values, type)
                    arrays[f"{name}/attr/{k}/{a}"] = v[1]
                    attrs[a] = {"tensor": f"{name}/attr/{k}/{a}"}
                else:
                    attrs[a] = v
            entry["nodes"].append(dict(op=n["op"], inputs=n["inputs"], outputs=n["outputs"], attrs=attrs))
        arrays[f"{name}/expected"] = exp
        manifest[name] = entry
    out = Path(__file__).resolve().parent
    np.savez_compressed(out / "reference_fixtures.npz", **arrays)
    (out / "reference_fixtures.json").write_text(json.dumps(manifest, indent=1))
    print(f"wrote {len(manifest)} cases, {sum(a.nbytes for a in arrays.values())} bytes of arrays")


if __name__ == "__main__":
    main()
