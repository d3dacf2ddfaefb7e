"""Test infrastructure: builds oracle/_ref/libsofie_ref.so = the reference's own emitted CPU code.

For every case below the UNMODIFIED reference generator (oracle/_ref/ref_emit, compiled from the
reference sources where they lie) emits <case>.hxx + <case>.dat; the headers are compiled at -O3
with a tiny extern "C" wrapper each and linked against the multithreaded OpenBLAS that ships in
the scipy wheel. Everything lands in oracle/_ref/ (git-ignored; it travels to the GPU box as
built files). Needs the reference checkout; on a machine without it the prebuilt files are used.

usage: python oracle/build_ref.py [path of the reference checkout]
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
sys.path.insert(0, str(ROOT))
from sofie_b200 import configs  # noqa: E402

REF_OUT = HERE / "_ref"


def small_cases():
    """Extra single-operator cases with awkward sizes, seeded."""
    rng = np.random.Generator(np.random.PCG64(20260100))
    cases = {}
    # Gemm, B stored [K,N] (transB=0), alpha/beta not 1, odd sizes
    m = configs.Model("ref_gemm_nt", "x", (37, 53), [])
    m.weights["W"] = rng.standard_normal((53, 29)).astype(np.float32)
    m.weights["b"] = rng.standard_normal((29,)).astype(np.float32)
    m.layers.append(dict(op="Gemm", A="x", B="W", C="b", Y="y", transB=0, alpha=0.5, beta=2.0, relu=True))
    m.output_name = "y"
    cases["ref_gemm_nt"] = (m, rng.standard_normal((37, 53)).astype(np.float32))
    # MatMul (no bias)
    m = configs.Model("ref_matmul", "x", (8, 100), [])
    m.weights["W"] = rng.standard_normal((100, 12)).astype(np.float32)
    m.layers.append(dict(op="Gemm", A="x", B="W", Y="y", transB=0, alpha=1.0, beta=0.0, relu=False))
    m.output_name = "y"
    cases["ref_matmul"] = (m, rng.standard_normal((8, 100)).astype(np.float32))
    # strided, grouped convolution + Relu + MaxPool with pads
    m = configs.Model("ref_conv_grp", "x", (3, 4, 11, 9), [])
    m.weights["W"] = rng.standard_normal((6, 2, 3, 3)).astype(np.float32)
    m.weights["b"] = rng.standard_normal((6,)).astype(np.float32)
    m.layers.append(dict(op="Conv", X="x", W="W", B="b", Y="c", pads=(1, 1, 1, 1), strides=(2, 1), kernel=(3, 3), group=2))
    m.layers.append(dict(op="Relu", X="c", Y="r"))
    m.layers.append(dict(op="MaxPool", X="r", Y="p", kernel=(3, 2), strides=(2, 1), pads=(1, 1, 1, 1)))
    m.output_name = "p"
    cases["ref_conv_grp"] = (m, rng.standard_normal((3, 4, 11, 9)).astype(np.float32))
    # 5x5 convolution without bias, pad 2
    m = configs.Model("ref_conv5", "x", (2, 3, 12, 12), [])
    m.weights["W"] = rng.standard_normal((5, 3, 5, 5)).astype(np.float32)
    m.layers.append(dict(op="Conv", X="x", W="W", Y="c", pads=(2, 2, 2, 2), strides=(1, 1), kernel=(5, 5), group=1))
    m.output_name = "c"
    cases["ref_conv5"] = (m, rng.standard_normal((2, 3, 12, 12)).astype(np.float32))
    # softmax over the last axis of a [16, 10] tensor after a Gemm
    m = configs.Model("ref_softmax", "x", (16, 20), [])
    m.weights["W"] = rng.standard_normal((10, 20)).astype(np.float32)
    m.weights["b"] = rng.standard_normal((10,)).astype(np.float32)
    m.layers.append(dict(op="Gemm", A="x", B="W", C="b", Y="g", transB=1, alpha=1.0, beta=1.0, relu=False))
    m.layers.append(dict(op="Softmax", X="g", Y="y", axis=-1))
    m.output_name = "y"
    cases["ref_softmax"] = (m, rng.standard_normal((16, 20)).astype(np.float32))
    return cases


def all_cases():
    cases = small_cases()
    m, x = configs.mlp_f32()
    m.name = "ref_c1"
    cases["ref_c1"] = (m, x)
    m, x = configs.cnn_f32()
    m.name = "ref_c2"
    cases["ref_c2"] = (m, x)
    m, x = configs.cnn_f32(batch=4)
    m.name = "ref_c2_b4"
    cases["ref_c2_b4"] = (m, x)
    # residual block with BatchNormalization and the activation family
    m, x = configs.resblock_f32()
    m.name = "ref_resblock"
    cases["ref_resblock"] = (m, x)
    m, x = configs.mlp_activations_f32()
    m.name = "ref_mlp_act"
    cases["ref_mlp_act"] = (m, x)
    # transposed convolutions (strided, padded, output_padding, with and without bias)
    m, x = configs.upsample_f32()
    m.name = "ref_upsample"
    cases["ref_upsample"] = (m, x)
    return cases


def description(m) -> tuple[str, np.ndarray]:
    """Text description for ref_emit plus the weight blob (float32, in description order)."""
    lines = [f"model {m.name}", "input %s %s" % (m.input_name, " ".join(str(d) for d in m.input_shape))]
    blob = []
    for name, arr in m.weights.items():
        lines.append("weight %s %s" % (name, " ".join(str(d) for d in arr.shape)))
        blob.append(np.ascontiguousarray(arr, np.float32).ravel())
    for L in m.layers:
        op = L["op"]
        if op == "Gemm":
            lines.append(f"gemm {L.get('alpha', 1.0)} {L.get('beta', 1.0) if L.get('C') else 0.0} 0 {L.get('transB', 0)} "
                         f"{L['A']} {L['B']} {L.get('C') or '-'} {L['Y']} {int(bool(L.get('relu')))}")
        elif op == "Conv":
            p, s, k = L["pads"], L["strides"], L["kernel"]
            lines.append(f"conv {L.get('group', 1)} {k[0]} {k[1]} {p[0]} {p[1]} {p[2]} {p[3]} {s[0]} {s[1]} 1 1 "
                         f"{L['X']} {L['W']} {L.get('B') or '-'} {L['Y']}")
        elif op == "ConvTranspose":
            p, s, k, q = L["pads"], L["strides"], L["kernel"], L.get("output_padding", (0, 0))
            lines.append(f"convtr {k[0]} {k[1]} {p[0]} {p[1]} {p[2]} {p[3]} {s[0]} {s[1]} {q[0]} {q[1]} "
                         f"{L['X']} {L['W']} {L.get('B') or '-'} {L['Y']}")
        elif op == "Relu":
            lines.append(f"relu {L['X']} {L['Y']}")
        elif op == "MaxPool":
            p, s, k = L["pads"], L["strides"], L["kernel"]
            lines.append(f"maxpool {k[0]} {k[1]} {p[0]} {p[1]} {p[2]} {p[3]} {s[0]} {s[1]} {L['X']} {L['Y']}")
        elif op == "Flatten":
            lines.append(f"flatten {L.get('axis', 1)} {L['X']} {L['Y']}")
        elif op == "Softmax":
            lines.append(f"softmax {L.get('axis', -1)} {L['X']} {L['Y']}")
        elif op in ("Sigmoid", "Tanh", "LeakyRelu", "Selu", "Elu"):
            lines.append(f"unary {op} {L.get('alpha', 0.01 if op == 'LeakyRelu' else 1.0)} {L['X']} {L['Y']}")
        elif op in ("Add", "Sub", "Mul", "Div"):
            lines.append(f"binary {op} {L['A']} {L['B']} {L['Y']}")
        elif op == "BatchNormalization":
            lines.append(f"batchnorm {L.get('epsilon', 1e-5)} {L['X']} {L['scale']} {L['bias']} {L['mean']} {L['var']} {L['Y']} "
                         f"{int(bool(L.get('relu')))}")
        else:
            raise NotImplementedError(op)
    lines.append(f"output {m.output_name}")
    return "\n".join(lines) + "\n", np.concatenate(blob) if blob else np.zeros(0, np.float32)


WRAPPER = """#include "{name}.hxx"
#include <memory>
#include <cstring>
extern "C" long ref_{name}_infer(const char *dat, const float *x, float *y, long ny) {{
   static std::unique_ptr<SOFIE_{name}::Session> session;
   try {{
      if (!session) session.reset(new SOFIE_{name}::Session(dat));
      std::vector<float> out = session->infer(const_cast<float *>(x));
      if (y && (long)out.size() <= ny) std::memcpy(y, out.data(), out.size() * sizeof(float));
      return (long)out.size();
   }} catch (...) {{
      return -1;
   }}
}}
"""


def scipy_openblas() -> Path:
    import scipy
    libs = glob.glob(str(Path(scipy.__file__).resolve().parent.parent / "scipy.libs" / "libscipy_openblas*.so"))
    if not libs:
        raise RuntimeError("scipy's OpenBLAS not found")
    return Path(libs[0])


def reference_dir(argv=None) -> Path:
    """Where the reference checkout lies: the command line, else the environment variable SOFIE_REFERENCE_DIR, else a
    directory `reference` next to this repository."""
    if argv and len(argv) > 1:
        return Path(argv[1])
    return Path(os.environ.get("SOFIE_REFERENCE_DIR", HERE.parent.parent / "reference"))


def main(argv=None):
    ref = reference_dir(argv)
    if not (ref / "src/SOFIE_core/src/RModel.cxx").exists():
        print(f"{ref} absent: keeping the prebuilt files in {REF_OUT}")
        return 0
    subprocess.run(["make", "-C", str(HERE), f"REFERENCE={ref}", "_ref/ref_emit"], check=True)
    inc = ["-I", str(HERE / "root_shim"), "-I", str(ref / "src/SOFIE_core/inc"), "-I", str(REF_OUT)]
    objs = []
    for name, (m, x) in all_cases().items():
        text, blob = description(m)
        (REF_OUT / f"{name}.txt").write_text(text)
        blob.tofile(REF_OUT / f"{name}.f32")
        # the reference's generator prints the tensors it broadcasts: kept out of the build log
        subprocess.run([str(REF_OUT / "ref_emit"), str(REF_OUT / f"{name}.txt"), str(REF_OUT / f"{name}.f32"), str(REF_OUT)],
                       check=True, stdout=subprocess.DEVNULL)
        os.remove(REF_OUT / f"{name}.f32")
        (REF_OUT / f"{name}_wrap.cxx").write_text(WRAPPER.format(name=name))
        obj = REF_OUT / f"{name}_wrap.o"
        subprocess.run(["g++", "-std=c++20", "-O3", "-march=x86-64-v3", "-fPIC", *inc, "-c", str(REF_OUT / f"{name}_wrap.cxx"),
                        "-o", str(obj)], check=True)
        objs.append(str(obj))
    blas = scipy_openblas()
    subprocess.run(["gcc", "-O2", "-fPIC", "-c", str(HERE / "blas_shim.c"), "-o", str(REF_OUT / "blas_shim.o")], check=True)
    subprocess.run(["g++", "-shared", "-o", str(REF_OUT / "libsofie_ref.so"), *objs, str(REF_OUT / "blas_shim.o"),
                    str(REF_OUT / "SOFIE_common.o"), str(blas), f"-Wl,-rpath,{blas.parent}"], check=True)
    print("built", REF_OUT / "libsofie_ref.so")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
