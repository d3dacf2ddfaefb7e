"""Whole-configuration parity on the GPU: the five seeded configurations run through the C ABI
(tests/mirror_session.py = a Python mirror of the emitted Session) against
  - the reference's own emitted CPU code (stored outputs, tests/golden/ref_outputs.npz) for the fp32
    configurations at their full sizes,
  - the CPU oracle at sizes it finishes in seconds for the int8 / FP8 configurations, and
  - size-independent properties at the full sizes (sample independence, replay idempotence)."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN, rel_err
from oracle import build_ref, run_model
import mirror_session as runner
from sofie_b200 import configs

pytestmark = pytest.mark.gpu
REF = np.load(GOLDEN / "ref_outputs.npz")


@pytest.mark.parametrize("case", sorted(REF.files))
def test_fp32_models_match_reference_emitted_code(case, cuda_device):
    m, x = build_ref.all_cases()[case]
    for nhwc in (True, False):
        s = runner.Session(m, use_graph=False, nhwc=nhwc)
        y = s.infer(x)
        assert y.size == REF[case].size
        assert rel_err(y, REF[case]) <= 1e-5


def test_c1_graph_replay_and_e2e(cuda_device):
    m, x = configs.mlp_f32()
    s = runner.Session(m, use_graph=True)
    y1 = s.infer(x)
    y2 = s.infer(x)
    assert np.array_equal(y1, y2)
    assert rel_err(y1, REF["ref_c1"]) <= 1e-5
    # another batch through the same captured graph
    y3 = s.infer(x[::-1].copy())
    assert rel_err(y3[::-1], REF["ref_c1"].reshape(y3.shape)) <= 1e-5


def test_c2_intermediates_match_oracle(cuda_device):
    m, x = configs.cnn_f32(batch=8)
    ref = run_model.run(m, x, return_all=True)
    s = runner.Session(m, use_graph=False)
    t = s.infer_device(torch.from_numpy(x).cuda(), return_all=True)
    for name in ("p1", "p2", "logits"):
        y = s.output_to_nchw(name, t[name]).cpu().numpy()
        assert rel_err(y, ref[name]) <= 1e-5, name


def test_c3_int8_mlp_bit_exact(cuda_device):
    m, x = configs.mlp_i8(batch=2048)
    ref = run_model.run(m, x, return_all=True)
    s = runner.Session(m, use_graph=False)
    t = s.infer_device(torch.from_numpy(x).cuda(), return_all=True)
    for name in ("q0", "q1", "q2"):   # q3 never exists on the device: the last product writes the dequantised floats itself
        assert np.array_equal(t[name].cpu().numpy(), ref[name]), name
    assert "q3" not in t
    assert np.array_equal(t["y"].cpu().numpy().view(np.uint32), ref["y"].view(np.uint32))


def test_c3_full_size_sample_independence(cuda_device):
    """At the full batch the oracle is replaced by a property: every sample's result is independent
    of the batch it travels in, so a slice of the batch run alone gives identical bytes."""
    m, x = configs.mlp_i8()
    s = runner.Session(m, use_graph=False)
    xd = torch.from_numpy(x).cuda()
    full = s.infer_device(xd)
    part = s.infer_device(xd[4096:4096 + 512].contiguous())
    assert torch.equal(full[4096:4096 + 512], part)
    ref = run_model.run(m, x[4096:4096 + 64])
    assert np.array_equal(part[:64].cpu().numpy().view(np.uint32), ref.view(np.uint32))


def test_c5_int8_cnn_bit_exact(cuda_device):
    m, x = configs.cnn_i8(batch=24)
    ref = run_model.run(m, x, return_all=True)
    for nhwc in (True, False):
        s = runner.Session(m, use_graph=False, nhwc=nhwc)
        t = s.infer_device(torch.from_numpy(x).cuda(), return_all=True)
        for name in ("q", "p0", "p1", "p2", "p3", "f0"):   # f1 is written dequantised by its own product
            y = s.output_to_nchw(name, t[name]).cpu().numpy()
            assert np.array_equal(y, ref[name]), (name, nhwc)
        assert np.array_equal(t["y"].cpu().numpy().view(np.uint32), ref["y"].view(np.uint32))
    assert len(np.unique(ref["p3"])) > 50


def test_c4_fp8_chain(cuda_device):
    """Reduced width for the oracle (it evaluates the dequantised chain in double); tolerance 2e-2 of
    the tensor scale, layer by layer and end to end."""
    m, x = configs.gemm_chain_fp8(rows=512, width=1024)
    scales = run_model.calibrate_fp8_scales(m, x)
    ref = run_model.run(m, x, fp8_scales=scales)
    s = runner.Session(m, fp8_scales=scales, use_graph=False)
    y = s.infer(x)
    assert y.shape == ref.shape
    assert rel_err(y, ref) <= 2e-2


def test_c4_full_width_sampled_rows(cuda_device):
    """K = N = 4096 as in the configuration, 4096 rows on the GPU; the oracle checks 32 sampled rows
    (rows of a GEMM chain are independent)."""
    m, x = configs.gemm_chain_fp8(rows=4096, width=4096)
    scales = run_model.calibrate_fp8_scales(m, x)
    s = runner.Session(m, fp8_scales=scales, use_graph=False)
    y = s.infer(x)
    rows = np.random.default_rng(0).choice(4096, 32, replace=False)
    ref = run_model.run(m, x[rows], fp8_scales=scales)
    assert rel_err(y[rows], ref) <= 2e-2


# ------------------------------------------------------------------------------------ full-size configurations
def test_c5_full_batch_sampled_images_bit_exact(cuda_device):
    """C5 at its configured batch of 16384 images through the emitted Session; the oracle checks 48 images spread over
    the batch (first and last tiles of the tile walkers included). Images are independent of the batch they travel in."""
    from sofie_b200 import generated
    m, x = configs.cnn_i8()
    assert m.batch() == 16384
    y = generated.session_from_model(m, "c5_full").infer(x).reshape(16384, 2)
    rows = np.unique(np.concatenate([np.arange(8), np.arange(16376, 16384), np.random.default_rng(5).choice(16384, 32, replace=False)]))
    m_s, _ = configs.cnn_i8(batch=len(rows), with_input=False)
    ref = run_model.run(m_s, x[rows])
    assert np.array_equal(y[rows].view(np.uint32), ref.view(np.uint32))
    assert len(np.unique(y)) > 30                                   # not a constant output (uint8 codes, dequantised)


def test_c4_full_rows_sampled_rows(cuda_device):
    """C4 at its configured 65536 rows (K = N = 4096, four layers) through the emitted Session; the oracle checks 24 rows
    spread over the matrix, the last row tile included."""
    from sofie_b200 import generated
    m, x = configs.gemm_chain_fp8()
    assert m.batch() == 65536
    scales = configs.calibrate_fp8_scales(m, x[:512])
    y = generated.session_from_model(m, "c4_full", binary=True, fp8_scales=scales).infer(x).reshape(65536, 4096)
    rows = np.unique(np.concatenate([np.arange(4), np.arange(65532, 65536), np.random.default_rng(6).choice(65536, 16, replace=False)]))
    ref = run_model.run(m, x[rows], fp8_scales=scales)
    assert rel_err(y[rows], ref) <= 2e-2                            # the tolerance the benchmark definition gives FP8
    assert np.isfinite(y).all()


# ------------------------------------------------------------------------------------ fp32 accuracy, stated comparatively
def _fp64(m, x):
    """The model in float64 (torch on the CPU): the exact answer, as far as this test needs one."""
    import torch.nn.functional as F
    t = {m.input_name: torch.from_numpy(np.asarray(x, np.float64))}
    w = {k: torch.from_numpy(np.asarray(v, np.float64)) for k, v in m.weights.items()}
    for L in m.layers:
        op = L["op"]
        if op == "Gemm":
            B = w[L["B"]].T if L.get("transB") else w[L["B"]]
            y = L.get("alpha", 1.0) * (t[L["A"]] @ B)
            if L.get("C"):
                y = y + L.get("beta", 1.0) * w[L["C"]]
            t[L["Y"]] = torch.relu(y) if L.get("relu") else y
        elif op == "Conv":
            t[L["Y"]] = F.conv2d(t[L["X"]], w[L["W"]], w.get(L.get("B")), stride=tuple(L["strides"]), padding=(L["pads"][0], L["pads"][1]),
                                 groups=L.get("group", 1))
        elif op == "Relu":
            t[L["Y"]] = torch.relu(t[L["X"]])
        elif op == "MaxPool":
            t[L["Y"]] = F.max_pool2d(t[L["X"]], tuple(L["kernel"]), tuple(L["strides"]))
        elif op == "Flatten":
            t[L["Y"]] = t[L["X"]].flatten(1)
        else:
            raise NotImplementedError(op)
    return t[m.output_name].numpy()


def _floored_err(y, exact):
    """Per-element error with a floor: max_i |y_i - e_i| / max(|e_i|, 1e-3 max|e|)."""
    y, exact = np.asarray(y, np.float64).ravel(), np.asarray(exact, np.float64).ravel()
    return float((np.abs(y - exact) / np.maximum(np.abs(exact), 1e-3 * np.abs(exact).max())).max())


@pytest.mark.parametrize("case", ["ref_c1", "ref_c2", "ref_gemm_nt"])
def test_gpu_is_as_close_to_float64_as_the_reference_emitted_code(case, cuda_device):
    """Two correct fp32 evaluations of a K = 4096 dot product differ by more than 1e-5 of a small output, so the honest
    statement is comparative: measured against float64, the GPU result (3xTF32 with fp32 accumulation) is no further
    away than the reference's own emitted C++ with OpenBLAS is -- within a factor 2 -- element by element with a floor of
    1e-3 of the tensor's scale."""
    from sofie_b200 import generated
    m, x = build_ref.all_cases()[case]
    exact = _fp64(m, x)
    gpu = generated.session_from_model(m, case + "_cmp").infer(x)
    e_gpu, e_ref = _floored_err(gpu, exact), _floored_err(REF[case], exact)
    assert e_gpu <= max(2.0 * e_ref, 2e-6), (e_gpu, e_ref)
    assert e_gpu <= 1e-3 and e_ref <= 1e-3          # both are fp32 evaluations: a few ulp of the tensor's scale
