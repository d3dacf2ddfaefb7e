"""Whole-configuration parity on the GPU: the five seeded configurations run through the C ABI
(sofie_b200.runner.Session = the Python mirror of the emitted Session) against
  - the reference's own emitted CPU code (stored outputs, tests/golden/ref_outputs.npz) for the fp32
    configurations at their full sizes,
  - the CPU oracle at sizes it finishes in seconds for the int8 / FP8 configurations, and
  - size-independent properties at the full sizes (sample independence, replay idempotence)."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN, rel_err
from oracle import build_ref, run_model
from sofie_b200 import configs, runner

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
