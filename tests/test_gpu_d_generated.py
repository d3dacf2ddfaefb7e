"""The full drop-in path on the GPU: ONNX file -> RModelParser_ONNX::Parse -> RModel::Generate ->
emitted header compiled with g++ -> Session(file).infer(host pointer) -> host vector, compared with
the reference's own golden vectors, with the reference's own emitted CPU code and with the oracle."""
import numpy as np
import pytest

from helpers import FIXTURE_CASES, GOLDEN, fixture_onnx_bytes, load_fixtures, rel_err
from oracle import build_ref, run_model
from sofie_b200 import configs, generated, onnx_wire

pytestmark = pytest.mark.gpu
REF = np.load(GOLDEN / "ref_outputs.npz")


@pytest.mark.parametrize("name", FIXTURE_CASES)
def test_reference_golden_vectors_through_generated_session(name, cuda_device):
    """The reference's own .onnx file (byte for byte) -> Parse -> Generate -> g++ -> Session::infer against the expected
    output the reference's test holds for it."""
    manifest, arrays = load_fixtures()
    hxx = generated.emit(fixture_onnx_bytes(name), name)
    exp = arrays[f"{name}/expected"]
    s = generated.GeneratedSession(generated.compile_session(hxx, name), hxx.with_suffix(".dat"), exp.size)
    xs = [arrays[f"{name}/in/{i}"] for i in manifest[name]["inputs"]]  # Add, Sub, Mul, Div take two graph inputs
    y = s.infer(xs)
    assert np.abs(y - exp).max() <= 1e-3  # the reference's tolerance for its fixtures


@pytest.mark.parametrize("case", ["ref_c1", "ref_c2", "ref_c2_b4", "ref_gemm_nt", "ref_matmul", "ref_conv_grp", "ref_conv5", "ref_softmax", "ref_resblock", "ref_mlp_act", "ref_upsample"])
def test_generated_session_matches_reference_emitted_code(case, cuda_device):
    m, x = build_ref.all_cases()[case]
    s = generated.session_from_model(m, case + "_cuda")
    y1 = s.infer(x)
    y2 = s.infer(x)  # second call replays the captured graph
    assert np.array_equal(y1, y2)
    assert rel_err(y1, REF[case]) <= 1e-5


def test_generated_decoder_with_product_form_conv_transpose(cuda_device):
    """ConvTranspose layers with 32 and 16 input channels: emitted as the filter GEMM (tensor cores) plus gather, against the oracle."""
    m, x = configs.upsample_f32(batch=6, hw=16, channels=(32, 16))
    s = generated.session_from_model(m, "upsample_wide_b6")
    assert "sofie_cuda_conv_transpose2d_f32_gemm(" in s.hxx.read_text()
    y1 = s.infer(x)
    assert np.array_equal(y1, s.infer(x))
    assert rel_err(y1, run_model.run(m, x).ravel()) <= 1e-5


def test_generated_volume_network(cuda_device):
    """Conv3d + Relu, MaxPool3d, grouped strided Conv3d through the emitted Session, against the oracle."""
    m, x = configs.volume_f32(batch=3)
    s = generated.session_from_model(m, "volume_b3")
    y1 = s.infer(x)
    assert np.array_equal(y1, s.infer(x))
    assert rel_err(y1, run_model.run(m, x).ravel()) <= 1e-5


def test_generated_int8_sessions_bit_exact(cuda_device):
    m, x = configs.mlp_i8(batch=512)
    y = generated.session_from_model(m, "c3_b512").infer(x)
    assert np.array_equal(y.view(np.uint32), run_model.run(m, x).ravel().view(np.uint32))
    m, x = configs.cnn_i8(batch=8)
    y = generated.session_from_model(m, "c5_b8").infer(x)
    assert np.array_equal(y.view(np.uint32), run_model.run(m, x).ravel().view(np.uint32))


def test_missing_and_truncated_weight_file_throw(cuda_device, tmp_path):
    m, x = configs.mlp_f32(batch=16)
    s = generated.session_from_model(m, "c1_b16")
    hxx = next((generated.WORK).glob("c1_b16_*/c1_b16.hxx"))
    so = hxx.with_suffix(".so")
    with pytest.raises(RuntimeError, match="failed to open file"):
        generated.GeneratedSession(so, tmp_path / "nope.dat", 160)
    text = hxx.with_suffix(".dat").read_text()
    (tmp_path / "short.dat").write_text(text[: len(text) // 2])
    with pytest.raises(RuntimeError, match="failed to read"):
        generated.GeneratedSession(so, tmp_path / "short.dat", 160)
    (tmp_path / "renamed.dat").write_text(text.replace("tensor_W0_nk_y0", "tensor_other", 1))
    with pytest.raises(RuntimeError, match="correct tensor name"):
        generated.GeneratedSession(so, tmp_path / "renamed.dat", 160)
    assert s.infer(x).shape == (160,)


def test_binary_weight_file_gives_the_same_session(cuda_device, tmp_path):
    m, x = configs.cnn_f32(batch=4)
    y_text = generated.session_from_model(m, "c2_b4_text").infer(x)
    y_bin = generated.session_from_model(m, "c2_b4_bin", binary=True).infer(x)
    assert np.array_equal(y_text, y_bin)
    # a text weight file given to a Session generated for the binary form is refused
    hxx = generated.emit(onnx_wire.model_to_onnx(m), "c2_b4_bin", binary=True)
    so = generated.compile_session(hxx, "c2_b4_bin")
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"tensor_x 3\n1 2 3\n")
    with pytest.raises(RuntimeError, match="not the binary weight file"):
        generated.GeneratedSession(so, bad, y_bin.size)
    short = tmp_path / "short.bin"
    short.write_bytes(hxx.with_suffix(".bin").read_bytes()[:4000])
    with pytest.raises(RuntimeError, match="SOFIE failed to read"):
        generated.GeneratedSession(so, short, y_bin.size)


def test_fp8_chain_through_generated_session(cuda_device):
    import mirror_session as runner
    m, x = configs.gemm_chain_fp8(rows=512, width=512, layers=3)
    scales = configs.calibrate_fp8_scales(m, x)
    y = generated.session_from_model(m, "c4_r512", binary=True, fp8_scales=scales).infer(x)
    # the same launches as the Python mirror of the Session: identical bits
    y_mirror = runner.Session(m, fp8_scales=scales, use_graph=False).infer(x)
    assert np.array_equal(y, np.asarray(y_mirror, np.float32).ravel())
    ref = run_model.run(m, x, fp8_scales=scales)
    assert rel_err(y, ref) <= 2e-2


def test_functor_with_one_session_per_slot_on_three_threads(cuda_device, tmp_path):
    import subprocess
    from helpers import build_functor_program, tiny_regressor
    m = tiny_regressor()
    exe, dat = build_functor_program(m, "regressor", 4)
    rows = 60
    x = np.random.default_rng(5).standard_normal((rows, 4)).astype(np.float32)
    (tmp_path / "x.f32").write_bytes(x.tobytes())
    r = subprocess.run([str(exe), str(dat), str(tmp_path / "x.f32"), str(rows)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    y = np.array([float(v) for v in r.stdout.split()])
    m.input_shape = (rows, 4)
    ref = run_model.run(m, x).ravel()
    assert y.size == rows + 1
    assert rel_err(y[:rows].astype(np.float32), ref) <= 1e-5
    assert abs(y[rows] - ref[0]) <= 1e-5 * np.abs(ref).max()


def test_pipelined_upload_from_pinned_and_pageable_memory(cuda_device):
    """C2 at batch 256 with the pipelined upload forced: the emitted infer() copies the input in four parts and launches the first convolution per part.
    Pinned host memory takes the copy stream, pageable memory the staging path; both give the reference's numbers."""
    import torch
    m, x = configs.cnn_f32()
    s = generated.session_from_model(m, "c2_b256_pipe", pipelined=True)
    y_pageable = s.infer(x)
    xp = torch.from_numpy(x).pin_memory()
    yp = torch.empty(s.out_elems, dtype=torch.float32).pin_memory()
    for _ in range(3):      # eager first call, then graph replays
        s.infer_ptr(xp.data_ptr(), yp.data_ptr())
    assert np.array_equal(yp.numpy(), y_pageable)
    assert rel_err(y_pageable, REF["ref_c2"]) <= 1e-5
    # another batch through the same Session: no stale slice survives
    x2 = np.ascontiguousarray(x[::-1])
    xp.copy_(torch.from_numpy(x2))
    s.infer_ptr(xp.data_ptr(), yp.data_ptr())
    assert rel_err(yp.numpy().reshape(256, -1)[::-1], REF["ref_c2"].reshape(256, -1)) <= 1e-5


@pytest.mark.parametrize("key,batch", [("C5", 512), ("C5", 8), ("C3", 1024), ("C4", 512), ("ACT", 256), ("C2", 64), ("RES", 64)])
def test_whole_model_per_uploaded_part(key, batch, cuda_device):
    """The pipelined upload with every sliceable operator launched per quarter of the batch (C5 at 512: all of them; at 8: the last
    product stays in the graph): the results are the oracle's, from pinned and from pageable memory, call after call."""
    import torch
    if key == "C4":
        m, x = configs.gemm_chain_fp8(rows=batch, width=256, layers=2)
    elif key == "ACT":
        m, x = configs.mlp_activations_f32(batch=batch)      # Gemm, unary and binary operators (one operand a constant row): all per part
    elif key == "RES":
        m, x = configs.resblock_f32(batch=batch)             # Add of two batch-shaped tensors, both read slice by slice
    else:
        m, x = configs.BUILDERS[key](batch=batch)
    scales = configs.calibrate_fp8_scales(m, x[:64]) if key == "C4" else None
    s = generated.session_from_model(m, f"{key.lower()}_b{batch}_pipe", pipelined=True, fp8_scales=scales)
    assert "void LaunchHead(int part)" in s.hxx.read_text()
    ref = run_model.run(m, x, fp8_scales=scales).ravel() if key == "C4" else run_model.run(m, x).ravel()
    xp = torch.from_numpy(x).pin_memory()
    yp = torch.empty(s.out_elems, dtype=torch.float32).pin_memory()
    for _ in range(3):
        yp.zero_()
        s.infer_ptr(xp.data_ptr(), yp.data_ptr())
        if key == "C4":
            assert rel_err(yp.numpy(), ref) <= 2e-2
        elif key in ("ACT", "C2", "RES"):
            assert rel_err(yp.numpy(), ref) <= 1e-5
        else:
            assert np.array_equal(yp.numpy().view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(s.infer(x), yp.numpy())


def test_relu_pool_softmax_per_uploaded_part(cuda_device):
    """A model of stand-alone Relu, 3x3 MaxPool, Flatten and Softmax with the pipelined upload: all four are launched per quarter of
    the batch (slices of the elementwise count, of the images, of the rows) and give the oracle's numbers."""
    import torch
    rng = np.random.default_rng(11)
    m = configs.Model("relu_pool_softmax_b256", "x", (256, 4, 16, 16), [])
    m.layers.append(dict(op="Relu", X="x", Y="r"))
    m.layers.append(dict(op="MaxPool", X="r", Y="p", kernel=(3, 3), strides=(1, 1), pads=(1, 1, 1, 1)))
    m.layers.append(dict(op="Flatten", X="p", Y="f"))
    m.layers.append(dict(op="Softmax", X="f", Y="y", axis=1))
    m.output_name = "y"
    x = rng.standard_normal((256, 4, 16, 16)).astype(np.float32)
    s = generated.session_from_model(m, "relu_pool_softmax_b256_pipe", pipelined=True)
    text = s.hxx.read_text()
    head = text[text.index("void LaunchHead(int part)"):text.index("void Launch() {")]
    assert "sofie_cuda_relu_f32(" in head and "sofie_cuda_pool2d_f32(" in head and "sofie_cuda_softmax_f32(" in head and "void Run() {\n}" in text
    ref = run_model.run(m, x).ravel()
    xp = torch.from_numpy(x).pin_memory()
    yp = torch.empty(s.out_elems, dtype=torch.float32).pin_memory()
    for _ in range(2):
        yp.zero_()
        s.infer_ptr(xp.data_ptr(), yp.data_ptr())
        assert rel_err(yp.numpy(), ref) <= 1e-5
    assert np.array_equal(s.infer(x), yp.numpy())


@pytest.mark.parametrize("key,kw,bit_exact", [("C1", {}, False), ("C2", {}, False), ("C3", {}, True), ("C5", {}, True)])
def test_run_time_batch_session(key, kw, bit_exact, cuda_device):
    """One Session constructed for 48 samples serves batches of 48, 17, 1 and 48 again (the graph is captured anew when the
    batch changes); each result equals the oracle's for those samples, and a larger batch is refused."""
    m, x = configs.BUILDERS[key](batch=48, **kw)
    s = generated.dynamic_session_from_model(m, f"{key.lower()}_dyn48", 48)
    per = s.out_per_sample
    for bs in (48, 17, 17, 1, 48):
        mb, _ = configs.BUILDERS[key](batch=bs, with_input=False, **kw)
        ref = run_model.run(mb, x[:bs]).ravel()
        y = s.infer(x[:bs])
        assert y.size == bs * per
        if bit_exact:
            assert np.array_equal(y.view(np.uint32), ref.view(np.uint32)), bs
        else:
            assert rel_err(y, ref) <= 1e-5, bs
    with pytest.raises(RuntimeError, match="constructed for at most 48"):
        s.infer(np.zeros((49,) + x.shape[1:], np.float32))
    assert s.infer(x[:0]).size == 0


def test_conv1d_model_through_generated_session(cuda_device):
    """The reference's 1-D convolution test shape (two Conv1d layers, the second grouped) against the oracle's 2-D convolution on
    the same data seen as images of height 1, and against torch's conv1d in float64."""
    import torch
    import torch.nn.functional as F
    from helpers import conv1d_model_onnx
    from oracle import cpu_oracle as o
    for batch, length in ((1, 10), (5, 33)):
        g, w, x = conv1d_model_onnx(batch, length)
        name = f"conv1d_b{batch}_l{length}"
        hxx = generated.emit(g, name)
        t = F.relu(F.conv1d(torch.from_numpy(x).double(), torch.from_numpy(w["w0"]).double(), torch.from_numpy(w["b0"]).double(), padding=1))
        t = F.relu(F.conv1d(t, torch.from_numpy(w["w1"]).double(), torch.from_numpy(w["b1"]).double(), padding=1, groups=2)).numpy()
        r = o.conv2d_f32(x[:, :, None, :], w["w0"][:, :, None, :], w["b0"], pad=(0, 1), relu=True)
        r = o.conv2d_f32(r, w["w1"][:, :, None, :], w["b1"], pad=(0, 1), group=2, relu=True)[:, :, 0, :]
        assert r.shape == t.shape and rel_err(r, t) <= 1e-6
        s = generated.GeneratedSession(generated.compile_session(hxx, name), hxx.with_suffix(".dat"), r.size)
        assert rel_err(s.infer(x), r) <= 1e-5


def test_stacked_matmul_and_stacked_einsum_through_generated_session(cuda_device):
    rng = np.random.default_rng(8)
    a = rng.standard_normal((2, 3, 70, 64)).astype(np.float32)
    b = rng.standard_normal((2, 3, 64, 48)).astype(np.float32)
    ref = np.matmul(a.astype(np.float64), b.astype(np.float64))
    # MatMul, both operands run-time tensors
    g = onnx_wire.model("g", [onnx_wire.node("MatMul", ["a", "b"], ["y"])], [onnx_wire.value_info("a", 1, list(a.shape)), onnx_wire.value_info("b", 1, list(b.shape))],
                        [onnx_wire.value_info("y", 1, [])], [])
    hxx = generated.emit(g, "stacked_mm_run")
    s = generated.GeneratedSession(generated.compile_session(hxx, "stacked_mm_run"), hxx.with_suffix(".dat"), ref.size)
    assert rel_err(s.infer([a, b]), ref) <= 1e-5
    # MatMul with constant stacked weights followed by a bias Add (fused into the product) 
    bias = rng.standard_normal(48).astype(np.float32)
    g = onnx_wire.model("g", [onnx_wire.node("MatMul", ["a", "w"], ["h"]), onnx_wire.node("Add", ["h", "c"], ["y"])], [onnx_wire.value_info("a", 1, list(a.shape))],
                        [onnx_wire.value_info("y", 1, [])], [onnx_wire.tensor("w", b), onnx_wire.tensor("c", bias)])
    hxx = generated.emit(g, "stacked_mm_const_run")
    s = generated.GeneratedSession(generated.compile_session(hxx, "stacked_mm_const_run"), hxx.with_suffix(".dat"), ref.size)
    assert rel_err(s.infer(a), ref + bias) <= 1e-5
    # Einsum, stacked with a transposed second operand
    bt = np.ascontiguousarray(b.transpose(0, 1, 3, 2))
    g = onnx_wire.model("g", [onnx_wire.node("Einsum", ["a", "b"], ["y"], [onnx_wire.attr_str("equation", "pqik,pqjk->pqij")])],
                        [onnx_wire.value_info("a", 1, list(a.shape)), onnx_wire.value_info("b", 1, list(bt.shape))], [onnx_wire.value_info("y", 1, [])], [])
    hxx = generated.emit(g, "stacked_einsum_run")
    assert "sofie_cuda_gemm_f32_batched(" in hxx.read_text()
    s = generated.GeneratedSession(generated.compile_session(hxx, "stacked_einsum_run"), hxx.with_suffix(".dat"), ref.size)
    assert rel_err(s.infer([a, bt]), ref) <= 1e-5


def test_fp8_chain_with_scales_from_amax_at_run_time(cuda_device):
    """The FP8 chain with every activation scale computed on the device from the tensor's own max|x| (DynamicQuantizeE4M3 in front of each
    layer, the layer reading the scale from device memory) against the oracle doing the same in float32; and the scale the device
    computed for the input is bit for bit max|x| / 448."""
    import ctypes as C
    import torch
    from sofie_b200 import capi
    m, x = configs.gemm_chain_fp8(rows=512, width=1024)
    ref = run_model.run(m, x, fp8_scales="dynamic")
    s = generated.session_from_model(m, "c4_dynamic_scales", binary=True, fp8_scales="dynamic")
    y = s.infer(x)
    assert rel_err(y, ref.ravel()) <= 2e-2
    # other data through the same Session: the scales follow the data (a static calibration would saturate here)
    x2 = (x * 37.0).astype(np.float32)
    assert rel_err(s.infer(x2), run_model.run(m, x2, fp8_scales="dynamic").ravel()) <= 2e-2
    # the entry point alone: scale and codes against the oracle's quantiser
    xd = torch.from_numpy(x).to(cuda_device)
    q = torch.empty(x.shape, dtype=torch.uint8, device=cuda_device)
    sc = torch.full((1,), -1.0, device=cuda_device)
    capi.call("sofie_cuda_dynamic_quantize_e4m3_f32", None, C.c_void_p(xd.data_ptr()), C.c_void_p(q.data_ptr()), xd.numel(), C.c_void_p(sc.data_ptr()))
    torch.cuda.synchronize()
    scale = np.float32(np.abs(x).max()) / np.float32(448.0)
    assert sc.cpu().numpy()[0].view(np.uint32) == np.float32(scale).view(np.uint32)
    from oracle import cpu_oracle as o
    assert np.array_equal(q.cpu().numpy(), o.quantize_e4m3(x, float(scale)))
    z = torch.zeros(64, device=cuda_device)
    capi.call("sofie_cuda_dynamic_quantize_e4m3_f32", None, C.c_void_p(z.data_ptr()), C.c_void_p(q.data_ptr()), 64, C.c_void_p(sc.data_ptr()))
    assert float(sc.cpu()[0]) == 1.0                      # an all-zero tensor keeps a usable scale


def test_batch_sharded_over_sessions_with_the_helper(cuda_device, tmp_path):
    """SofieSharded: one batch cut into contiguous shards, one Session per shard (here three Sessions; on a box with several GPUs
    each on its own device, on one GPU all on device 0), rows back in batch order, bit-identical to the whole batch on the oracle."""
    import subprocess
    import torch
    from helpers import build_sharded_program
    m, x = configs.cnn_i8(batch=50)
    exe, dat = build_sharded_program(m, "c5_sharded")
    xin = tmp_path / "x.f32"
    x.tofile(xin)
    ngpu = torch.cuda.device_count()
    devices = [str(i % ngpu) for i in range(3)]
    r = subprocess.run([str(exe), str(dat), str(xin), "50", str(64 * 64)] + devices, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    full, small = r.stdout.split("#")
    y = np.array([float(v) for v in full.split()], np.float32)
    y7 = np.array([float(v) for v in small.split()], np.float32)
    ref = run_model.run(m, x).ravel()
    assert np.array_equal(y.view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(y7.view(np.uint32), ref[:14].view(np.uint32))
