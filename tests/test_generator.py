"""The C++ generator (sofie_b200/host): same user-facing flow as the reference --
RModelParser_ONNX::Parse -> RModel::Generate -> OutputGenerated -- checked without a GPU: the models
parse, the emitted header has the reference's Session / infer signatures, calls only libSOFIE_cuda,
and compiles and links with a plain C++17 compiler."""
import re

import numpy as np
import pytest

from helpers import FIXTURE_CASES, REENCODABLE_CASES, build_functor_program, fixture_onnx_bytes, fixture_to_onnx, load_fixtures, tiny_regressor
from sofie_b200 import configs, generated, onnx_wire


def _emit(model, name):
    return generated.emit(onnx_wire.model_to_onnx(model), name)


def test_c2_header_has_reference_signatures_and_fused_plan():
    m, _ = configs.cnn_f32(batch=8)
    hxx = _emit(m, "c2_b8")
    text = hxx.read_text()
    assert "namespace SOFIE_c2_b8{" in text
    assert 'Session(std::string filename ="c2_b8.dat")' in text
    assert "std::vector<float> infer(float* tensor_x){" in text
    assert '#include "sofie_cuda.h"' in text and "sgemm_" not in text and "Im2col" not in text
    # Conv+Relu(+MaxPool) collapse into three launches, Flatten is an alias, one Gemm
    assert text.count("sofie_cuda_conv2d_f32(") == 3 and text.count("sofie_cuda_gemm_f32(") == 1
    assert "sofie_cuda_relu_f32(" not in text and "sofie_cuda_pool2d_f32(" not in text
    assert "dev_flat = reinterpret_cast<float*>(dev_p2);" in text
    # layouts: first conv reads NCHW and writes NHWC; later convs read packed weights
    descs = re.findall(r"sofie_conv2d_desc d = \{([^}]*)\}", text)
    fields = [[int(v) for v in d.split(",")] for d in descs]
    assert [f[14:17] for f in fields] == [[0, 1, 0], [1, 1, 1], [1, 1, 1]]       # x_layout, y_layout, w_packed
    assert [f[17:19] for f in fields] == [[1, 0], [1, 2], [1, 2]]                # relu, pool
    dat = hxx.with_suffix(".dat").read_text().split()
    assert dat[0] == "tensor_cb0" and dat[1] == "16"


def test_arena_slices_do_not_overlap_while_alive():
    m, _ = configs.mlp_activations_f32(batch=64)   # Gemm / activation / binary operators alternate: nothing fuses away
    text = _emit(m, "mlp_act_b64").read_text()
    slices = {n: (int(o), int(b)) for o, b, n in re.findall(r"sofie_cuda_ctx_arena\(fCtx, (\d+), (\d+), reinterpret_cast<void\*\*>\(&dev_(\w+)\)", text)}
    assert {"x", "g0", "a0", "g1", "a1", "sh", "g2", "a2", "d"} <= set(slices)
    # the small result is not in the arena at all: the last kernel writes it into mapped host memory
    assert "y" not in slices and re.search(r"sofie_cuda_ctx_host_output\(fCtx, \d+, reinterpret_cast<void\*\*>\(&dev_y\)\)", text)
    # an operator's input and output are alive together: their slices are disjoint
    for a, b in [("x", "g0"), ("g0", "a0"), ("a0", "g1"), ("g1", "a1"), ("a1", "sh"), ("sh", "g2"), ("g2", "a2"), ("a2", "d")]:
        (o0, b0), (o1, b1) = slices[a], slices[b]
        assert o0 + b0 <= o1 or o1 + b1 <= o0, (a, b)
    assert all(o % 256 == 0 for o, _ in slices.values())
    arena = int(re.search(r"sofie_cuda_ctx_create\(&fCtx, -1, (\d+)\)", text).group(1))
    assert arena >= max(o + b for o, b in slices.values())
    # slices are reused once their tensor is dead: the arena is smaller than the sum of all slices
    assert arena < sum(b for _, b in slices.values())


def test_small_gemm_chain_is_one_fused_launch():
    m, _ = configs.mlp_f32(batch=64)
    text = _emit(m, "c1_b64").read_text()
    assert text.count("sofie_cuda_mlp_f32(") == 1 and "sofie_cuda_gemm_f32(" not in text
    assert "{64, 3, {64, 128, 128, 10}, {1, 1, 0}, {1, 1, 1}}" in text
    # the intermediate activations of the chain have no arena slice any more
    assert "dev_y0" not in text and "dev_y1" not in text
    # a wide layer is outside the fused kernel: one GEMM per layer again
    m2 = configs.Model("wide", "x", (16, 300), [])
    rng = np.random.default_rng(0)
    m2.weights["w0"] = rng.standard_normal((64, 300)).astype(np.float32)
    m2.weights["w1"] = rng.standard_normal((8, 64)).astype(np.float32)
    m2.layers.append(dict(op="Gemm", A="x", B="w0", Y="h", transB=1, relu=True))
    m2.layers.append(dict(op="Gemm", A="h", B="w1", Y="y", transB=1))
    m2.output_name = "y"
    text2 = _emit(m2, "wide").read_text()
    assert text2.count("sofie_cuda_gemm_f32(") == 2 and "sofie_cuda_mlp_f32(" not in text2


@pytest.mark.parametrize("key,kw", [("C1", {}), ("C2", {"batch": 4}), ("C3", {"batch": 32}), ("C5", {"batch": 2})])
def test_configurations_emit_and_compile(key, kw):
    m, _ = configs.BUILDERS[key](**kw)
    name = f"{key.lower()}_gen"
    hxx = _emit(m, name)
    so = generated.compile_session(hxx, name)
    assert so.exists()


@pytest.mark.parametrize("name", FIXTURE_CASES)
def test_reference_fixture_files_parse_and_emit(name):
    """The reference's own .onnx files, byte for byte, through RModelParser_ONNX::Parse and Generate."""
    hxx = generated.emit(fixture_onnx_bytes(name), name)
    text = hxx.read_text()
    assert "infer(" in text and f"namespace SOFIE_{name}" in text


@pytest.mark.parametrize("name", REENCODABLE_CASES)
def test_reencoded_fixture_graphs_emit_the_same_launches(name):
    """The test-side ONNX writer against the reference's files: both spellings of a graph give the same calls."""
    manifest, arrays = load_fixtures()
    calls = lambda hxx: re.findall(r"Check\((sofie_cuda_(?!ctx_)\w+)\(", hxx.read_text())
    assert calls(generated.emit(fixture_to_onnx(name, manifest, arrays), name + "_rewritten")) == calls(generated.emit(fixture_onnx_bytes(name), name))


def test_constant_and_identity_nodes_become_initialised_tensors():
    w = np.arange(6, dtype=np.float32).reshape(3, 2)
    shape = np.array([2, 3], np.int64)
    g = onnx_wire.model("g", [onnx_wire.node("Constant", [], ["shape"], [onnx_wire.attr_tensor("value", "s", shape)]),
                              onnx_wire.node("Identity", ["w"], ["w2"]),
                              onnx_wire.node("MatMul", ["x", "w2"], ["h"]),
                              onnx_wire.node("Identity", ["h"], ["h2"]),
                              onnx_wire.node("Reshape", ["h2", "shape"], ["y"])],
                        [onnx_wire.value_info("x", 1, [3, 3])], [onnx_wire.value_info("y", 1, [])], [onnx_wire.tensor("w", w)])
    text = generated.emit(g, "const_ident").read_text()
    # the shared weight is uploaded under its second name, the run-time Identity and the Reshape are aliases, one GEMM runs
    assert text.count("sofie_cuda_gemm_f32(") == 1 and "Identity op_" in text and "Reshape op_" in text
    assert "tensor_w2" in text.replace("dev_", "tensor_") and "tensor_shape" not in text
    with pytest.raises(RuntimeError, match="not yet supporting attribute"):
        generated.emit(onnx_wire.model("g", [onnx_wire.node("Constant", [], ["c"], [onnx_wire.attr_str("value_string", "a")]),
                                             onnx_wire.node("Relu", ["x"], ["y"])],
                                       [onnx_wire.value_info("x", 1, [2])], [onnx_wire.value_info("y", 1, [])], []), "const_bad")


def test_unsupported_operator_and_bad_file_raise():
    with pytest.raises(RuntimeError, match="not yet supported"):
        generated.emit(onnx_wire.model("g", [onnx_wire.node("LSTM", ["x"], ["y"])], [onnx_wire.value_info("x", 1, [1, 2, 3])],
                                       [onnx_wire.value_info("y", 1, [])], []), "bad_op")
    with pytest.raises(RuntimeError):
        generated.emit(b"\x00\x01garbage", "bad_file")


def test_session_without_gpu_throws_the_reference_way():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    m, _ = configs.mlp_f32(batch=4)
    with pytest.raises(RuntimeError, match="SOFIE CUDA"):
        generated.session_from_model(m, "c1_nogpu")


def test_batchnorm_is_folded_into_the_convolution_and_emitted_alone_otherwise():
    m, _ = configs.resblock_f32(batch=2)
    text = generated.emit(onnx_wire.model_to_onnx(m), "resblock_fold").read_text()
    assert text.count("sofie_cuda_conv2d_f32(") == 2
    assert "sofie_cuda_batchnorm_f32(" not in text          # both normalisations live in the conv weights
    assert text.count("sofie_cuda_binary_f32(") == 2 and "sofie_cuda_unary_f32(" in text
    # a normalisation that does not follow a convolution stays an operator of its own
    m2 = configs.Model("bn_alone", "x", (2, 4, 6, 6), [])
    rng = np.random.default_rng(1)
    for k in ("g", "b", "mu", "v"):
        m2.weights[k] = rng.uniform(0.5, 1.5, 4).astype(np.float32)
    m2.layers.append(dict(op="MaxPool", X="x", Y="p", kernel=(2, 2), strides=(2, 2), pads=(0, 0, 0, 0)))
    m2.layers.append(dict(op="BatchNormalization", X="p", Y="y", scale="g", bias="b", mean="mu", var="v", relu=True))
    m2.output_name = "y"
    text2 = generated.emit(onnx_wire.model_to_onnx(m2), "bn_alone").read_text()
    assert "sofie_cuda_batchnorm_f32(" in text2 and "BatchNorm" in text2 and "+ Relu" in text2
    assert "sofie_cuda_relu_f32(" not in text2               # the Relu behind it is fused as the reference does


def test_binary_weight_file_option_emits_and_compiles():
    m, _ = configs.cnn_f32(batch=2)
    hxx = generated.emit(onnx_wire.model_to_onnx(m), "c2_binary", binary=True)
    text = hxx.read_text()
    assert 'Session(std::string filename ="c2_binary.bin"' in text and "SOFIEBW1" in text and "std::fread" in text
    blob = hxx.with_suffix(".bin").read_bytes()
    assert blob[:8] == b"SOFIEBW1" and not hxx.with_suffix(".dat").exists()
    # every weight is stored once, raw: the file is barely larger than the weights themselves
    nbytes = sum(v.nbytes for v in m.weights.values())
    assert nbytes <= len(blob) <= nbytes + 4096
    generated.compile_session(hxx, "c2_binary")


def test_fp8_chain_parses_and_emits_through_the_generator():
    m, x = configs.gemm_chain_fp8(rows=128, width=256, layers=3)
    scales = configs.calibrate_fp8_scales(m, x)
    hxx = generated.emit(onnx_wire.model_to_onnx(m, scales), "c4_tiny", binary=True)
    text = hxx.read_text()
    assert text.count("sofie_cuda_gemm_e4m3(") == 2 and text.count("sofie_cuda_quantize_e4m3_f32(") == 1
    # the Cast to float behind the last layer is written by that layer's own launch
    assert text.count("sofie_cuda_gemm_e4m3_f32(") == 1 and "sofie_cuda_cast_bf16_f32(" not in text
    assert re.search(r"std::vector<float>\s+infer\(float\*\s*tensor_x\)", text)
    generated.compile_session(hxx, "c4_tiny")
    with pytest.raises(ValueError):
        onnx_wire.model_to_onnx(m)  # the chain cannot be written without its calibrated scales


def test_conv_transpose_emits_one_call_and_refuses_what_the_reference_refuses():
    m, _ = configs.upsample_f32(batch=2)
    text = _emit(m, "upsample_b2").read_text()
    assert text.count("sofie_cuda_conv_transpose2d_f32(") == 2 and "_xcol" not in text and "col2im" not in text
    descs = re.findall(r"sofie_conv_transpose2d_desc d = \{([^}]*)\}", text)
    assert [int(v) for v in descs[0].split(",")] == [2, 8, 12, 12, 6, 2, 2, 0, 0, 2, 2, 1, 1, 0, 0, 0]
    assert [int(v) for v in descs[1].split(",")] == [2, 6, 24, 24, 3, 3, 3, 1, 1, 2, 2, 1, 1, 1, 1, 0]
    generated.compile_session(_emit(m, "upsample_b2"), "upsample_b2")
    # 16 or more input channels: the product form (one GEMM for all images, then a gather) with its slice of the arena,
    # which lives only during the operator; with a run-time batch the direct kernel is kept
    m, _ = configs.upsample_f32(batch=2, channels=(32, 16))
    text = _emit(m, "upsample_wide_b2").read_text()
    assert text.count("sofie_cuda_conv_transpose2d_f32_gemm(") == 2 and "sofie_cuda_conv_transpose2d_f32(" not in text
    assert "dev_u1_products" in text and "dev_u2_products" in text
    generated.compile_session(_emit(m, "upsample_wide_b2"), "upsample_wide_b2")
    dyn = generated.emit(onnx_wire.model_to_onnx(m, batch_param="bs"), "upsample_wide_dyn").read_text()
    assert "sofie_cuda_conv_transpose2d_f32_gemm(" not in dyn and dyn.count("sofie_cuda_conv_transpose2d_f32(") == 2

    def graph(attrs):
        w = np.zeros((3, 2, 3, 3), np.float32)
        return onnx_wire.model("g", [onnx_wire.node("ConvTranspose", ["x", "w"], ["y"], attrs)], [onnx_wire.value_info("x", 1, [1, 3, 4, 4])],
                               [onnx_wire.value_info("y", 1, [])], [onnx_wire.tensor("w", w)])
    with pytest.raises(RuntimeError, match="output_shape explicitly set"):
        generated.emit(graph([onnx_wire.attr_ints("output_shape", [8, 8])]), "convtr_oshape")
    with pytest.raises(RuntimeError, match="group"):
        generated.emit(graph([onnx_wire.attr_int("group", 3)]), "convtr_group")


def test_sessions_are_movable_and_the_functor_helper_compiles():
    exe, dat = build_functor_program(tiny_regressor(), "regressor", 4)
    assert exe.exists() and dat.exists()
    text = exe.with_name("regressor.hxx").read_text()
    assert "Session(Session && other) noexcept" in text and "other.fCtx = nullptr;" in text


def test_large_input_is_uploaded_in_parts_under_the_first_convolution():
    m, _ = configs.cnn_f32(batch=256)
    text = generated.emit(onnx_wire.model_to_onnx(m), "c2_b256", pipelined=True).read_text()
    # four copies on the copy stream, the first convolution once per part, the rest of the model as the captured graph
    assert "void LaunchHead(int part)" in text and text.count("sofie_cuda_ctx_h2d_part(") == 1 and "sofie_cuda_ctx_wait_part(fCtx, part)" in text
    assert "const sofie_conv2d_desc d = {64, 3, 32, 32, 16," in text       # a quarter of the batch per launch
    assert "dev_x + (size_t)part * 196608" in text and "dev_r0 + (size_t)part * 1048576" in text
    assert text.count("sofie_cuda_conv2d_f32(") == 3 and "sofie_cuda_ctx_h2d(fCtx" not in text
    # without the option an input of a few megabytes is copied in one piece (a copy's fixed cost outweighs the overlap) ...
    plain = _emit(m, "c2_b256").read_text()
    assert "LaunchHead" not in plain and "sofie_cuda_ctx_h2d(fCtx, dev_x" in plain
    # ... and from 32 MB on the parts come by themselves
    big = _emit(configs.cnn_f32(batch=4096, with_input=False)[0], "c2_b4096").read_text()
    assert "void LaunchHead(int part)" in big and "const sofie_conv2d_desc d = {1024, 3, 32, 32, 16," in big


def test_every_leading_operator_that_can_be_sliced_runs_per_uploaded_part():
    """C5 with the pipelined upload: QuantizeLinear, the four convolutions, Flatten and both products are launched per quarter of the
    batch, nothing is left for the graph. At a batch whose last tensor does not split into 256-byte aligned quarters the last product
    stays behind, in Launch()."""
    m, _ = configs.cnn_i8(batch=512, with_input=False)
    text = generated.emit(onnx_wire.model_to_onnx(m), "c5_b512_pipe", pipelined=True).read_text()
    head = text[text.index("void LaunchHead(int part)"):text.index("void Launch() {")]
    assert head.count("sofie_cuda_quantize_u8(") == 1 and head.count("sofie_cuda_qlinear_conv2d(") == 4
    assert head.count("sofie_cuda_qlinear_matmul(") == 1 and head.count("sofie_cuda_qlinear_matmul_f32(") == 1
    assert "const sofie_qconv2d_desc d = {128, 1, 64, 64, 32," in head and "const sofie_qgemm_desc d = {128, 2, 256," in head
    assert "(dev_x + (size_t)part * 524288)" in head and "(dev_y + (size_t)part * 256)" in head
    assert "void Run() {\n}" in text and "sofie_cuda_ctx_graph_begin" not in text
    small = generated.emit(onnx_wire.model_to_onnx(configs.cnn_i8(batch=8, with_input=False)[0]), "c5_b8_pipe", pipelined=True).read_text()
    head = small[small.index("void LaunchHead(int part)"):small.index("void Launch() {")]
    tail = small[small.index("void Launch() {"):small.index("void Run() {")]
    assert head.count("sofie_cuda_qlinear_matmul(") == 1 and "sofie_cuda_qlinear_matmul_f32(" not in head
    assert "sofie_cuda_qlinear_matmul_f32(fStream, &d, dev_f0," in tail and "sofie_cuda_ctx_graph_begin" in small


def test_inputs_of_128_mb_and_more_are_uploaded_in_eight_parts():
    """C5 at its full batch (268 MB of floats) without any option: eight parts of 2048 images, every operator launched per part;
    half the batch (134 MB) still eight parts, a quarter (67 MB) four."""
    for batch, parts in ((16384, 8), (8192, 8), (4096, 4)):
        m, _ = configs.cnn_i8(batch=batch, with_input=False)
        text = _emit(m, f"c5_b{batch}").read_text()
        assert f"for (int part = 0; part < {parts}; part++) LaunchHead(part);" in text
        per = batch // parts
        assert f"const sofie_qconv2d_desc d = {{{per}, 1, 64, 64, 32," in text and f"(dev_x + (size_t)part * {per * 4096})" in text
        assert f"sofie_cuda_ctx_h2d_part(fCtx, dev_x + (size_t)part * {per * 4096}, tensor_x + (size_t)part * {per * 4096}, {per * 4096 * 4}, part)" in text


def test_sliced_operators_end_at_the_first_one_that_cannot_be_sliced():
    """The decoder stack: the convolution (Relu fused) runs per uploaded part; the ConvTranspose behind it has no sliced form, so it
    and everything after it stay in the graph. The MLP with Sub / Div of constant rows between its layers is sliced throughout:
    a binary operator reads its batch-shaped operand slice by slice and the constant one whole."""
    m, _ = configs.upsample_f32(batch=64, with_input=False)
    text = generated.emit(onnx_wire.model_to_onnx(m), "upsample_b64_pipe", pipelined=True).read_text()
    head = text[text.index("void LaunchHead(int part)"):text.index("void Launch() {")]
    tail = text[text.index("void Launch() {"):text.index("void Run() {")]
    assert head.count("sofie_cuda_conv2d_f32(") == 1 and "sofie_cuda_conv_transpose2d" not in head and "one of 4 slices of the batch" in head
    assert tail.count("sofie_cuda_conv_transpose2d_f32") >= 2 and "part" not in tail.replace("sofie_cuda_ctx_mark", "")
    m, _ = configs.mlp_activations_f32(batch=256, with_input=False)
    text = generated.emit(onnx_wire.model_to_onnx(m), "mlp_act_b256_pipe", pipelined=True).read_text()
    head = text[text.index("void LaunchHead(int part)"):text.index("void Launch() {")]
    assert head.count("sofie_cuda_gemm_f32(") == 3 and head.count("sofie_cuda_unary_f32(") == 4 and head.count("sofie_cuda_binary_f32(") == 2
    assert "const sofie_gemm_f32_desc d = {64, 48, 32," in head and "void Run() {\n}" in text
    # Sub of a constant row [48] from [256, 48]: 64 rows per launch, the activation sliced, the row whole
    assert "{1, 1, 64, 48}, {0, 0, 48, 1}, {0, 0, 0, 1}" in head and "(dev_a1 + (size_t)part * 3072), dev_shift, (dev_sh + (size_t)part * 3072)" in head


def test_tensors_of_sliced_operators_share_no_arena_bytes():
    """Slice 1 of a model's first tensor is written after slice 0 of its last one, and the input's later parts arrive in between:
    the tensors of the operators launched per part must not reuse each other's bytes, as tensors of a whole-batch plan do."""
    import re

    def slices(text):
        return {n: (int(o), int(b)) for o, b, n in re.findall(r"sofie_cuda_ctx_arena\(fCtx, (\d+), (\d+), reinterpret_cast<void\*\*>\(&dev_(\w+)\)\)", text)}

    def overlaps(sl):
        names = sorted(sl)
        return [(a, b) for i, a in enumerate(names) for b in names[i + 1:]
                if sl[a][0] < sl[b][0] + sl[b][1] and sl[b][0] < sl[a][0] + sl[a][1]]

    for m, tag in ((configs.cnn_f32(batch=256, with_input=False)[0], "c2_b256"), (configs.cnn_i8(batch=512, with_input=False)[0], "c5_b512")):
        onnx = onnx_wire.model_to_onnx(m)
        piped = slices(generated.emit(onnx, tag + "_pipe", pipelined=True).read_text())
        whole = slices(generated.emit(onnx, tag + "_whole", pipelined=False).read_text())
        assert piped.keys() == whole.keys() and len(piped) >= 4
        assert overlaps(piped) == []
        assert overlaps(whole) != []         # the whole-batch plan does reuse dead tensors' bytes


def test_trailing_dequantize_is_written_by_the_last_quantised_product():
    m, _ = configs.mlp_i8(batch=64)
    text = _emit(m, "c3_b64").read_text()
    assert text.count("sofie_cuda_qlinear_matmul(") == 2 and text.count("sofie_cuda_qlinear_matmul_f32(") == 1
    assert "sofie_cuda_dequantize_u8(" not in text and not re.search(r"\bdev_q3\b", text)   # the uint8 tensor has no slice


def test_einsum_goes_to_the_gemm_or_to_the_general_kernel_and_refuses_the_rest():
    def graph(eq, sa, sb, n_in=2):
        names = ["a", "b", "c"][:n_in]
        shapes = [sa, sb, sb][:n_in]
        return onnx_wire.model("g", [onnx_wire.node("Einsum", names, ["y"], [onnx_wire.attr_str("equation", eq)])],
                               [onnx_wire.value_info(n, 1, list(s)) for n, s in zip(names, shapes)], [onnx_wire.value_info("y", 1, [])], [])
    plain = generated.emit(graph("ik,kj->ij", (4, 5), (5, 6)), "einsum_mm").read_text()
    assert "sofie_cuda_gemm_f32(" in plain and "sofie_cuda_einsum_f32(" not in plain
    # a stacked matrix product reaches the GEMM kernels too, one product per stack index (either operand may be transposed)
    bmm = generated.emit(graph("bij, bjk -> bik", (3, 4, 5), (3, 5, 2)), "einsum_bmm").read_text()
    assert "const sofie_gemm_f32_desc d = {4, 2, 5, 0, 0, 1.0f, 0.0f, 0, 0};" in bmm
    assert "sofie_cuda_gemm_f32_batched(fStream, &d, dev_a, dev_b, nullptr, dev_y, 3, 20, 10, 8)" in bmm and "sofie_cuda_einsum_f32(" not in bmm
    bmm_t = generated.emit(graph("abki,abjk->abij", (2, 3, 5, 4), (2, 3, 6, 5)), "einsum_bmm_t").read_text()
    assert "const sofie_gemm_f32_desc d = {4, 6, 5, 1, 1, 1.0f, 0.0f, 0, 0};" in bmm_t and ", 6, 20, 30, 24)" in bmm_t
    # anything else (here the stack label sits in another position of the output) is the general kernel
    general = generated.emit(graph("bij, bjk -> ibk", (3, 4, 5), (3, 5, 2)), "einsum_general").read_text()
    assert "const sofie_einsum_desc d = {3, 1, {4, 3, 2, 5, 0, 0, 0, 0}, {5, 20, 0, 1, 0, 0, 0, 0}, {0, 10, 1, 2, 0, 0, 0, 0}};" in general
    for eq, sa, sb, n_in, what in (("...ij,...jk->...ik", (3, 4, 5), (3, 5, 2), 2, "ellipsis"), ("ii,ij->j", (4, 4), (4, 3), 2, "repeated"),
                                   ("ij,jk,kl->il", (2, 3), (3, 4), 3, "operands"), ("ij,kk->i", (2, 3), (3, 4), 2, "repeated|extents")):
        with pytest.raises(RuntimeError, match=what):
            generated.emit(graph(eq, sa, sb, n_in), "einsum_bad")


def _emit_and_compile_worker(tag, out):
    # what every rank of a multi-GPU run does at start-up: same model, same name, at the same moment
    import ctypes
    try:
        m, _ = configs.cnn_f32(batch=6)
        hxx = generated.emit(onnx_wire.model_to_onnx(m), "race_c2_b6")
        so = generated.compile_session(hxx, "race_c2_b6")
        lib = ctypes.CDLL(str(so))
        ok = all(hasattr(lib, f) for f in ("sofie_session_create", "sofie_session_infer", "sofie_session_destroy"))
        dat = hxx.with_suffix(".dat").read_text().split()
        out.put((tag, str(so), ok and dat[0] == "tensor_cb0" and len(dat) > 1000, ""))
    except BaseException as e:  # reported to the parent instead of lost with the child
        out.put((tag, "", False, f"{type(e).__name__}: {e}"))


def test_eight_processes_emit_and_compile_the_same_model_at_once():
    """The generated-Session cache is shared by the ranks of one job: nobody may read a header, weight file or
    shared object that another process is still writing, and the model is emitted and compiled once."""
    import multiprocessing as mp
    import shutil
    for old in generated.WORK.glob("race_c2_b6_*"):
        shutil.rmtree(old)
    generated.build_generator()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_emit_and_compile_worker, args=(i, out)) for i in range(8)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert all(r[2] for r in results), results
    assert len({r[1] for r in results}) == 1                      # one cache entry serves all eight
    assert len(list(generated.WORK.glob("race_c2_b6_*"))) == 1    # and no temporary directory is left behind
    assert not list(generated.WORK.glob(".race_c2_b6_*.*/"))


def test_run_time_batch_parameter_keeps_the_reference_signatures():
    """Generate() without a batch size on a model whose input has a batch parameter: the emitted Session takes the
    parameter in its constructor (the largest batch, which sizes the arena) and in infer() (reference: RModel.cxx:680-713,
    876-884); every number that scales with the batch is written in terms of it."""
    m, _ = configs.cnn_f32(batch=4, with_input=False)
    text = generated.emit(onnx_wire.model_to_onnx(m, batch_param="bs"), "c2_dynamic").read_text()
    assert re.search(r'Session\(std::string filename ="c2_dynamic.dat",\s+size_t bs = 1\)', text)
    assert "std::vector<float> infer(size_t bs,float* tensor_x){" in text
    assert "1000003" not in text                                                    # no trace of the stand-in batch
    assert "const sofie_conv2d_desc d = {static_cast<int32_t>(1 * fBatch), 3, 32, 32, 16," in text
    assert "sofie_cuda_ctx_h2d(fCtx, dev_x, tensor_x, (size_t(12288) * fBatch))" in text
    assert "if (bs != fBatch) { fBatch = bs; fGraphReady = false; }" in text and "if (bs > fMaxBatch) throw" in text
    # slices scale with the batch and stay 256-byte aligned for every batch: one sample's bytes are rounded up
    slices = re.findall(r"sofie_cuda_ctx_arena\(fCtx, (?:\(size_t\((\d+)\) \* fBatch\)|0), \(size_t\((\d+)\) \* fBatch\)", text)
    assert len(slices) == 5 and all(int(o or 0) % 256 == 0 for o, _ in slices)
    assert "LaunchHead" not in text                                                 # the upload is never split: a part is not a whole number of samples
    generated.compile_session(generated.emit(onnx_wire.model_to_onnx(m, batch_param="bs"), "c2_dynamic"), "c2_dynamic")
    # with a batch size given, the same file generates the fixed-batch Session as before
    fixed = generated.emit(onnx_wire.model_to_onnx(m, batch_param="bs"), "c2_dynamic_fixed", batch=8).read_text()
    assert "std::vector<float> infer(float* tensor_x){" in fixed and "size_t bs = 8" in fixed and "fBatch" not in fixed
    assert "const sofie_conv2d_desc d = {8, 3, 32, 32, 16," in fixed


def test_conv1d_is_emitted_as_an_image_of_height_one():
    from helpers import conv1d_model_onnx
    g, _, _ = conv1d_model_onnx(batch=3, length=10)
    text = generated.emit(g, "conv1d_b3").read_text()
    descs = [[int(v) for v in d.split(",")] for d in re.findall(r"sofie_conv2d_desc d = \{([^}]*)\}", text)]
    # N, C, H, W, Cout, kH, kW, pad_h, pad_w, strides, dilations, group, layouts, packed, relu, pool
    assert descs[0] == [3, 2, 1, 10, 4, 1, 2, 0, 1, 1, 1, 1, 1, 1, 0, 0, 0, 1, 0]
    assert descs[1] == [3, 4, 1, 11, 8, 1, 3, 0, 1, 1, 1, 1, 1, 2, 0, 0, 0, 1, 0]     # kernel 2 with pad 1 lengthens the axis to 11
    assert "sofie_cuda_relu_f32(" not in text                                          # both Relus are fused
    with pytest.raises(RuntimeError, match="rank-3, rank-4 and rank-5"):               # a 4-D convolution has no operator
        w = np.zeros((2, 2, 3, 3, 3, 3), np.float32)
        generated.emit(onnx_wire.model("g", [onnx_wire.node("Conv", ["x", "w"], ["y"])], [onnx_wire.value_info("x", 1, [1, 2, 5, 5, 5, 5])],
                                       [onnx_wire.value_info("y", 1, [])], [onnx_wire.tensor("w", w)]), "conv4d_refused")


def test_stacked_matmul_is_one_batched_gemm_call():
    """MatMul of operands with the same leading dimensions: every stack index multiplies ITS matrices (the ONNX definition;
    the reference's emitted loop advances only the output offset, ROperator_Gemm.hxx:353-387)."""
    w = np.arange(2 * 3 * 5 * 4, dtype=np.float32).reshape(2, 3, 5, 4)
    act = onnx_wire.model("g", [onnx_wire.node("MatMul", ["a", "b"], ["y"])], [onnx_wire.value_info("a", 1, [2, 3, 7, 5]), onnx_wire.value_info("b", 1, [2, 3, 5, 4])],
                          [onnx_wire.value_info("y", 1, [])], [])
    text = generated.emit(act, "stacked_mm").read_text()
    assert "const sofie_gemm_f32_desc d = {7, 4, 5, 0, 0, 1.0f, 0.0f, 0, 0};" in text
    assert "sofie_cuda_gemm_f32_batched(fStream, &d, dev_a, dev_b, nullptr, dev_y, 6, 35, 20, 28)" in text
    const = onnx_wire.model("g", [onnx_wire.node("MatMul", ["a", "w"], ["y"])], [onnx_wire.value_info("a", 1, [2, 3, 7, 5])],
                            [onnx_wire.value_info("y", 1, [])], [onnx_wire.tensor("w", w)])
    text = generated.emit(const, "stacked_mm_const").read_text()
    # constant stacked weights are stored [N,K] per matrix, the layout the tensor-core GEMM takes
    assert "const sofie_gemm_f32_desc d = {7, 4, 5, 0, 1, 1.0f, 0.0f, 0, 0};" in text and "dev_w_nk_y" in text
    with pytest.raises(RuntimeError, match="same leading dimensions"):
        generated.emit(onnx_wire.model("g", [onnx_wire.node("MatMul", ["a", "b"], ["y"])], [onnx_wire.value_info("a", 1, [2, 7, 5]), onnx_wire.value_info("b", 1, [3, 5, 4])],
                                       [onnx_wire.value_info("y", 1, [])], []), "stacked_mm_bad")


def test_fp8_chain_with_run_time_scales_emits_the_dynamic_calls():
    m, x = configs.gemm_chain_fp8(rows=128, width=256, layers=3)
    text = generated.emit(onnx_wire.model_to_onnx(m, "dynamic"), "c4_dyn_emit", binary=True).read_text()
    assert text.count("sofie_cuda_dynamic_quantize_e4m3_f32(") == 1 and text.count("sofie_cuda_dynamic_quantize_e4m3_bf16(") == 2
    assert text.count("sofie_cuda_gemm_e4m3_dynamic(") == 3 and "sofie_cuda_gemm_e4m3(" not in text
    # the scale is a device tensor handed from the quantiser to the product; the last product writes the floats itself
    assert "sofie_cuda_gemm_e4m3_dynamic(fStream, &d, dev_x_q, dev_x_scale, dev_W0_e4m3, dev_b0, dev_y0_bf16, nullptr)" in text
    assert re.search(r"sofie_cuda_gemm_e4m3_dynamic\(fStream, &d, dev_y1_q, dev_y1_scale, dev_W2_e4m3, dev_b2, nullptr, dev_y2\)", text)


def test_sharded_helper_compiles_against_a_run_time_batch_session():
    from helpers import build_sharded_program
    m, _ = configs.cnn_i8(batch=8, with_input=False)
    exe, dat = build_sharded_program(m, "c5_sharded")
    assert exe.exists() and dat.exists()


def test_volume_operators_emit_3d_calls():
    """Rank-5 tensors: Conv (+ fused Relu) and MaxPool emit the 3-D entry points; nothing is folded into a 2-D call."""
    m, _ = configs.volume_f32(batch=2)
    text = _emit(m, "volume_b2").read_text()
    assert text.count("sofie_cuda_conv3d_f32(") == 2 and text.count("sofie_cuda_pool3d_f32(") == 1
    assert "sofie_cuda_conv2d_f32(" not in text and "sofie_cuda_relu_f32(" not in text
    descs = re.findall(r"sofie_conv3d_desc d = \{([^}]*)\}", text)
    assert [int(v) for v in descs[0].split(",")] == [2, 2, 6, 8, 10, 8, 3, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1]
    assert [int(v) for v in descs[1].split(",")] == [2, 8, 3, 4, 5, 4, 2, 3, 1, 0, 0, 0, 1, 2, 1, 1, 1, 1, 2, 0]
    pool = re.search(r"sofie_pool3d_desc d = \{([^;]*)\};", text).group(1)
    assert [int(v) for v in re.findall(r"-?\d+", pool)] == [0, 2, 8, 6, 8, 10, 2, 2, 2, 2, 2, 2, 0, 0, 0, 0, 0, 0, 0]
    generated.compile_session(_emit(m, "volume_b2"), "volume_b2")
