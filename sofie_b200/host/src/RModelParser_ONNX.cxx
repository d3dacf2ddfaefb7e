// ONNX -> RModel. Same flow as the reference's front end (src/SOFIE_parsers/src/RModelParser_ONNX.cxx:
// Parse :344-375, ParseONNXGraph :454-755, ParseOperator :279-341): register inputs, read
// initialisers, order the nodes topologically, build one ROperator per node (MatMul followed by an
// Add of a constant becomes a Gemm, as ParseFuseMatMulAdd.cxx does), name the outputs. Relu / MaxPool
// fusion into the contraction epilogues is not done here but in the model's device plan.
#include "SOFIE/RModelParser_ONNX.hxx"

#include <algorithm>
#include <ctime>
#include <fstream>
#include <iostream>
#include <sstream>

#include "SOFIE/ROperator_BasicBinary.hxx"
#include "SOFIE/ROperator_BasicUnary.hxx"
#include "SOFIE/ROperator_BatchNormalization.hxx"
#include "SOFIE/ROperator_Conv.hxx"
#include "SOFIE/ROperator_Fp8.hxx"
#include "SOFIE/ROperator_Gemm.hxx"
#include "SOFIE/ROperator_Identity.hxx"
#include "SOFIE/ROperator_ConvTranspose.hxx"
#include "SOFIE/ROperator_Einsum.hxx"
#include "SOFIE/ROperator_Pool.hxx"
#include "SOFIE/ROperator_QLinear.hxx"
#include "SOFIE/ROperator_Relu.hxx"
#include "SOFIE/ROperator_Reshape.hxx"
#include "SOFIE/ROperator_Softmax.hxx"

namespace SOFIE {

namespace {

std::vector<size_t> attr_ints(const onnx::NodeProto &n, const std::string &name)
{
   std::vector<size_t> out;
   if (auto *a = n.find_attribute(name))
      for (auto v : a->ints()) out.push_back((size_t)v);
   return out;
}
int64_t attr_int(const onnx::NodeProto &n, const std::string &name, int64_t def)
{
   auto *a = n.find_attribute(name);
   return a ? a->i() : def;
}
float attr_float(const onnx::NodeProto &n, const std::string &name, float def)
{
   auto *a = n.find_attribute(name);
   return a ? a->f() : def;
}
std::string attr_string(const onnx::NodeProto &n, const std::string &name, const std::string &def)
{
   auto *a = n.find_attribute(name);
   return a ? a->s() : def;
}
void require_type(RModelParser_ONNX &p, const std::string &tensor, const std::string &op)
{
   if (!p.IsRegisteredTensorType(tensor))
      throw std::runtime_error("SOFIE ONNX Parser " + op + " op has input tensor " + tensor + " but its type is not yet registered");
}

std::unique_ptr<ROperator> ParseGemm(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "Gemm");
   ETensorType type = p.GetTensorType(n.input(0));
   if (type != ETensorType::FLOAT)
      throw std::runtime_error("SOFIE - Unsupported - Operator Gemm does not yet support input type " + std::to_string((int)type));
   float alpha = attr_float(n, "alpha", 1.f), beta = attr_float(n, "beta", 1.f);
   int_t transA = attr_int(n, "transA", 0), transB = attr_int(n, "transB", 0);
   std::unique_ptr<ROperator> op;
   if (n.input_size() == 2)
      op.reset(new ROperator_Gemm<float>(alpha, beta, transA, transB, n.input(0), n.input(1), n.output(0)));
   else
      op.reset(new ROperator_Gemm<float>(alpha, beta, transA, transB, n.input(0), n.input(1), n.input(2), n.output(0)));
   p.RegisterTensorType(n.output(0), type);
   return op;
}

std::unique_ptr<ROperator> ParseMatMul(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "MatMul");
   ETensorType type = p.GetTensorType(n.input(0));
   if (type != ETensorType::FLOAT) throw std::runtime_error("SOFIE - Unsupported - Operator MatMul does not yet support this input type");
   p.RegisterTensorType(n.output(0), type);
   return std::unique_ptr<ROperator>(new ROperator_Gemm<float>(1.f, 0.f, 0, 0, n.input(0), n.input(1), n.output(0)));
}

std::unique_ptr<ROperator> ParseEinsum(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   std::string eq = attr_string(n, "equation", "");
   eq.erase(std::remove(eq.begin(), eq.end(), ' '), eq.end());
   if (eq == "ik,kj->ij" && n.input_size() == 2) return ParseMatMul(p, n); // a plain matrix product: the GEMM kernels
   if (n.input_size() != 2) throw std::runtime_error("SOFIE - Einsum with " + std::to_string(n.input_size()) + " operands is not generated for the CUDA path");
   require_type(p, n.input(0), "Einsum");
   if (p.GetTensorType(n.input(0)) != ETensorType::FLOAT) throw std::runtime_error("SOFIE - Unsupported - Operator Einsum does not yet support this input type");
   p.RegisterTensorType(n.output(0), ETensorType::FLOAT);
   return std::unique_ptr<ROperator>(new ROperator_Einsum<float>(eq, {n.input(0), n.input(1)}, n.output(0)));
}

std::unique_ptr<ROperator> ParseConv(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "Conv");
   ETensorType type = p.GetTensorType(n.input(0));
   if (type != ETensorType::FLOAT) throw std::runtime_error("SOFIE - Unsupported - Operator Conv does not yet support this input type");
   std::string bias = n.input_size() > 2 ? n.input(2) : "";
   p.RegisterTensorType(n.output(0), type);
   return std::unique_ptr<ROperator>(new ROperator_Conv<float>(attr_string(n, "auto_pad", "NOTSET"), attr_ints(n, "dilations"),
                                                               (size_t)attr_int(n, "group", 1), attr_ints(n, "kernel_shape"),
                                                               attr_ints(n, "pads"), attr_ints(n, "strides"), n.input(0), n.input(1),
                                                               bias, n.output(0)));
}

std::unique_ptr<ROperator> ParseConvTranspose(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "ConvTranspose");
   ETensorType type = p.GetTensorType(n.input(0));
   if (type != ETensorType::FLOAT)
      throw std::runtime_error("SOFIE - Unsupported - Operator ConvTranspose does not yet support this input type");
   std::string bias = n.input_size() > 2 ? n.input(2) : "";
   p.RegisterTensorType(n.output(0), type);
   return std::unique_ptr<ROperator>(new ROperator_ConvTranspose<float>(
      attr_string(n, "auto_pad", "NOTSET"), attr_ints(n, "dilations"), (size_t)attr_int(n, "group", 1), attr_ints(n, "kernel_shape"),
      attr_ints(n, "output_padding"), attr_ints(n, "output_shape"), attr_ints(n, "pads"), attr_ints(n, "strides"), n.input(0), n.input(1),
      bias, n.output(0)));
}

std::unique_ptr<ROperator> ParseRelu(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "Relu");
   p.RegisterTensorType(n.output(0), p.GetTensorType(n.input(0)));
   return std::unique_ptr<ROperator>(new ROperator_Relu<float>(n.input(0), n.output(0)));
}

std::unique_ptr<ROperator> ParsePool(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), n.op_type());
   PoolOpMode mode = n.op_type() == "MaxPool" ? MaxPool : (n.op_type() == "AveragePool" ? AveragePool : GlobalAveragePool);
   RAttributes_Pool attr;
   attr.auto_pad = attr_string(n, "auto_pad", "NOTSET");
   attr.ceil_mode = (int)attr_int(n, "ceil_mode", 0);
   attr.count_include_pad = (int)attr_int(n, "count_include_pad", 0);
   attr.storage_order = (int)attr_int(n, "storage_order", 0);
   attr.dilations = attr_ints(n, "dilations");
   attr.kernel_shape = attr_ints(n, "kernel_shape");
   attr.pads = attr_ints(n, "pads");
   attr.strides = attr_ints(n, "strides");
   if (attr.ceil_mode) throw std::runtime_error("SOFIE - Pool with ceil_mode is not supported");
   p.RegisterTensorType(n.output(0), p.GetTensorType(n.input(0)));
   return std::unique_ptr<ROperator>(new ROperator_Pool<float>(mode, attr, n.input(0), n.output(0)));
}

std::unique_ptr<ROperator> ParseReshape(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), n.op_type());
   p.RegisterTensorType(n.output(0), p.GetTensorType(n.input(0)));
   const std::string &t = n.op_type();
   if (t == "Flatten")
      return std::unique_ptr<ROperator>(new ROperator_Reshape(Flatten, (int)attr_int(n, "axis", 1), n.input(0), "", n.output(0)));
   if (t == "Reshape")
      return std::unique_ptr<ROperator>(new ROperator_Reshape(Reshape, (int)attr_int(n, "allowzero", 0), n.input(0), n.input(1), n.output(0)));
   ReshapeOpMode mode = t == "Squeeze" ? Squeeze : Unsqueeze;
   if (n.input_size() > 1) return std::unique_ptr<ROperator>(new ROperator_Reshape(mode, 0, n.input(0), n.input(1), n.output(0)));
   std::vector<int64_t> axes;
   if (auto *a = n.find_attribute("axes")) axes = a->ints();
   return std::unique_ptr<ROperator>(new ROperator_Reshape(mode, axes, n.input(0), n.output(0)));
}

std::unique_ptr<ROperator> ParseSoftmax(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "Softmax");
   p.RegisterTensorType(n.output(0), p.GetTensorType(n.input(0)));
   return std::unique_ptr<ROperator>(new ROperator_Softmax<float>(attr_int(n, "axis", -1), n.input(0), n.output(0)));
}

// Elementwise family (reference: ParseSigmoid.cxx, ParseTanh.cxx, ParseLeakyRelu.cxx, ParseSelu.cxx, ParseElu.cxx,
// ParseBasicUnary.cxx, ParseBasicBinary.cxx, ParseBatchNormalization.cxx): float only, output type = input type.
template <typename Make>
std::unique_ptr<ROperator> ParseUnaryWith(RModelParser_ONNX &p, const onnx::NodeProto &n, Make make)
{
   require_type(p, n.input(0), n.op_type());
   if (p.GetTensorType(n.input(0)) != ETensorType::FLOAT)
      throw std::runtime_error("SOFIE - Unsupported - Operator " + n.op_type() + " does not yet support this input type");
   p.RegisterTensorType(n.output(0), ETensorType::FLOAT);
   return std::unique_ptr<ROperator>(make());
}
std::unique_ptr<ROperator> ParseSigmoid(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_Sigmoid<float>(n.input(0), n.output(0)); });
}
std::unique_ptr<ROperator> ParseTanh(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_Tanh<float>(n.input(0), n.output(0)); });
}
std::unique_ptr<ROperator> ParseSelu(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_Selu<float>(n.input(0), n.output(0)); });
}
std::unique_ptr<ROperator> ParseLeakyRelu(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_LeakyRelu<float>(attr_float(n, "alpha", 0.01f), n.input(0), n.output(0)); });
}
std::unique_ptr<ROperator> ParseElu(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_Elu<float>(attr_float(n, "alpha", 1.f), n.input(0), n.output(0)); });
}
template <EBasicUnaryOperator Op>
std::unique_ptr<ROperator> ParseBasicUnary(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_BasicUnary<float, Op>(n.input(0), n.output(0)); });
}
std::unique_ptr<ROperator> ParseErf(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_Erf<float>(n.input(0), n.output(0)); });
}
std::unique_ptr<ROperator> ParseSwish(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   return ParseUnaryWith(p, n, [&] { return new ROperator_Swish<float>(n.input(0), n.output(0)); });
}
// Identity of a run-time tensor (reference: ParseIdentity.cxx:7-35, float only there; any type here since nothing is
// computed). An Identity of a constant is resolved in ParseONNXGraph and never gets here.
std::unique_ptr<ROperator> ParseIdentity(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), n.op_type());
   p.RegisterTensorType(n.output(0), p.GetTensorType(n.input(0)));
   return std::unique_ptr<ROperator>(new ROperator_Identity<float>(n.input(0), n.output(0)));
}
// Constant nodes become initialised tensors in ParseONNXGraph (the reference keeps an operator that copies the values
// into the output at Session construction, ParseConstant.cxx:9-175 / ROperator_Constant.hxx); nothing is left to emit.
std::unique_ptr<ROperator> ParseConstant(RModelParser_ONNX &, const onnx::NodeProto &n)
{
   throw std::runtime_error("SOFIE - Constant node " + n.output(0) + " reached the operator stage");
}
template <EBasicBinaryOperator Op>
std::unique_ptr<ROperator> ParseBasicBinary(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   if (n.input_size() != 2) throw std::runtime_error("SOFIE - binary operator " + n.op_type() + " needs two inputs");
   for (int i = 0; i < 2; i++) {
      require_type(p, n.input(i), n.op_type());
      if (p.GetTensorType(n.input(i)) != ETensorType::FLOAT)
         throw std::runtime_error("SOFIE - Unsupported - Operator " + n.op_type() + " does not yet support this input type");
   }
   p.RegisterTensorType(n.output(0), ETensorType::FLOAT);
   return std::unique_ptr<ROperator>(new ROperator_BasicBinary<float, Op>(n.input(0), n.input(1), n.output(0)));
}
std::unique_ptr<ROperator> ParseBatchNormalization(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "BatchNormalization");
   if (p.GetTensorType(n.input(0)) != ETensorType::FLOAT)
      throw std::runtime_error("SOFIE - Unsupported - Operator BatchNormalization does not yet support this input type");
   if (n.input_size() != 5) throw std::runtime_error("SOFIE - BatchNormalization needs X, scale, B, mean and var");
   p.RegisterTensorType(n.output(0), ETensorType::FLOAT);
   return std::unique_ptr<ROperator>(new ROperator_BatchNormalization<float>(attr_float(n, "epsilon", 1e-5f), attr_float(n, "momentum", 0.9f),
                                                                             (size_t)attr_int(n, "training_mode", 0), n.input(0), n.input(1),
                                                                             n.input(2), n.input(3), n.input(4), n.output(0)));
}

std::unique_ptr<ROperator> ParseQuantizeLinear(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "QuantizeLinear");
   if (n.input_size() < 3) throw std::runtime_error("SOFIE - QuantizeLinear needs x, y_scale and y_zero_point (uint8 output)");
   // the type of the zero point selects the output type (ONNX QuantizeLinear, opset 19)
   if (p.IsRegisteredTensorType(n.input(2)) && p.GetTensorType(n.input(2)) == ETensorType::FLOAT8E4M3FN) {
      p.RegisterTensorType(n.output(0), ETensorType::FLOAT8E4M3FN);
      return std::unique_ptr<ROperator>(new ROperator_QuantizeE4M3(n.input(0), n.input(1), n.output(0)));
   }
   p.RegisterTensorType(n.output(0), ETensorType::UINT8);
   return std::unique_ptr<ROperator>(new ROperator_QuantizeLinear(n.input(0), n.input(1), n.input(2), n.output(0)));
}

std::unique_ptr<ROperator> ParseCast(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "Cast");
   ETensorType to = static_cast<ETensorType>(attr_int(n, "to", 1));
   p.RegisterTensorType(n.output(0), to);
   return std::unique_ptr<ROperator>(new ROperator_Cast(to, n.input(0), n.output(0)));
}

// Custom operator of the FP8 chain (see ROperator_Fp8.hxx): inputs A (E4M3), W (E4M3 constant [N, K]), optional bias;
// attributes a_scale, w_scale, out_scale (0: bfloat16 output), relu.
std::unique_ptr<ROperator> ParseFp8Gemm(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "Fp8Gemm");
   if (n.input_size() < 2) throw std::runtime_error("SOFIE - Fp8Gemm needs A and W");
   float out_scale = attr_float(n, "out_scale", 0.f);
   p.RegisterTensorType(n.output(0), out_scale > 0.f ? ETensorType::FLOAT8E4M3FN : ETensorType::BFLOAT16);
   // optional fourth input: the activation scale as a run-time tensor (second output of DynamicQuantizeE4M3)
   return std::unique_ptr<ROperator>(new ROperator_Fp8Gemm(attr_float(n, "a_scale", 1.f), attr_float(n, "w_scale", 1.f), out_scale,
                                                           attr_int(n, "relu", 0) != 0, n.input(0), n.input(1),
                                                           n.input_size() > 2 ? n.input(2) : "", n.output(0), n.input_size() > 3 ? n.input(3) : ""));
}

std::unique_ptr<ROperator> ParseDynamicQuantizeE4M3(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "DynamicQuantizeE4M3");
   if (n.output_size() != 2) throw std::runtime_error("SOFIE - DynamicQuantizeE4M3 has two outputs: the E4M3 tensor and its scale");
   p.RegisterTensorType(n.output(0), ETensorType::FLOAT8E4M3FN);
   p.RegisterTensorType(n.output(1), ETensorType::FLOAT);
   return std::unique_ptr<ROperator>(new ROperator_DynamicQuantizeE4M3(n.input(0), n.output(0), n.output(1)));
}

std::unique_ptr<ROperator> ParseDequantizeLinear(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "DequantizeLinear");
   p.RegisterTensorType(n.output(0), ETensorType::FLOAT);
   return std::unique_ptr<ROperator>(new ROperator_DequantizeLinear(n.input(0), n.input(1), n.input_size() > 2 ? n.input(2) : "", n.output(0)));
}

std::unique_ptr<ROperator> ParseQLinearMatMul(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "QLinearMatMul");
   if (n.input_size() != 8) throw std::runtime_error("SOFIE - QLinearMatMul needs 8 inputs");
   p.RegisterTensorType(n.output(0), ETensorType::UINT8);
   return std::unique_ptr<ROperator>(new ROperator_QLinearMatMul(n.input(0), n.input(1), n.input(2), n.input(3), n.input(4), n.input(5),
                                                                 n.input(6), n.input(7), n.output(0)));
}

std::unique_ptr<ROperator> ParseQLinearConv(RModelParser_ONNX &p, const onnx::NodeProto &n)
{
   require_type(p, n.input(0), "QLinearConv");
   if (n.input_size() < 8) throw std::runtime_error("SOFIE - QLinearConv needs at least 8 inputs");
   p.RegisterTensorType(n.output(0), ETensorType::UINT8);
   return std::unique_ptr<ROperator>(new ROperator_QLinearConv(
      attr_string(n, "auto_pad", "NOTSET"), attr_ints(n, "dilations"), (size_t)attr_int(n, "group", 1), attr_ints(n, "kernel_shape"),
      attr_ints(n, "pads"), attr_ints(n, "strides"), n.input(0), n.input(1), n.input(2), n.input(3), n.input(4), n.input(5), n.input(6),
      n.input(7), n.input_size() > 8 ? n.input(8) : "", n.output(0)));
}

template <typename T> std::shared_ptr<void> tensor_data(const onnx::TensorProto &t, size_t length)
{
   std::shared_ptr<void> data(malloc(length * sizeof(T) + 1), free);
   T *dst = static_cast<T *>(data.get());
   if (t.has_raw_data()) {
      if (t.raw_data().size() != length * sizeof(T))
         throw std::runtime_error("SOFIE ONNX Parser: raw_data of tensor " + t.name() + " has the wrong size");
      std::memcpy(dst, t.raw_data().data(), length * sizeof(T)); // ONNX raw data is little-endian, as is this machine
   } else if (std::is_same<T, float>::value) {
      if ((size_t)t.float_data_size() != length) throw std::runtime_error("SOFIE ONNX Parser: float_data of tensor " + t.name() + " has the wrong size");
      for (size_t i = 0; i < length; i++) dst[i] = (T)t.float_data((int)i);
   } else if (std::is_same<T, int64_t>::value) {
      if ((size_t)t.int64_data_size() != length) throw std::runtime_error("SOFIE ONNX Parser: int64_data of tensor " + t.name() + " has the wrong size");
      for (size_t i = 0; i < length; i++) dst[i] = (T)t.int64_data((int)i);
   } else {
      if ((size_t)t.int32_data_size() != length) throw std::runtime_error("SOFIE ONNX Parser: int32_data of tensor " + t.name() + " has the wrong size");
      for (size_t i = 0; i < length; i++) dst[i] = (T)t.int32_data((int)i);
   }
   return data;
}

} // namespace

// ---------------------------------------------------------------------------------- registration
RModelParser_ONNX::RModelParser_ONNX() noexcept : fOperatorsMapImpl(std::make_unique<OperatorsMapImpl>())
{
   RegisterOperator("Gemm", ParseGemm);
   RegisterOperator("MatMul", ParseMatMul);
   RegisterOperator("Einsum", ParseEinsum);
   RegisterOperator("Conv", ParseConv);
   RegisterOperator("ConvTranspose", ParseConvTranspose);
   RegisterOperator("Relu", ParseRelu);
   RegisterOperator("MaxPool", ParsePool);
   RegisterOperator("AveragePool", ParsePool);
   RegisterOperator("GlobalAveragePool", ParsePool);
   RegisterOperator("Reshape", ParseReshape);
   RegisterOperator("Flatten", ParseReshape);
   RegisterOperator("Squeeze", ParseReshape);
   RegisterOperator("Unsqueeze", ParseReshape);
   RegisterOperator("Softmax", ParseSoftmax);
   RegisterOperator("Sigmoid", ParseSigmoid);
   RegisterOperator("Tanh", ParseTanh);
   RegisterOperator("Selu", ParseSelu);
   RegisterOperator("LeakyRelu", ParseLeakyRelu);
   RegisterOperator("Elu", ParseElu);
   RegisterOperator("Neg", ParseBasicUnary<EBasicUnaryOperator::kNeg>);
   RegisterOperator("Exp", ParseBasicUnary<EBasicUnaryOperator::kExp>);
   RegisterOperator("Log", ParseBasicUnary<EBasicUnaryOperator::kLog>);
   RegisterOperator("Sqrt", ParseBasicUnary<EBasicUnaryOperator::kSqrt>);
   RegisterOperator("Reciprocal", ParseBasicUnary<EBasicUnaryOperator::kReciprocal>);
   RegisterOperator("Abs", ParseBasicUnary<EBasicUnaryOperator::kAbs>);
   RegisterOperator("Cos", ParseBasicUnary<EBasicUnaryOperator::kCos>);
   RegisterOperator("Sin", ParseBasicUnary<EBasicUnaryOperator::kSin>);
   RegisterOperator("Erf", ParseErf);
   RegisterOperator("Swish", ParseSwish);
   RegisterOperator("Identity", ParseIdentity);
   RegisterOperator("Constant", ParseConstant);
   RegisterOperator("Add", ParseBasicBinary<Add>);
   RegisterOperator("Sub", ParseBasicBinary<Sub>);
   RegisterOperator("Mul", ParseBasicBinary<Mul>);
   RegisterOperator("Div", ParseBasicBinary<Div>);
   RegisterOperator("BatchNormalization", ParseBatchNormalization);
   RegisterOperator("Cast", ParseCast);
   RegisterOperator("Fp8Gemm", ParseFp8Gemm);
   RegisterOperator("DynamicQuantizeE4M3", ParseDynamicQuantizeE4M3);
   RegisterOperator("QuantizeLinear", ParseQuantizeLinear);
   RegisterOperator("DequantizeLinear", ParseDequantizeLinear);
   RegisterOperator("QLinearMatMul", ParseQLinearMatMul);
   RegisterOperator("QLinearConv", ParseQLinearConv);
}

RModelParser_ONNX::~RModelParser_ONNX() = default;

void RModelParser_ONNX::RegisterOperator(const std::string &name, ParserFuncSignature func) { fOperatorsMapImpl->fOperatorsMap[name] = func; }
bool RModelParser_ONNX::IsRegisteredOperator(const std::string &name) { return fOperatorsMapImpl->fOperatorsMap.count(name); }
std::vector<std::string> RModelParser_ONNX::GetRegisteredOperators()
{
   std::vector<std::string> ops;
   for (auto &it : fOperatorsMapImpl->fOperatorsMap) ops.push_back(it.first);
   std::sort(ops.begin(), ops.end());
   return ops;
}
void RModelParser_ONNX::RegisterTensorType(const std::string &name, ETensorType type) { fTensorTypeMap[UTILITY::Clean_name(name)] = type; }
bool RModelParser_ONNX::IsRegisteredTensorType(const std::string &name) { return fTensorTypeMap.count(UTILITY::Clean_name(name)); }
ETensorType RModelParser_ONNX::GetTensorType(const std::string &name) { return fTensorTypeMap[UTILITY::Clean_name(name)]; }

// ---------------------------------------------------------------------------------- operators
std::unique_ptr<ROperator> RModelParser_ONNX::ParseOperator(const size_t i, const onnx::GraphProto &g, const std::vector<size_t> &nodes,
                                                            const std::vector<int> &children)
{
   if (i >= nodes.size()) throw std::runtime_error("SOFIE - Error in parsing ordered operators " + std::to_string(i));
   const onnx::NodeProto &node = g.node((int)nodes[i]);
   const std::string &type = node.op_type();
   if (fVerbose) std::cout << "Parsing operator " << type << std::endl;
   // MatMul whose only reader is an Add of a constant: one Gemm with bias (reference: ParseFuseMatMulAdd.cxx:8-57)
   if (type == "MatMul" && children.size() == 1) {
      const onnx::NodeProto &child = g.node((int)nodes[children[0]]);
      if (child.op_type() == "Add" && child.input_size() == 2) {
         std::string bias = child.input(0) == node.output(0) ? child.input(1) : child.input(0);
         bool bias_is_constant = false;
         for (int k = 0; k < g.initializer_size(); k++) bias_is_constant |= g.initializer(k).name() == bias;
         if (bias_is_constant && IsRegisteredTensorType(node.input(0)) && GetTensorType(node.input(0)) == ETensorType::FLOAT) {
            fFusedOperators[children[0]] = true;
            RegisterTensorType(child.output(0), ETensorType::FLOAT);
            return std::unique_ptr<ROperator>(new ROperator_Gemm<float>(1.f, 1.f, 0, 0, node.input(0), node.input(1), bias, child.output(0)));
         }
      }
   }
   // BatchNormalization whose only reader is a Relu: one operator with the activation fused
   // (reference: ParseFuseBatchnormRelu.cxx, RModelParser_ONNX.cxx:322-330)
   if (type == "BatchNormalization" && children.size() == 1 && node.input_size() == 5) {
      const onnx::NodeProto &child = g.node((int)nodes[children[0]]);
      if (child.op_type() == "Relu" && IsRegisteredTensorType(node.input(0)) && GetTensorType(node.input(0)) == ETensorType::FLOAT) {
         fFusedOperators[children[0]] = true;
         RegisterTensorType(child.output(0), ETensorType::FLOAT);
         return std::unique_ptr<ROperator>(new ROperator_BatchNormalization<float>(
            attr_float(node, "epsilon", 1e-5f), attr_float(node, "momentum", 0.9f), (size_t)attr_int(node, "training_mode", 0), node.input(0),
            node.input(1), node.input(2), node.input(3), node.input(4), child.output(0), EActivationType::RELU));
      }
   }
   auto it = fOperatorsMapImpl->fOperatorsMap.find(type);
   if (it == fOperatorsMapImpl->fOperatorsMap.end())
      throw std::runtime_error("SOFIE Operator type " + type + " is not yet supported on the CUDA dense-contraction path");
   return it->second(*this, node);
}

std::unique_ptr<onnx::ModelProto> RModelParser_ONNX::LoadModel(std::string filename)
{
   std::ifstream in(filename, std::ios::binary);
   if (!in.is_open()) throw std::runtime_error("SOFIE - Failed to open onnx file " + filename);
   std::stringstream ss;
   ss << in.rdbuf();
   auto model = std::make_unique<onnx::ModelProto>();
   model->ParseFromString(ss.str());
   return model;
}

void RModelParser_ONNX::CheckGraph(const onnx::GraphProto &g, int &level, std::map<std::string, int> &missingOperators)
{
   (void)level;
   for (int i = 0; i < g.node_size(); i++) {
      const std::string &t = g.node(i).op_type();
      if (!IsRegisteredOperator(t)) missingOperators[t]++;
   }
}

bool RModelParser_ONNX::CheckModel(std::string filename, bool verbose)
{
   fVerbose = verbose;
   auto model = LoadModel(filename);
   std::map<std::string, int> missing;
   int level = 1;
   CheckGraph(model->graph(), level, missing);
   if (!missing.empty()) {
      std::cout << "List of missing operators for model loaded from file " << filename << std::endl;
      for (auto &op : missing) std::cout << op.first << "  " << op.second << std::endl;
      return false;
   }
   if (verbose) std::cout << "All operators in the loaded model are supported!\n";
   return true;
}

RModel RModelParser_ONNX::Parse(std::string filename, bool verbose)
{
   fVerbose = verbose;
   fTensorTypeMap.clear();
   auto model = LoadModel(filename);
   std::string filename_nodir = filename;
   auto slash = filename.find_last_of("/\\");
   if (slash != std::string::npos) filename_nodir = filename.substr(slash + 1);
   std::time_t ttime = std::time(0);
   std::tm *gmt_time = std::gmtime(&ttime);
   std::string parsetime(std::asctime(gmt_time));
   RModel rmodel(filename_nodir, parsetime);
   ParseONNXGraph(rmodel, model->graph());
   return rmodel;
}

void RModelParser_ONNX::ParseONNXGraph(RModel &rmodel, const onnx::GraphProto &graph, std::string graphName)
{
   (void)graphName;
   std::unordered_map<std::string, bool> initializer_names;
   for (int i = 0; i < graph.initializer_size(); i++) initializer_names[graph.initializer(i).name()] = true;

   // ---- inputs: graph inputs that are not initialisers
   for (int i = 0; i < graph.input_size(); i++) {
      const auto &vi = graph.input(i);
      if (initializer_names.count(vi.name())) continue;
      ETensorType type = static_cast<ETensorType>(vi.fElemType);
      if (type != ETensorType::FLOAT && type != ETensorType::UINT8 && type != ETensorType::INT32 && type != ETensorType::INT64)
         throw std::runtime_error("SOFIE Data type in input tensor " + vi.name() + " not supported!");
      RegisterTensorType(vi.name(), type);
      if (!vi.fHasShape) throw std::runtime_error("SOFIE data node with no shape restrictions is not supported yet");
      std::vector<Dim> shape;
      bool parametric = false;
      for (auto &d : vi.fDims) {
         if (d.fHasValue && d.fValue > 0) shape.emplace_back((size_t)d.fValue);
         else {
            parametric = true;
            shape.emplace_back(d.fParam.empty() ? std::string("bs") : UTILITY::Clean_name(d.fParam), 0);
         }
      }
      if (parametric) rmodel.AddInputTensorInfo(vi.name(), type, shape);
      else rmodel.AddInputTensorInfo(vi.name(), type, ConvertShapeToInt(shape));
      rmodel.AddInputTensorName(vi.name());
   }

   // ---- initialisers (the reference accepts FLOAT / DOUBLE / INT32 / INT64 only,
   //      RModelParser_ONNX.cxx:560-591; UINT8 and INT8 are needed by the quantised operators)
   auto add_constant = [&](const onnx::TensorProto &t, const std::string &name) {
      std::vector<size_t> shape;
      size_t length = 1;
      for (int j = 0; j < t.dims_size(); j++) {
         shape.push_back((size_t)t.dims(j));
         length *= (size_t)t.dims(j);
      }
      if (t.dims_size() == 0) shape = {1}; // scalar
      ETensorType type = static_cast<ETensorType>(t.data_type());
      RegisterTensorType(name, type);
      std::shared_ptr<void> data;
      switch (type) {
      case ETensorType::FLOAT: data = tensor_data<float>(t, length); break;
      case ETensorType::DOUBLE: data = tensor_data<double>(t, length); break;
      case ETensorType::INT32: data = tensor_data<int32_t>(t, length); break;
      case ETensorType::INT64: data = tensor_data<int64_t>(t, length); break;
      case ETensorType::UINT8: data = tensor_data<uint8_t>(t, length); break;
      case ETensorType::INT8: data = tensor_data<int8_t>(t, length); break;
      case ETensorType::FLOAT8E4M3FN: data = tensor_data<uint8_t>(t, length); break; // raw bit patterns
      default: throw std::runtime_error("SOFIE Data type in weight tensor " + name + " not supported!\n");
      }
      rmodel.AddInitializedTensor(name, type, shape, data);
   };
   for (int i = 0; i < graph.initializer_size(); i++) add_constant(graph.initializer(i), graph.initializer(i).name());

   // ---- Constant nodes, and Identity nodes of constants, are initialised tensors under another spelling
   //      (reference: ParseConstant.cxx:46-165 reads the same attributes; exporters write the shape of a Reshape
   //      and shared weights this way). They produce no operator.
   std::vector<bool> folded(graph.node_size(), false);
   for (bool again = true; again;) {
      again = false;
      for (int i = 0; i < graph.node_size(); i++) {
         const auto &node = graph.node(i);
         if (folded[i] || node.output_size() != 1) continue;
         const std::string &out = node.output(0);
         if (node.op_type() == "Constant" && node.input_size() == 0) {
            if (node.attribute_size() != 1) throw std::runtime_error("SOFIE ONNX Parser Constant needs exactly one attribute");
            const auto &a = node.attribute(0);
            onnx::TensorProto t;
            if (a.name() == "value") t = a.t();
            else if (a.name() == "value_float") { t.fDataType = onnx::TensorProto::FLOAT; t.fDims = {1}; t.fFloatData = {a.f()}; }
            else if (a.name() == "value_floats") { t.fDataType = onnx::TensorProto::FLOAT; t.fDims = {(int64_t)a.fFloats.size()}; t.fFloatData = a.fFloats; }
            else if (a.name() == "value_int") { t.fDataType = onnx::TensorProto::INT64; t.fDims = {1}; t.fInt64Data = {a.i()}; }
            else if (a.name() == "value_ints") { t.fDataType = onnx::TensorProto::INT64; t.fDims = {(int64_t)a.fInts.size()}; t.fInt64Data = a.fInts; }
            else throw std::runtime_error("SOFIE ONNX Parser Constant op: not yet supporting attribute " + a.name());
            add_constant(t, out);
         } else if (node.op_type() == "Identity" && node.input_size() == 1 && initializer_names.count(node.input(0))) {
            const std::string src = UTILITY::Clean_name(node.input(0));
            const auto &t = rmodel.GetInitializedTensor(src);
            RegisterTensorType(out, t.type());
            rmodel.AddInitializedTensor(out, t.type(), t.shape(), t.sharedptr());
         } else {
            continue;
         }
         folded[i] = true;
         initializer_names[out] = true;
         again = true;
      }
   }

   // ---- execution order: a node is ready when all its inputs exist
   std::unordered_map<std::string, bool> available;
   for (auto &n : initializer_names) available[n.first] = true;
   for (int i = 0; i < graph.input_size(); i++) available[graph.input(i).name()] = true;
   std::vector<size_t> order;
   std::vector<bool> placed = folded;
   const size_t nLive = (size_t)std::count(folded.begin(), folded.end(), false);
   while (order.size() < nLive) {
      bool progress = false;
      for (int i = 0; i < graph.node_size(); i++) {
         if (placed[i]) continue;
         bool ready = true;
         for (int j = 0; j < graph.node(i).input_size(); j++) {
            const std::string &in = graph.node(i).input(j);
            if (!in.empty() && !available.count(in)) ready = false;
         }
         if (!ready) continue;
         placed[i] = true;
         progress = true;
         order.push_back(i);
         for (int j = 0; j < graph.node(i).output_size(); j++) available[graph.node(i).output(j)] = true;
      }
      if (!progress) throw std::runtime_error("SOFIE - cannot find a new node ready to be executed: the graph has a cycle or a missing input");
   }
   // children of every node, as indices into `order`
   std::vector<std::vector<int>> children(order.size());
   for (size_t a = 0; a < order.size(); a++)
      for (size_t b = a + 1; b < order.size(); b++) {
         bool reads = false;
         for (int j = 0; j < graph.node((int)order[b]).input_size(); j++)
            for (int k = 0; k < graph.node((int)order[a]).output_size(); k++)
               reads |= graph.node((int)order[b]).input(j) == graph.node((int)order[a]).output(k);
         if (reads) children[a].push_back((int)b);
      }

   fFusedOperators.assign(order.size(), false);
   for (size_t i = 0; i < order.size(); i++) {
      if (fFusedOperators[i]) continue;
      auto op = ParseOperator(i, graph, order, children[i]);
      if (!op) continue;
      rmodel.AddOperator(std::move(op));
   }

   std::vector<std::string> outputs;
   for (int i = 0; i < graph.output_size(); i++) outputs.push_back(graph.output(i).name());
   rmodel.AddOutputTensorNameList(outputs);
}

} // namespace SOFIE
