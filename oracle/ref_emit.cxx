// Test infrastructure (not part of the product): drives the UNMODIFIED reference generator.
//
// Builds a model through the reference's own RModel / ROperator_* classes (compiled from the
// reference sources where they lie, never copied) from a small text description, then calls the
// reference's Generate() and OutputGenerated(), which write <name>.hxx and <name>.dat -- the
// reference's emitted CPU inference code (copy-bias + sgemm_ + relu sweep, Im2col + sgemm_ +
// saxpy_, scalar pooling loops). Those emitted headers are what the CUDA path is checked against.
//
// Model description, one statement per line:
//   model   <name>
//   input   <tensor> <d0> <d1> ...
//   weight  <tensor> <d0> <d1> ...           (float32 values taken, in order, from the blob file)
//   gemm    <alpha> <beta> <transA> <transB> <A> <B> <C|-> <Y> <relu 0|1>
//   conv    <group> <kh> <kw> <pad_t> <pad_l> <pad_b> <pad_r> <sh> <sw> <dh> <dw> <X> <W> <B|-> <Y>
//   convtr  <kh> <kw> <pad_t> <pad_l> <pad_b> <pad_r> <sh> <sw> <oph> <opw> <X> <W> <B|-> <Y>
//   relu    <X> <Y>
//   maxpool <kh> <kw> <p0> <p1> <p2> <p3> <sh> <sw> <X> <Y>      (pads exactly as the ONNX attribute)
//   avgpool <kh> <kw> <p0> <p1> <p2> <p3> <sh> <sw> <X> <Y>
//   flatten <axis> <X> <Y>
//   softmax <axis> <X> <Y>
//   output  <Y>
//
// usage: ref_emit <description.txt> <weights.f32> <out_dir>
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator_Gemm.hxx"
#include "SOFIE/ROperator_Conv.hxx"
#include "SOFIE/ROperator_ConvTranspose.hxx"
#include "SOFIE/ROperator_Relu.hxx"
#include "SOFIE/ROperator_Pool.hxx"
#include "SOFIE/ROperator_Reshape.hxx"
#include "SOFIE/ROperator_Softmax.hxx"
#include "SOFIE/ROperator_Sigmoid.hxx"
#include "SOFIE/ROperator_Tanh.hxx"
#include "SOFIE/ROperator_LeakyRelu.hxx"
#include "SOFIE/ROperator_Selu.hxx"
#include "SOFIE/ROperator_Elu.hxx"
#include "SOFIE/ROperator_BasicBinary.hxx"
#include "SOFIE/ROperator_BatchNormalization.hxx"

#include <cstdio>
#include <fstream>
#include <iostream>
#include <sstream>

using namespace SOFIE;

int main(int argc, char **argv)
{
   if (argc != 4) {
      std::fprintf(stderr, "usage: %s <description.txt> <weights.f32> <out_dir>\n", argv[0]);
      return 2;
   }
   std::ifstream desc(argv[1]);
   std::ifstream blob(argv[2], std::ios::binary);
   std::string outDir = argv[3];
   if (!desc || !blob) {
      std::fprintf(stderr, "ref_emit: cannot open inputs\n");
      return 2;
   }
   std::unique_ptr<RModel> model;
   std::string name;
   std::vector<std::string> outputs;
   int order = 0;
   std::string line;
   try {
      while (std::getline(desc, line)) {
         std::istringstream ss(line);
         std::string kw;
         if (!(ss >> kw) || kw[0] == '#') continue;
         if (kw == "model") {
            ss >> name;
            model = std::make_unique<RModel>(name + ".onnx", "oracle ");
         } else if (kw == "input" || kw == "weight") {
            std::string t;
            ss >> t;
            std::vector<size_t> shape;
            size_t d;
            while (ss >> d) shape.push_back(d);
            if (kw == "input") {
               model->AddInputTensorInfo(t, ETensorType::FLOAT, shape);
               model->AddInputTensorName(t);
            } else {
               size_t len = ConvertShapeToLength(shape);
               std::vector<float> buf(len);
               blob.read(reinterpret_cast<char *>(buf.data()), len * sizeof(float));
               if (!blob) throw std::runtime_error("weight blob too short for " + t);
               model->AddInitializedTensor<float>(t, shape, buf.data());
            }
         } else if (kw == "gemm") {
            float alpha, beta;
            int tA, tB, relu;
            std::string A, B, C, Y;
            ss >> alpha >> beta >> tA >> tB >> A >> B >> C >> Y >> relu;
            auto act = relu ? EActivationType::RELU : EActivationType::UNDEFINED;
            if (C == "-")
               model->AddOperator(std::make_unique<ROperator_Gemm<float>>(alpha, beta, tA, tB, A, B, Y, act), order++);
            else
               model->AddOperator(std::make_unique<ROperator_Gemm<float>>(alpha, beta, tA, tB, A, B, C, Y, act), order++);
         } else if (kw == "conv") {
            size_t g, kh, kw_, pt, pl, pb, pr, sh, sw, dh, dw;
            std::string X, W, B, Y;
            ss >> g >> kh >> kw_ >> pt >> pl >> pb >> pr >> sh >> sw >> dh >> dw >> X >> W >> B >> Y;
            std::vector<size_t> dil{dh, dw}, ks{kh, kw_}, pads{pt, pl, pb, pr}, str{sh, sw};
            if (B == "-")
               model->AddOperator(std::make_unique<ROperator_Conv<float>>("NOTSET", dil, g, ks, pads, str, X, W, Y), order++);
            else
               model->AddOperator(std::make_unique<ROperator_Conv<float>>("NOTSET", dil, g, ks, pads, str, X, W, B, Y), order++);
         } else if (kw == "convtr") {
            size_t kh, kw_, pt, pl, pb, pr, sh, sw, oph, opw;
            std::string X, W, B, Y;
            ss >> kh >> kw_ >> pt >> pl >> pb >> pr >> sh >> sw >> oph >> opw >> X >> W >> B >> Y;
            std::vector<size_t> dil{1, 1}, ks{kh, kw_}, pads{pt, pl, pb, pr}, str{sh, sw}, opad{oph, opw};
            model->AddOperator(std::make_unique<ROperator_ConvTranspose<float>>("NOTSET", dil, 1, ks, opad, std::vector<size_t>{}, pads,
                                                                                 str, X, W, B == "-" ? std::string() : B, Y),
                               order++);
         } else if (kw == "relu") {
            std::string X, Y;
            ss >> X >> Y;
            model->AddOperator(std::make_unique<ROperator_Relu<float>>(X, Y), order++);
         } else if (kw == "maxpool" || kw == "avgpool") {
            size_t kh, kw_, p0, p1, p2, p3, sh, sw;
            std::string X, Y;
            ss >> kh >> kw_ >> p0 >> p1 >> p2 >> p3 >> sh >> sw >> X >> Y;
            RAttributes_Pool attr;
            attr.kernel_shape = {kh, kw_};
            attr.pads = {p0, p1, p2, p3};
            attr.strides = {sh, sw};
            model->AddOperator(std::make_unique<ROperator_Pool<float>>(kw == "maxpool" ? MaxPool : AveragePool, attr, X, Y), order++);
         } else if (kw == "flatten") {
            int axis;
            std::string X, Y;
            ss >> axis >> X >> Y;
            model->AddOperator(std::make_unique<ROperator_Reshape>(Flatten, axis, X, "", Y), order++);
         } else if (kw == "softmax") {
            int axis;
            std::string X, Y;
            ss >> axis >> X >> Y;
            model->AddOperator(std::make_unique<ROperator_Softmax<float>>(axis, X, Y), order++);
         } else if (kw == "unary") {
            std::string op, X, Y;
            float alpha;
            ss >> op >> alpha >> X >> Y;
            if (op == "Sigmoid") model->AddOperator(std::make_unique<ROperator_Sigmoid<float>>(X, Y), order++);
            else if (op == "Tanh") model->AddOperator(std::make_unique<ROperator_Tanh<float>>(X, Y), order++);
            else if (op == "LeakyRelu") model->AddOperator(std::make_unique<ROperator_LeakyRelu<float>>(alpha, X, Y), order++);
            else if (op == "Selu") model->AddOperator(std::make_unique<ROperator_Selu<float>>(X, Y), order++);
            else if (op == "Elu") model->AddOperator(std::make_unique<ROperator_Elu<float>>(alpha, X, Y), order++);
            else throw std::runtime_error("unknown unary operator: " + op);
         } else if (kw == "binary") {
            std::string op, A, B, Y;
            ss >> op >> A >> B >> Y;
            if (op == "Add") model->AddOperator(std::make_unique<ROperator_BasicBinary<float, Add>>(A, B, Y), order++);
            else if (op == "Sub") model->AddOperator(std::make_unique<ROperator_BasicBinary<float, Sub>>(A, B, Y), order++);
            else if (op == "Mul") model->AddOperator(std::make_unique<ROperator_BasicBinary<float, Mul>>(A, B, Y), order++);
            else if (op == "Div") model->AddOperator(std::make_unique<ROperator_BasicBinary<float, Div>>(A, B, Y), order++);
            else throw std::runtime_error("unknown binary operator: " + op);
         } else if (kw == "batchnorm") {
            float eps;
            int relu;
            std::string X, S, B, Mn, V, Y;
            ss >> eps >> X >> S >> B >> Mn >> V >> Y >> relu;
            model->AddOperator(std::make_unique<ROperator_BatchNormalization<float>>(
                                  eps, 0.9f, 0, X, S, B, Mn, V, Y, relu ? EActivationType::RELU : EActivationType::UNDEFINED),
                               order++);
         } else if (kw == "output") {
            std::string Y;
            ss >> Y;
            outputs.push_back(Y);
         } else {
            throw std::runtime_error("unknown statement: " + kw);
         }
      }
      model->AddOutputTensorNameList(outputs);
      model->Generate();
      model->OutputGenerated(outDir + "/" + name + ".hxx");
   } catch (std::exception &e) {
      std::fprintf(stderr, "ref_emit: %s\n", e.what());
      return 1;
   }
   return 0;
}
