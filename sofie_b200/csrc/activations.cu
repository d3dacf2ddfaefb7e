// Elementwise family next to the contractions: unary activations and maths, binary operators with
// broadcasting, inference-mode BatchNormalization. All are HBM-bound: 16-byte accesses where the
// tensors allow, a grid of a few waves of 148 SMs. The arithmetic follows the text the reference
// emits for each operator (cited per case), evaluated in the same precision.
#include "common.cuh"

namespace sofie {
namespace {

constexpr int kActThreads = 256;

inline int act_grid(size_t items)
{
   size_t blocks = (items + kActThreads - 1) / kActThreads;
   const size_t cap = size_t(kNumSMs) * 8;
   if (blocks > cap) blocks = cap;
   return blocks ? (int)blocks : 1;
}

__device__ __forceinline__ float unary_apply(int op, float x, float alpha)
{
   switch (op) {
   case SOFIE_UNARY_SIGMOID: return __fdiv_rn(1.f, __fadd_rn(1.f, expf(-x)));          // ROperator_Sigmoid.hxx:59
   case SOFIE_UNARY_TANH: return tanhf(x);                                             // ROperator_Tanh.hxx:60
   case SOFIE_UNARY_LEAKY_RELU: return x >= 0.f ? x : __fmul_rn(alpha, x);             // ROperator_LeakyRelu.hxx:73
   case SOFIE_UNARY_SELU: {                                                            // ROperator_Selu.hxx:59 (double constants)
      const double neg = 1.6732632423543772848170429916717 * (double)(expf(x) - 1.f);
      return (float)(1.0507009873554804934193349852946 * ((double)fmaxf(0.f, x) + fmin(0.0, neg)));
   }
   case SOFIE_UNARY_ELU: return x >= 0.f ? x : __fsub_rn(__fmul_rn(alpha, expf(x)), 1.f); // ROperator_Elu.hxx:71 (as written there)
   case SOFIE_UNARY_NEG: return -x;
   case SOFIE_UNARY_EXP: return expf(x);
   case SOFIE_UNARY_LOG: return logf(x);
   case SOFIE_UNARY_SQRT: return sqrtf(x);
   case SOFIE_UNARY_RECIPROCAL: return __fdiv_rn(1.f, x);
   case SOFIE_UNARY_ERF: return erff(x);                                               // ROperator_Erf.hxx:58
   case SOFIE_UNARY_SWISH: return __fdiv_rn(x, __fadd_rn(1.f, expf(-x)));              // ROperator_Swish.hxx:59
   case SOFIE_UNARY_COS: return cosf(x);
   case SOFIE_UNARY_SIN: return sinf(x);
   default: return fabsf(x); // SOFIE_UNARY_ABS
   }
}

__global__ void unary_f32_kernel(int op, float alpha, const float *__restrict__ X, float *__restrict__ Y, size_t n, bool vec)
{
   const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
   const size_t n4 = vec ? n / 4 : 0;
#pragma unroll 2
   for (size_t i = tid; i < n4; i += nthreads) {
      const float4 v = reinterpret_cast<const float4 *>(X)[i];
      reinterpret_cast<float4 *>(Y)[i] =
         make_float4(unary_apply(op, v.x, alpha), unary_apply(op, v.y, alpha), unary_apply(op, v.z, alpha), unary_apply(op, v.w, alpha));
   }
   for (size_t i = n4 * 4 + tid; i < n; i += nthreads) Y[i] = unary_apply(op, X[i], alpha);
}

__device__ __forceinline__ float binary_apply(int op, float a, float b)
{
   switch (op) { // ROperator_BasicBinary.hxx:18-43
   case SOFIE_BINARY_ADD: return __fadd_rn(a, b);
   case SOFIE_BINARY_SUB: return __fsub_rn(a, b);
   case SOFIE_BINARY_MUL: return __fmul_rn(a, b);
   default: return __fdiv_rn(a, b);
   }
}

__global__ void binary_same_f32_kernel(int op, const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ Y, size_t n,
                                       bool vec)
{
   const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
   const size_t n4 = vec ? n / 4 : 0;
#pragma unroll 2
   for (size_t i = tid; i < n4; i += nthreads) {
      const float4 a = reinterpret_cast<const float4 *>(A)[i], b = reinterpret_cast<const float4 *>(B)[i];
      reinterpret_cast<float4 *>(Y)[i] =
         make_float4(binary_apply(op, a.x, b.x), binary_apply(op, a.y, b.y), binary_apply(op, a.z, b.z), binary_apply(op, a.w, b.w));
   }
   for (size_t i = n4 * 4 + tid; i < n; i += nthreads) Y[i] = binary_apply(op, A[i], B[i]);
}

// General form: the output index is split into up to four coordinates; a broadcast dimension of an
// operand has stride 0.
__global__ void binary_bcast_f32_kernel(sofie_binary_desc d, const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ Y,
                                        size_t n)
{
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
      size_t rem = i, ao = 0, bo = 0;
#pragma unroll
      for (int k = 3; k >= 0; k--) {
         const size_t c = rem % (size_t)d.shape[k];
         rem /= (size_t)d.shape[k];
         ao += c * (size_t)d.a_stride[k];
         bo += c * (size_t)d.b_stride[k];
      }
      Y[i] = binary_apply(d.op, A[ao], B[bo]);
   }
}

// y = ((x - mean[c]) * scale[c]) + bias[c], optional Relu; the three steps are separate roundings as
// in the emitted scopy / saxpy / multiply / saxpy sequence (ROperator_BatchNormalization.hxx:200-226).
__global__ void batchnorm_f32_kernel(sofie_batchnorm_desc d, const float *__restrict__ X, const float *__restrict__ scale,
                                     const float *__restrict__ bias, const float *__restrict__ mean, float *__restrict__ Y, size_t n)
{
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
      const int c = d.layout == SOFIE_LAYOUT_NHWC ? (int)(i % (size_t)d.C) : (int)((i / (size_t)d.HW) % (size_t)d.C);
      float y = __fadd_rn(__fmul_rn(__fsub_rn(X[i], mean[c]), scale[c]), bias[c]);
      Y[i] = d.relu ? relu_ref(y) : y;
   }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

} // namespace
} // namespace sofie

using namespace sofie;

extern "C" int sofie_cuda_unary_f32(void *stream, int32_t op, float alpha, const float *X, float *Y, size_t n)
{
   SOFIE_REQUIRE(op >= SOFIE_UNARY_SIGMOID && op <= SOFIE_UNARY_SIN, "unknown unary operator %d", op);
   if (n == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   const bool vec = aligned16(X) && aligned16(Y);
   unary_f32_kernel<<<act_grid(vec ? n / 4 + 1 : n), kActThreads, 0, as_stream(stream)>>>(op, alpha, X, Y, n, vec);
   SOFIE_LAUNCH_CHECK("unary_f32_kernel");
   return SOFIE_CUDA_OK;
}

extern "C" int sofie_cuda_binary_f32(void *stream, const sofie_binary_desc *d, const float *A, const float *B, float *Y)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->op >= SOFIE_BINARY_ADD && d->op <= SOFIE_BINARY_DIV, "unknown binary operator %d", d->op);
   size_t n = 1;
   bool same = true;
   size_t dense = 1;
   for (int k = 3; k >= 0; k--) {
      SOFIE_REQUIRE(d->shape[k] >= 0 && d->a_stride[k] >= 0 && d->b_stride[k] >= 0, "negative extent or stride");
      if (d->shape[k] > 1) same = same && (size_t)d->a_stride[k] == dense && (size_t)d->b_stride[k] == dense;
      dense *= (size_t)d->shape[k];
      n *= (size_t)d->shape[k];
   }
   if (n == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && B && Y, "NULL tensor");
   cudaStream_t s = as_stream(stream);
   if (same) {
      const bool vec = aligned16(A) && aligned16(B) && aligned16(Y);
      binary_same_f32_kernel<<<act_grid(vec ? n / 4 + 1 : n), kActThreads, 0, s>>>(d->op, A, B, Y, n, vec);
   } else {
      binary_bcast_f32_kernel<<<act_grid(n), kActThreads, 0, s>>>(*d, A, B, Y, n);
   }
   SOFIE_LAUNCH_CHECK("binary_f32_kernel");
   return SOFIE_CUDA_OK;
}

extern "C" int sofie_cuda_batchnorm_f32(void *stream, const sofie_batchnorm_desc *d, const float *X, const float *scale, const float *bias,
                                        const float *mean, float *Y)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->N >= 0 && d->C > 0 && d->HW > 0, "bad BatchNormalization shape %d x %d x %d", d->N, d->C, d->HW);
   SOFIE_REQUIRE(d->layout == SOFIE_LAYOUT_NCHW || d->layout == SOFIE_LAYOUT_NHWC, "unknown layout");
   const size_t n = (size_t)d->N * d->C * d->HW;
   if (n == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(X && Y && scale && bias && mean, "NULL tensor");
   batchnorm_f32_kernel<<<act_grid(n), kActThreads, 0, as_stream(stream)>>>(*d, X, scale, bias, mean, Y, n);
   SOFIE_LAUNCH_CHECK("batchnorm_f32_kernel");
   return SOFIE_CUDA_OK;
}
