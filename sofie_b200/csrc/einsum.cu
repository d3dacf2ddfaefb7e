// Einsum of two operands in its general form: Y[out labels] = sum over every other label of A[...] * B[...].
// The reference emits this as nested loops over the output and then the summation labels, or as one sgemm_ per
// stack index when the equation is a (stacked) matrix product (ROperator_Einsum.hxx:200-332); "ik,kj->ij" goes to
// the GEMM kernels before it gets here. A thread owns one output element and walks the summation labels with an
// odometer, so any label order, repeated batch labels and labels that only one operand carries all work; the kernel is
// meant for the small contractions of exported graphs, not for large products.
#include "common.cuh"

namespace sofie {
namespace {

__global__ void __launch_bounds__(256)
einsum_f32_kernel(sofie_einsum_desc d, long long out_total, long long sum_total, const float *__restrict__ A, const float *__restrict__ B,
                  float *__restrict__ Y)
{
   for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < out_total; o += (long long)gridDim.x * blockDim.x) {
      long long rem = o, a0 = 0, b0 = 0;
      for (int i = d.n_out - 1; i >= 0; i--) {
         const long long idx = rem % d.extent[i];
         rem /= d.extent[i];
         a0 += idx * d.a_stride[i];
         b0 += idx * d.b_stride[i];
      }
      int idx[SOFIE_EINSUM_MAX_LABELS];
#pragma unroll
      for (int i = 0; i < SOFIE_EINSUM_MAX_LABELS; i++) idx[i] = 0;
      long long a = a0, b = b0;
      float acc = 0.f;
      for (long long q = 0; q < sum_total; q++) {
         acc = fmaf(__ldg(A + a), __ldg(B + b), acc);
         // odometer over the summation labels, last label fastest
         for (int i = d.n_sum - 1; i >= 0; i--) {
            const int l = d.n_out + i;
            a += d.a_stride[l];
            b += d.b_stride[l];
            if (++idx[i] < d.extent[l]) break;
            a -= d.a_stride[l] * d.extent[l];
            b -= d.b_stride[l] * d.extent[l];
            idx[i] = 0;
         }
      }
      Y[o] = acc;
   }
}

} // namespace
} // namespace sofie

using namespace sofie;

extern "C" int sofie_cuda_einsum_f32(void *stream, const sofie_einsum_desc *d, const float *A, const float *B, float *Y)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->n_out >= 0 && d->n_sum >= 0 && d->n_out + d->n_sum <= SOFIE_EINSUM_MAX_LABELS, "at most %d labels", SOFIE_EINSUM_MAX_LABELS);
   long long out_total = 1, sum_total = 1;
   for (int i = 0; i < d->n_out + d->n_sum; i++) {
      SOFIE_REQUIRE(d->extent[i] >= 0 && d->extent[i] < (1LL << 31) && d->a_stride[i] >= 0 && d->b_stride[i] >= 0, "bad label extent or stride");
      (i < d->n_out ? out_total : sum_total) *= d->extent[i];
      SOFIE_REQUIRE(out_total < (1LL << 40) && sum_total < (1LL << 40), "Einsum too large");
   }
   if (out_total == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && B && Y, "NULL tensor");
   long long blocks = (out_total + 255) / 256;
   if (blocks > 8LL * kNumSMs) blocks = 8LL * kNumSMs;
   einsum_f32_kernel<<<(int)blocks, 256, 0, as_stream(stream)>>>(*d, out_total, sum_total, A, B, Y);
   SOFIE_LAUNCH_CHECK("einsum_f32_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}
