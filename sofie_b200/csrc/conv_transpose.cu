// ConvTranspose 2-D (group 1), the gather form: an output pixel (oh, ow) collects, for every filter tap
// (r, s), the input pixel ih = (oh + pad - r * dil) / stride when that division is exact and in range.
// Nothing like the reference's per-image filter GEMM + col2im scatter (ROperator_ConvTranspose.icc:364-474,
// SOFIE_common.hxx:576-620) is materialised: no xcol buffer, no zero fill, no second pass for the bias.
// A thread owns one output pixel of four consecutive output channels, so that an input value is read
// once for four filters; threads of a warp walk ow, which makes the input reads contiguous at stride 1.
// X [N,C,H,W], W [C,Cout,kH,kW] (the ONNX layout), Y [N,Cout,oH,oW], fp32 FMA, taps in (r, s, ic) order.
#include "common.cuh"

namespace sofie {
namespace {

constexpr int kOcPerThread = 4;
constexpr int kThreads = 256;

// grid-stride launch: at most eight waves of blocks
inline int grid_for(size_t work_items)
{
   size_t blocks = ceil_div<size_t>(work_items, kThreads);
   const size_t cap = size_t(kNumSMs) * 8;
   return (int)(blocks > cap ? cap : (blocks == 0 ? 1 : blocks));
}

__global__ void __launch_bounds__(kThreads)
conv_transpose2d_f32_kernel(sofie_conv_transpose2d_desc d, int oH, int oW, size_t total, const float *__restrict__ X,
                            const float *__restrict__ Wt, const float *__restrict__ bias, float *__restrict__ Y)
{
   const int ocg = (d.Cout + kOcPerThread - 1) / kOcPerThread;
   const size_t in_hw = (size_t)d.H * d.W, out_hw = (size_t)oH * oW, taps = (size_t)d.kH * d.kW;
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const int ow = (int)(i % oW);
      size_t t = i / oW;
      const int oh = (int)(t % oH);
      t /= oH;
      const int oc0 = (int)(t % ocg) * kOcPerThread;
      const int n = (int)(t / ocg);
      float acc[kOcPerThread] = {0.f, 0.f, 0.f, 0.f};
      const float *x = X + (size_t)n * d.C * in_hw;
      for (int r = 0; r < d.kH; r++) {
         const int th = oh + d.pad_h - r * d.dil_h;
         if (th < 0 || th % d.stride_h) continue;
         const int ih = th / d.stride_h;
         if (ih >= d.H) continue;
         for (int s = 0; s < d.kW; s++) {
            const int tw = ow + d.pad_w - s * d.dil_w;
            if (tw < 0 || tw % d.stride_w) continue;
            const int iw = tw / d.stride_w;
            if (iw >= d.W) continue;
            const float *xp = x + (size_t)ih * d.W + iw;
            const float *wp = Wt + (size_t)oc0 * taps + (size_t)r * d.kW + s;
            for (int ic = 0; ic < d.C; ic++) {
               const float v = __ldg(xp + (size_t)ic * in_hw);
               const float *w = wp + (size_t)ic * d.Cout * taps;
#pragma unroll
               for (int j = 0; j < kOcPerThread; j++)
                  if (oc0 + j < d.Cout) acc[j] = fmaf(v, __ldg(w + (size_t)j * taps), acc[j]);
            }
         }
      }
#pragma unroll
      for (int j = 0; j < kOcPerThread; j++) {
         if (oc0 + j < d.Cout) {
            float v = acc[j] + (bias ? __ldg(bias + oc0 + j) : 0.f);
            if (d.relu) v = relu_ref(v);
            Y[((size_t)n * d.Cout + oc0 + j) * out_hw + (size_t)oh * oW + ow] = v;
         }
      }
   }
}

// ---- the product form: one GEMM over all images on the tensor cores, then a gather -------------------------------
// The reference computes, per image, filter^T [Cout*kH*kW, C] x image [C, H*W] with sgemm_ and scatters the columns
// into the output (col2im). Here the images are brought to channel-last once, so ALL of them are one K-major operand:
//     P [N*H*W, kH*kW*Cout] = Xt [N*H*W, C] x Wt [kH*kW*Cout, C]^T        (sofie_cuda_gemm_f32: tcgen05, 3xTF32)
// and an output pixel gathers its taps' products from P (the gather form of col2im: no atomics, no zero fill), adds the
// bias and applies Relu. Column order (tap, output channel) makes four output channels of a tap 16 contiguous bytes.
__global__ void conv_transpose_weights_kernel(const float *__restrict__ W, float *__restrict__ Wt, int C, int Cout, int taps)
{
   const size_t total = (size_t)C * Cout * taps;
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const int ic = (int)(i % C);
      const size_t row = i / C; // (tap, co)
      const int co = (int)(row % Cout), tap = (int)(row / Cout);
      Wt[i] = __ldg(W + ((size_t)ic * Cout + co) * taps + tap);
   }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
conv_transpose_gather_kernel(sofie_conv_transpose2d_desc d, int oH, int oW, size_t total, const float *__restrict__ P,
                             const float *__restrict__ bias, float *__restrict__ Y)
{
   const int ocg = (d.Cout + kOcPerThread - 1) / kOcPerThread;
   const size_t in_hw = (size_t)d.H * d.W, out_hw = (size_t)oH * oW;
   const size_t ncol = (size_t)d.kH * d.kW * d.Cout;
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const int ow = (int)(i % oW);
      size_t t = i / oW;
      const int oh = (int)(t % oH);
      t /= oH;
      const int oc0 = (int)(t % ocg) * kOcPerThread;
      const int n = (int)(t / ocg);
      float acc[kOcPerThread] = {0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < d.kH; r++) {
         const int th = oh + d.pad_h - r * d.dil_h;
         if (th < 0 || th % d.stride_h) continue;
         const int ih = th / d.stride_h;
         if (ih >= d.H) continue;
         for (int s = 0; s < d.kW; s++) {
            const int tw = ow + d.pad_w - s * d.dil_w;
            if (tw < 0 || tw % d.stride_w) continue;
            const int iw = tw / d.stride_w;
            if (iw >= d.W) continue;
            const float *p = P + ((size_t)n * in_hw + (size_t)ih * d.W + iw) * ncol + (size_t)(r * d.kW + s) * d.Cout + oc0;
            if (VEC) {
               const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
               acc[0] += v.x;
               acc[1] += v.y;
               acc[2] += v.z;
               acc[3] += v.w;
            } else {
#pragma unroll
               for (int j = 0; j < kOcPerThread; j++)
                  if (oc0 + j < d.Cout) acc[j] += __ldg(p + j);
            }
         }
      }
#pragma unroll
      for (int j = 0; j < kOcPerThread; j++) {
         if (oc0 + j < d.Cout) {
            float v = acc[j] + (bias ? __ldg(bias + oc0 + j) : 0.f);
            if (d.relu) v = relu_ref(v);
            Y[((size_t)n * d.Cout + oc0 + j) * out_hw + (size_t)oh * oW + ow] = v;
         }
      }
   }
}

// shape checks shared by the two entry points; the output extent on success
int check_conv_transpose(const sofie_conv_transpose2d_desc *d, long &oH, long &oW)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->N >= 0 && d->C > 0 && d->H > 0 && d->W > 0 && d->Cout > 0 && d->kH > 0 && d->kW > 0, "bad ConvTranspose shape");
   SOFIE_REQUIRE(d->stride_h > 0 && d->stride_w > 0 && d->dil_h > 0 && d->dil_w > 0 && d->pad_h >= 0 && d->pad_w >= 0 &&
                    d->out_pad_h >= 0 && d->out_pad_w >= 0,
                 "bad ConvTranspose strides, dilations or pads");
   // output_padding only makes sense below the stride (ONNX); larger values would leave rows nothing writes to
   SOFIE_REQUIRE(d->out_pad_h < d->stride_h || d->out_pad_h < d->dil_h, "output_padding must be smaller than the stride or the dilation");
   SOFIE_REQUIRE(d->out_pad_w < d->stride_w || d->out_pad_w < d->dil_w, "output_padding must be smaller than the stride or the dilation");
   oH = (long)d->stride_h * (d->H - 1) + (long)d->dil_h * (d->kH - 1) + 1 + d->out_pad_h - 2L * d->pad_h;
   oW = (long)d->stride_w * (d->W - 1) + (long)d->dil_w * (d->kW - 1) + 1 + d->out_pad_w - 2L * d->pad_w;
   SOFIE_REQUIRE(oH > 0 && oW > 0 && oH < (1L << 30) && oW < (1L << 30), "ConvTranspose output would be empty");
   return SOFIE_CUDA_OK;
}

} // namespace
} // namespace sofie

using namespace sofie;

extern "C" size_t sofie_cuda_conv_transpose2d_f32_gemm_scratch(const sofie_conv_transpose2d_desc *d)
{
   return d ? sofie_conv_transpose2d_gemm_scratch_bytes(d) : 0;
}

extern "C" int sofie_cuda_conv_transpose2d_f32_gemm(void *stream, const sofie_conv_transpose2d_desc *d, const float *X, const float *W,
                                                    const float *bias, float *Y, void *scratch, size_t scratch_bytes)
{
   long oH, oW;
   const int rc = check_conv_transpose(d, oH, oW);
   if (rc) return rc;
   const size_t need = sofie_conv_transpose2d_gemm_scratch_bytes(d);
   if (need == 0) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "this ConvTranspose shape is served by sofie_cuda_conv_transpose2d_f32 only");
   if (d->N == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(X && W && Y && scratch, "NULL tensor");
   SOFIE_REQUIRE(scratch_bytes >= need, "scratch of %zu bytes, %zu needed", scratch_bytes, need);
   SOFIE_REQUIRE((reinterpret_cast<uintptr_t>(scratch) & 255) == 0, "scratch must be 256-byte aligned");
   cudaStream_t s = as_stream(stream);
   const size_t pixels = (size_t)d->N * d->H * d->W;
   const int taps = d->kH * d->kW;
   float *Xt = static_cast<float *>(scratch);
   float *Wt = Xt + sofie_round_up_floats(pixels * d->C);
   float *P = Wt + sofie_round_up_floats((size_t)taps * d->Cout * d->C);
   int st = sofie_cuda_nchw_to_nhwc_f32(stream, X, Xt, d->N, d->C, d->H, d->W);
   if (st) return st;
   conv_transpose_weights_kernel<<<grid_for((size_t)taps * d->Cout * d->C), kThreads, 0, s>>>(W, Wt, d->C, d->Cout, taps);
   SOFIE_LAUNCH_CHECK("conv_transpose_weights_kernel");
   SOFIE_REQUIRE(pixels < (1u << 31) && (size_t)taps * d->Cout < (1u << 31), "ConvTranspose too large for the product form");
   const sofie_gemm_f32_desc g = {(int32_t)pixels, (int32_t)(taps * d->Cout), d->C, 0, 1, 1.f, 0.f, 0, 0};
   st = sofie_cuda_gemm_f32(stream, &g, Xt, Wt, nullptr, P); // records the engine that ran
   if (st) return st;
   const size_t total = (size_t)d->N * ((d->Cout + kOcPerThread - 1) / kOcPerThread) * oH * oW;
   if (d->Cout % 4 == 0)
      conv_transpose_gather_kernel<true><<<grid_for(total), kThreads, 0, s>>>(*d, (int)oH, (int)oW, total, P, bias, Y);
   else
      conv_transpose_gather_kernel<false><<<grid_for(total), kThreads, 0, s>>>(*d, (int)oH, (int)oW, total, P, bias, Y);
   SOFIE_LAUNCH_CHECK("conv_transpose_gather_kernel");
   return SOFIE_CUDA_OK;
}

extern "C" int sofie_cuda_conv_transpose2d_f32(void *stream, const sofie_conv_transpose2d_desc *d, const float *X, const float *W,
                                               const float *bias, float *Y)
{
   long oH, oW;
   const int rc = check_conv_transpose(d, oH, oW);
   if (rc) return rc;
   if (d->N == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(X && W && Y, "NULL tensor");
   const size_t total = (size_t)d->N * ((d->Cout + kOcPerThread - 1) / kOcPerThread) * oH * oW;
   conv_transpose2d_f32_kernel<<<grid_for(total), kThreads, 0, as_stream(stream)>>>(*d, (int)oH, (int)oW, total, X, W, bias, Y);
   SOFIE_LAUNCH_CHECK("conv_transpose2d_f32_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}
