// 3-D convolution and pooling on [N, C, D, H, W] tensors (reference: ROperator_Conv.hxx with fDim == 3 -- UTILITY::Im2col_3d,
// SOFIE_common.hxx:521-573, then one sgemm_ per image and group -- and the fDim == 3 loops of ROperator_Pool.hxx:266-476).
// Direct kernels on CUDA cores: one thread per output element, taps in (ic, kd, kh, kw) order, fp32 FMA; no column buffer.
// Volumes are rare on this path and small in the reference's own tests; the 2-D tensor-core kernels have no 3-D form yet.
#include "common.cuh"

namespace sofie {
namespace {

constexpr int kThreads = 256;
inline int grid_for(size_t work_items)
{
   size_t blocks = ceil_div<size_t>(work_items, kThreads);
   const size_t cap = size_t(kNumSMs) * 8;
   return (int)(blocks > cap ? cap : (blocks == 0 ? 1 : blocks));
}

__global__ void __launch_bounds__(kThreads)
conv3d_f32_kernel(sofie_conv3d_desc d, int oD, int oH, int oW, size_t total, const float *__restrict__ X, const float *__restrict__ Wt,
                  const float *__restrict__ bias, float *__restrict__ Y)
{
   const int cin_g = d.C / d.group, cout_g = d.Cout / d.group;
   const size_t in_plane = (size_t)d.D * d.H * d.W, taps = (size_t)d.kD * d.kH * d.kW;
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const int ow = (int)(i % oW);
      size_t t = i / oW;
      const int oh = (int)(t % oH);
      t /= oH;
      const int od = (int)(t % oD);
      t /= oD;
      const int co = (int)(t % d.Cout);
      const int n = (int)(t / d.Cout);
      const int g = co / cout_g;
      const float *x = X + ((size_t)n * d.C + (size_t)g * cin_g) * in_plane;
      const float *w = Wt + (size_t)co * cin_g * taps;
      float acc = 0.f;
      for (int ic = 0; ic < cin_g; ic++) {
         for (int kd = 0; kd < d.kD; kd++) {
            const int id = od * d.stride_d - d.pad_d + kd * d.dil_d;
            if (id < 0 || id >= d.D) continue;
            for (int kh = 0; kh < d.kH; kh++) {
               const int ih = oh * d.stride_h - d.pad_h + kh * d.dil_h;
               if (ih < 0 || ih >= d.H) continue;
               for (int kw = 0; kw < d.kW; kw++) {
                  const int iw = ow * d.stride_w - d.pad_w + kw * d.dil_w;
                  if (iw < 0 || iw >= d.W) continue;
                  acc = fmaf(__ldg(x + (size_t)ic * in_plane + ((size_t)id * d.H + ih) * d.W + iw),
                             __ldg(w + (size_t)ic * taps + ((size_t)kd * d.kH + kh) * d.kW + kw), acc);
               }
            }
         }
      }
      if (bias) acc += __ldg(bias + co);
      if (d.relu) acc = relu_ref(acc);
      Y[i] = acc;
   }
}

__global__ void __launch_bounds__(kThreads)
pool3d_f32_kernel(sofie_pool3d_desc d, int oD, int oH, int oW, size_t total, const float *__restrict__ X, float *__restrict__ Y)
{
   const bool padded = d.pads[0] || d.pads[1] || d.pads[2] || d.pads[3] || d.pads[4] || d.pads[5];
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const int ow = (int)(i % oW);
      size_t t = i / oW;
      const int oh = (int)(t % oH);
      t /= oH;
      const int od = (int)(t % oD);
      const size_t plane = t / oD; // n * C + c
      const float *x = X + plane * (size_t)d.D * d.H * d.W;
      const int d0 = od * d.stride_d - d.pads[0], h0 = oh * d.stride_h - d.pads[1], w0 = ow * d.stride_w - d.pads[2];
      float value = d.mode == 0 ? -INFINITY : 0.f;
      int count = (d.count_include_pad || !padded) ? d.kD * d.kH * d.kW : 0;
      for (int a = d0; a < d0 + d.kD; a++) {
         if (a < 0 || a >= d.D) continue;
         for (int b = h0; b < h0 + d.kH; b++) {
            if (b < 0 || b >= d.H) continue;
            for (int c = w0; c < w0 + d.kW; c++) {
               if (c < 0 || c >= d.W) continue;
               const float v = __ldg(x + ((size_t)a * d.H + b) * d.W + c);
               if (d.mode == 0) {
                  if (v > value) value = v;
               } else {
                  value += v;
                  if (!d.count_include_pad && padded) count++;
               }
            }
         }
      }
      if (d.mode == 1) value /= (float)count;
      Y[i] = value;
   }
}

} // namespace
} // namespace sofie

using namespace sofie;

extern "C" int sofie_cuda_conv3d_f32(void *stream, const sofie_conv3d_desc *d, const float *X, const float *W, const float *bias, float *Y)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->N >= 0 && d->C > 0 && d->D > 0 && d->H > 0 && d->W > 0 && d->Cout > 0 && d->kD > 0 && d->kH > 0 && d->kW > 0, "bad Conv shape");
   SOFIE_REQUIRE(d->stride_d > 0 && d->stride_h > 0 && d->stride_w > 0 && d->dil_d > 0 && d->dil_h > 0 && d->dil_w > 0 && d->pad_d >= 0 &&
                    d->pad_h >= 0 && d->pad_w >= 0,
                 "bad Conv strides, dilations or pads");
   SOFIE_REQUIRE(d->group > 0 && d->C % d->group == 0 && d->Cout % d->group == 0, "channels must be multiples of the group count");
   const long oD = ((long)d->D + 2L * d->pad_d - ((long)d->dil_d * (d->kD - 1) + 1)) / d->stride_d + 1;
   const long oH = ((long)d->H + 2L * d->pad_h - ((long)d->dil_h * (d->kH - 1) + 1)) / d->stride_h + 1;
   const long oW = ((long)d->W + 2L * d->pad_w - ((long)d->dil_w * (d->kW - 1) + 1)) / d->stride_w + 1;
   SOFIE_REQUIRE(oD > 0 && oH > 0 && oW > 0, "kernel larger than the padded input");
   if (d->N == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(X && W && Y, "NULL tensor");
   const size_t total = (size_t)d->N * d->Cout * oD * oH * oW;
   conv3d_f32_kernel<<<grid_for(total), kThreads, 0, as_stream(stream)>>>(*d, (int)oD, (int)oH, (int)oW, total, X, W, bias, Y);
   SOFIE_LAUNCH_CHECK("conv3d_f32_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

extern "C" int sofie_cuda_pool3d_f32(void *stream, const sofie_pool3d_desc *d, const float *X, float *Y)
{
   SOFIE_REQUIRE(d && X && Y, "NULL argument");
   SOFIE_REQUIRE(d->mode == 0 || d->mode == 1, "pool mode must be 0 (max) or 1 (average)");
   SOFIE_REQUIRE(d->N >= 0 && d->C > 0 && d->D > 0 && d->H > 0 && d->W > 0 && d->kD > 0 && d->kH > 0 && d->kW > 0 && d->stride_d > 0 &&
                    d->stride_h > 0 && d->stride_w > 0,
                 "bad pooling shape");
   for (int i = 0; i < 6; i++) SOFIE_REQUIRE(d->pads[i] >= 0, "negative pad");
   const int dspan = d->D + d->pads[0] + d->pads[3] - d->kD + 1, hspan = d->H + d->pads[1] + d->pads[4] - d->kH + 1,
             wspan = d->W + d->pads[2] + d->pads[5] - d->kW + 1;
   SOFIE_REQUIRE(dspan > 0 && hspan > 0 && wspan > 0, "pooling window larger than padded input");
   const int oD = ceil_div(dspan, d->stride_d), oH = ceil_div(hspan, d->stride_h), oW = ceil_div(wspan, d->stride_w);
   const size_t total = (size_t)d->N * d->C * oD * oH * oW;
   if (total == 0) return SOFIE_CUDA_OK;
   pool3d_f32_kernel<<<grid_for(total), kThreads, 0, as_stream(stream)>>>(*d, oD, oH, oW, total, X, Y);
   SOFIE_LAUNCH_CHECK("pool3d_f32_kernel");
   return SOFIE_CUDA_OK;
}
