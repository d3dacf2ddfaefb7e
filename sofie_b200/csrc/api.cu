// extern "C" entry points of the contractions: argument validation, choice between the tcgen05
// kernels and the CUDA-core kernels, and the host-side preparation of requantisation tables.
#include "contract.cuh"

#include <vector>

namespace sofie {

// Tensor cores first unless forced otherwise; UNSUPPORTED from the tensor-core launcher means
// "shape not covered", and the CUDA-core kernel takes the call.
template <typename Umma, typename Simt>
static int dispatch(Umma umma, Simt simt)
{
   const int forced = forced_engine();
   if (forced != SOFIE_ENGINE_SIMT) {
      int rc = umma();
      if (rc != SOFIE_CUDA_ERR_UNSUPPORTED || forced == SOFIE_ENGINE_TCGEN05) return rc;
   }
   return simt();
}

static int conv_geometry(ConvGeom &g, int N, int C, int H, int W, int Cout, int kH, int kW, int pad_h, int pad_w, int sh,
                         int sw, int dh, int dw, int group, int x_layout, int y_layout, int w_packed, int relu, int pool)
{
   SOFIE_REQUIRE(N >= 0 && C > 0 && H > 0 && W > 0 && Cout > 0 && kH > 0 && kW > 0, "bad convolution shape");
   SOFIE_REQUIRE(pad_h >= 0 && pad_w >= 0 && sh > 0 && sw > 0 && dh > 0 && dw > 0 && group > 0, "bad convolution attributes");
   SOFIE_REQUIRE(C % group == 0 && Cout % group == 0, "channels not divisible by group");
   SOFIE_REQUIRE((x_layout | 1) == 1 && (y_layout | 1) == 1, "unknown layout");
   SOFIE_REQUIRE(pool == 0 || pool == 2, "pool must be 0 or 2");
   SOFIE_REQUIRE(!w_packed || group == 1, "packed weights need group 1");
   const int eh = dh * (kH - 1) + 1, ew = dw * (kW - 1) + 1;
   SOFIE_REQUIRE(H + 2 * pad_h >= eh && W + 2 * pad_w >= ew, "kernel larger than padded input");
   g = ConvGeom{N, C, H, W, Cout, kH, kW, pad_h, pad_w, sh, sw, dh, dw, group, 0, 0, 0, 0,
                x_layout == SOFIE_LAYOUT_NHWC, y_layout == SOFIE_LAYOUT_NHWC, w_packed, relu, pool};
   g.oH = (H + 2 * pad_h - eh) / sh + 1;
   g.oW = (W + 2 * pad_w - ew) / sw + 1;
   // MaxPool 2x2 stride 2 without padding drops a trailing odd row / column, as the reference's
   // window loop does (ROperator_Pool.hxx:371-373).
   g.pH = pool == 2 ? g.oH / 2 : g.oH;
   g.pW = pool == 2 ? g.oW / 2 : g.oW;
   SOFIE_REQUIRE(g.pH > 0 && g.pW > 0, "empty convolution output");
   return SOFIE_CUDA_OK;
}

} // namespace sofie

using namespace sofie;

extern "C" {

int sofie_cuda_gemm_f32(void *stream, const sofie_gemm_f32_desc *d, const float *A, const float *B, const float *C,
                        float *Y)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0, "bad GEMM shape %d x %d x %d", d->M, d->N, d->K);
   SOFIE_REQUIRE(d->bias_kind >= 0 && d->bias_kind <= 2, "bias_kind must be 0, 1 or 2");
   SOFIE_REQUIRE(d->bias_kind == 0 || C != nullptr, "bias_kind set but C is NULL");
   if (d->M == 0) return SOFIE_CUDA_OK; // an empty batch has no rows to compute (and may have NULL A / Y)
   SOFIE_REQUIRE(A && B && Y, "NULL tensor");
   cudaStream_t s = as_stream(stream);
   // few rows, few columns, long K: split K over the grid instead of running on two or three SMs
   if (forced_engine() != SOFIE_ENGINE_TCGEN05 && splitk_shape_ok(*d) && ceil_div(d->M, 128) < 32) {
      if (rowblock_shape_ok(*d, A, B)) return launch_gemm_f32_rowblock(s, *d, A, B, C, Y); // small batch: one launch, no scratch
      const int rc = launch_gemm_f32_splitk_auto(s, *d, A, B, C, Y);
      // no scratch buffer to be had (every slot of the pool belongs to another live stream, or the first call on this
      // stream came during a capture, where nothing can be allocated): the general kernels below take the shape too
      if (rc != SOFIE_CUDA_ERR_NOMEM) return rc;
   }
   return dispatch([&] { return launch_gemm_f32_umma(s, *d, A, B, C, Y); },
                   [&] { return launch_gemm_f32_simt(s, *d, A, B, C, Y); });
}

int sofie_cuda_gemm_f32_batched(void *stream, const sofie_gemm_f32_desc *d, const float *A, const float *B, const float *C, float *Y,
                                int32_t batch, int64_t strideA, int64_t strideB, int64_t strideY)
{
   SOFIE_REQUIRE(d != nullptr && batch >= 0, "NULL descriptor or negative batch");
   SOFIE_REQUIRE(strideA >= 0 && strideB >= 0 && strideY > 0, "bad strides");
   SOFIE_REQUIRE(d->bias_kind != 2, "a stacked product takes a bias per column only");
   for (int32_t b = 0; b < batch; b++) {
      // every matrix of the stack goes through the same dispatch as a single product: tensor cores where the shape allows
      const int rc = sofie_cuda_gemm_f32(stream, d, A + (size_t)b * strideA, B + (size_t)b * strideB, C, Y + (size_t)b * strideY);
      if (rc) return rc;
   }
   return SOFIE_CUDA_OK;
}

int sofie_cuda_conv2d_f32(void *stream, const sofie_conv2d_desc *d, const float *X, const float *W, const float *bias,
                          float *Y)
{
   SOFIE_REQUIRE(d && X && W && Y, "NULL argument");
   ConvGeom g;
   int rc = conv_geometry(g, d->N, d->C, d->H, d->W, d->Cout, d->kH, d->kW, d->pad_h, d->pad_w, d->stride_h, d->stride_w,
                          d->dil_h, d->dil_w, d->group, d->x_layout, d->y_layout, d->w_packed, d->relu, d->pool);
   if (rc) return rc;
   if (d->N == 0) return SOFIE_CUDA_OK;
   cudaStream_t s = as_stream(stream);
   return dispatch([&] { return launch_conv2d_f32_umma(s, g, X, W, bias, Y); },
                   [&] { return launch_conv2d_f32_simt(s, g, X, W, bias, Y); });
}

int sofie_cuda_conv2d_pack_f32(void *stream, const sofie_conv2d_desc *d, const float *W, float *Wpacked)
{
   SOFIE_REQUIRE(d && W && Wpacked, "NULL argument");
   SOFIE_REQUIRE(d->group == 1, "packed weights need group 1");
   return launch_pack_ohwi<float>(as_stream(stream), W, Wpacked, d->Cout, d->C, d->kH, d->kW);
}

int sofie_cuda_qconv2d_pack_i8(void *stream, const sofie_qconv2d_desc *d, const int8_t *W, int8_t *Wpacked)
{
   SOFIE_REQUIRE(d && W && Wpacked, "NULL argument");
   return launch_pack_ohwi<int8_t>(as_stream(stream), W, Wpacked, d->Cout, d->C, d->kH, d->kW);
}

int sofie_cuda_qlinear_prepare(void *stream, int32_t N, int32_t rows_per_n, const int8_t *W_host, int32_t w_is_nk,
                               float a_scale, int32_t a_zp, const float *w_scale_host, float y_scale,
                               const int32_t *bias_host, float *mult_device, int32_t *corr_device)
{
   SOFIE_REQUIRE(N > 0 && rows_per_n > 0 && W_host && w_scale_host && mult_device && corr_device, "bad arguments");
   SOFIE_REQUIRE(y_scale > 0.f, "y_scale must be positive");
   std::vector<float> mult(N);
   std::vector<int32_t> corr(N);
   for (int n = 0; n < N; n++) {
      // fixed order: (a_scale * w_scale[n]) / y_scale, each step rounded to fp32
      volatile float t = a_scale * w_scale_host[n];
      volatile float m = t / y_scale;
      mult[n] = m;
      int64_t sum = 0;
      for (int k = 0; k < rows_per_n; k++)
         sum += w_is_nk ? W_host[(size_t)n * rows_per_n + k] : W_host[(size_t)k * N + n];
      int64_t c = (bias_host ? (int64_t)bias_host[n] : 0) - (int64_t)a_zp * sum;
      SOFIE_REQUIRE(c >= INT32_MIN && c <= INT32_MAX, "zero-point correction overflows int32");
      corr[n] = (int32_t)c;
   }
   cudaStream_t s = as_stream(stream);
   SOFIE_CUDA_TRY(cudaMemcpyAsync(mult_device, mult.data(), sizeof(float) * N, cudaMemcpyHostToDevice, s));
   SOFIE_CUDA_TRY(cudaMemcpyAsync(corr_device, corr.data(), sizeof(int32_t) * N, cudaMemcpyHostToDevice, s));
   SOFIE_CUDA_TRY(cudaStreamSynchronize(s)); // the host vectors go out of scope
   return SOFIE_CUDA_OK;
}

int sofie_cuda_qlinear_matmul(void *stream, const sofie_qgemm_desc *d, const uint8_t *A, const int8_t *W,
                              const float *mult, const int32_t *corr, uint8_t *Y)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0, "bad GEMM shape");
   SOFIE_REQUIRE(d->y_zp >= 0 && d->y_zp <= 255, "y_zp out of range");
   if (d->M == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && W && mult && Y, "NULL tensor");
   cudaStream_t s = as_stream(stream);
   return dispatch([&] { return launch_qgemm_umma(s, *d, A, W, mult, corr, Y, nullptr, 0.f); },
                   [&] { return launch_qgemm_simt(s, *d, A, W, mult, corr, Y, nullptr, 0.f); });
}

int sofie_cuda_qlinear_matmul_f32(void *stream, const sofie_qgemm_desc *d, const uint8_t *A, const int8_t *W, const float *mult,
                                  const int32_t *corr, float y_scale, float *Yf32)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0, "bad GEMM shape");
   SOFIE_REQUIRE(d->y_zp >= 0 && d->y_zp <= 255, "y_zp out of range");
   if (d->M == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && W && mult && Yf32, "NULL tensor");
   cudaStream_t s = as_stream(stream);
   return dispatch([&] { return launch_qgemm_umma(s, *d, A, W, mult, corr, nullptr, Yf32, y_scale); },
                   [&] { return launch_qgemm_simt(s, *d, A, W, mult, corr, nullptr, Yf32, y_scale); });
}

int sofie_cuda_qlinear_conv2d(void *stream, const sofie_qconv2d_desc *d, const uint8_t *X, const int8_t *W,
                              const float *mult, const int32_t *bias, uint8_t *Y)
{
   SOFIE_REQUIRE(d && X && W && mult && Y, "NULL argument");
   SOFIE_REQUIRE(d->x_zp >= 0 && d->x_zp <= 255 && d->y_zp >= 0 && d->y_zp <= 255, "zero point out of range");
   ConvGeom g;
   int rc = conv_geometry(g, d->N, d->C, d->H, d->W, d->Cout, d->kH, d->kW, d->pad_h, d->pad_w, d->stride_h, d->stride_w, 1,
                          1, 1, d->x_layout, d->y_layout, d->w_packed, d->relu, d->pool);
   if (rc) return rc;
   if (d->N == 0) return SOFIE_CUDA_OK;
   cudaStream_t s = as_stream(stream);
   return dispatch([&] { return launch_qconv2d_umma(s, g, X, W, mult, bias, d->x_zp, d->y_zp, Y); },
                   [&] { return launch_qconv2d_simt(s, g, X, W, mult, bias, d->x_zp, d->y_zp, Y); });
}

int sofie_cuda_gemm_e4m3(void *stream, const sofie_fp8_gemm_desc *d, const uint8_t *A, const uint8_t *W,
                         const float *bias, uint16_t *Ybf16, uint8_t *Yq)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0, "bad GEMM shape");
   SOFIE_REQUIRE(!Yq || d->q_scale > 0.f, "Yq given but q_scale is not positive");
   if (d->M == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && W && (Ybf16 || Yq), "NULL tensor");
   cudaStream_t s = as_stream(stream);
   return dispatch([&] { return launch_gemm_e4m3_umma(s, *d, A, W, bias, Ybf16, Yq, nullptr); },
                   [&] { return launch_gemm_e4m3_simt(s, *d, A, W, bias, Ybf16, Yq, nullptr); });
}

int sofie_cuda_gemm_e4m3_f32(void *stream, const sofie_fp8_gemm_desc *d, const uint8_t *A, const uint8_t *W, const float *bias,
                             float *Yf32)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0, "bad GEMM shape");
   if (d->M == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && W && Yf32, "NULL tensor");
   cudaStream_t s = as_stream(stream);
   return dispatch([&] { return launch_gemm_e4m3_umma(s, *d, A, W, bias, nullptr, nullptr, Yf32); },
                   [&] { return launch_gemm_e4m3_simt(s, *d, A, W, bias, nullptr, nullptr, Yf32); });
}

int sofie_cuda_gemm_e4m3_dynamic(void *stream, const sofie_fp8_gemm_desc *d, const uint8_t *A, const float *a_scale_device, const uint8_t *W,
                                 const float *bias, uint16_t *Ybf16, float *Yf32)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0, "bad GEMM shape");
   SOFIE_REQUIRE(d->w_scale > 0.f, "w_scale must be positive");
   if (d->M == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && W && a_scale_device && (Ybf16 || Yf32), "NULL tensor");
   cudaStream_t s = as_stream(stream);
   sofie_fp8_gemm_desc dd = *d;
   dd.q_scale = 0.f; // the next layer's scale is not known before this product is complete: nothing is quantised here
   return dispatch([&] { return launch_gemm_e4m3_umma(s, dd, A, W, bias, Ybf16, nullptr, Yf32, a_scale_device); },
                   [&] { return launch_gemm_e4m3_simt(s, dd, A, W, bias, Ybf16, nullptr, Yf32, a_scale_device); });
}

} // extern "C"
