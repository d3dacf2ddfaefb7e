/*
 * sofie_oracle.c -- CPU oracle for the dense-contraction inference path. TEST INFRASTRUCTURE ONLY.
 *
 * Only the tests, the smoke check and the CPU-baseline leg of the benchmark may call this file;
 * the product (libSOFIE_cuda and the code the generator emits) never does.
 *
 * fp32 part: a restatement, in plain C, of what the reference's *emitted* inference code computes
 * (paths are relative to the reference project root):
 *   - Gemm / MatMul   src/SOFIE_core/inc/SOFIE/ROperator_Gemm.hxx:292-390  (bias copy, sgemm_, relu sweep)
 *   - Conv            src/SOFIE_core/inc/SOFIE/ROperator_Conv.hxx:302-522  (weight repack, per-image Im2col,
 *                     sgemm_, saxpy_ of the broadcast bias)
 *   - Im2col          src/SOFIE_core/inc/SOFIE/SOFIE_common.hxx:485-518
 *   - Relu            src/SOFIE_core/inc/SOFIE/ROperator_Relu.hxx:54-66
 *   - MaxPool/AvgPool src/SOFIE_core/inc/SOFIE/ROperator_Pool.hxx:266-476
 *   - Softmax         src/SOFIE_core/inc/SOFIE/ROperator_Softmax.hxx:53-184
 * The BLAS behind sgemm_ is a third-party library that is not part of the reference tree (OpenBLAS,
 * no pinned version); its summation order is unspecified. The oracle therefore evaluates the BLAS
 * definition C = alpha*op(A)*op(B) + beta*C with a double accumulator and rounds once to fp32.
 * Parity pinning: checked against the reference's golden vectors (Linear_16/32/64, ConvWith*,
 * MaxPool2d, AvgPool, Softmax*) and against the reference's own emitted code run through OpenBLAS.
 *
 * int8 / FP8 part: PARITY UNPINNED. The reference has no QuantizeLinear / DequantizeLinear /
 * QLinearMatMul / QLinearConv / FP8 operators, no tests and no fixtures for them
 * (src/SOFIE_parsers/src/RModelParser_ONNX.cxx:154-236,560-591). These functions restate the ONNX
 * operator definitions in the reference's emission style (row-major, NCHW, same pad / stride
 * conventions as ROperator_Conv) with one fixed arithmetic recipe:
 *   acc (int32) = sum (a - a_zp) * (w - w_zp) [+ bias_i32];  mult = (a_scale * w_scale[n]) / y_scale (fp32);
 *   q = clamp(nearbyintf((float)acc * mult), qmin - y_zp, qmax - y_zp) + y_zp       (round half to even).
 * Compile with -ffp-contract=off so no FMA contraction changes the rounding.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------ */
/* A minimal parallel-for over independent rows / images (pthreads; the toolchain has no OpenMP */
/* runtime). ORACLE_THREADS in the environment caps the thread count; 1 runs inline.            */
/* ------------------------------------------------------------------------------------------ */
typedef void (*oracle_row_fn)(long begin, long end, void *ctx);
typedef struct { oracle_row_fn fn; void *ctx; long begin, end; } oracle_job;
static void *oracle_job_main(void *p)
{
   oracle_job *j = (oracle_job *)p;
   j->fn(j->begin, j->end, j->ctx);
   return NULL;
}
ORACLE_API int oracle_num_threads(void)
{
   const char *env = getenv("ORACLE_THREADS");
   long n = env ? atol(env) : sysconf(_SC_NPROCESSORS_ONLN);
   if (n < 1) n = 1;
   if (n > 256) n = 256;
   return (int)n;
}
static void oracle_parallel_for(long n, oracle_row_fn fn, void *ctx)
{
   int nt = oracle_num_threads();
   if (nt > n) nt = (int)(n > 0 ? n : 1);
   if (nt <= 1) {
      fn(0, n, ctx);
      return;
   }
   pthread_t tid[256];
   oracle_job job[256];
   long chunk = (n + nt - 1) / nt;
   int started = 0;
   for (int t = 0; t < nt; t++) {
      long b = t * chunk, e = b + chunk > n ? n : b + chunk;
      if (b >= e) break;
      job[t] = (oracle_job){fn, ctx, b, e};
      if (pthread_create(&tid[t], NULL, oracle_job_main, &job[t]) != 0) {
         fn(b, e, ctx); /* could not start a thread: do the chunk here */
         tid[t] = 0;
      }
      started = t + 1;
   }
   for (int t = 0; t < started; t++)
      if (tid[t]) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------------------------------ */
/* fp32                                                                                       */
/* ------------------------------------------------------------------------------------------ */

/* Gemm as emitted by ROperator_Gemm.hxx:360-381: Y <- bcast(C) ; Y = alpha*op(A)*op(B) + beta*Y ; relu.
 * A is [M,K] (or [K,M] when transA), B is [K,N] (or [N,K] when transB), all row-major.
 * bias_kind: 0 none (beta must be 0), 1 vector of N broadcast over rows, 2 full [M,N]. */
typedef struct {
   int transA, transB, M, N, K, bias_kind, relu;
   float alpha, beta;
   const float *A, *B, *C;
   float *Y;
} gemm_f32_args;
static void gemm_f32_rows(long begin, long end, void *ctx)
{
   const gemm_f32_args *g = (const gemm_f32_args *)ctx;
   const int transA = g->transA, transB = g->transB, M = g->M, N = g->N, K = g->K, bias_kind = g->bias_kind, relu = g->relu;
   const float alpha = g->alpha, beta = g->beta, *A = g->A, *B = g->B, *C = g->C;
   float *Y = g->Y;
   for (long m = begin; m < end; m++) {
      for (int n = 0; n < N; n++) {
         double acc = 0.0;
         for (int k = 0; k < K; k++) {
            float a = transA ? A[(size_t)k * M + m] : A[(size_t)m * K + k];
            float b = transB ? B[(size_t)n * K + k] : B[(size_t)k * N + n];
            acc += (double)a * (double)b;
         }
         double y = (double)alpha * acc;
         if (bias_kind == 1) y += (double)beta * (double)C[n];
         else if (bias_kind == 2) y += (double)beta * (double)C[(size_t)m * N + n];
         float r = (float)y;
         if (relu) r = (r > 0) ? r : 0; /* ROperator_Gemm.hxx:377-381: NaN and -0 become 0 */
         Y[(size_t)m * N + n] = r;
      }
   }
}
ORACLE_API void oracle_gemm_f32(int transA, int transB, int M, int N, int K, float alpha, const float *A,
                                const float *B, float beta, const float *C, int bias_kind, int relu, float *Y)
{
   gemm_f32_args g = {transA, transB, M, N, K, bias_kind, relu, alpha, beta, A, B, C, Y};
   oracle_parallel_for(M, gemm_f32_rows, &g);
}

/* Im2col restated from SOFIE_common.hxx:485-518: col[(c,kr,kc)][(oh,ow)], zero outside the image. */
ORACLE_API void oracle_im2col_f32(const float *im, int channels, int height, int width, int kernel_h, int kernel_w,
                                  int pad_h, int pad_w, int stride_h, int stride_w, int dil_h, int dil_w, float *col)
{
   const int out_h = (height + 2 * pad_h - (dil_h * (kernel_h - 1) + 1)) / stride_h + 1;
   const int out_w = (width + 2 * pad_w - (dil_w * (kernel_w - 1) + 1)) / stride_w + 1;
   size_t o = 0;
   for (int c = 0; c < channels; c++) {
      const float *plane = im + (size_t)c * height * width;
      for (int kr = 0; kr < kernel_h; kr++) {
         for (int kc = 0; kc < kernel_w; kc++) {
            for (int oh = 0; oh < out_h; oh++) {
               int ih = -pad_h + kr * dil_h + oh * stride_h;
               for (int ow = 0; ow < out_w; ow++) {
                  int iw = -pad_w + kc * dil_w + ow * stride_w;
                  col[o++] = (ih >= 0 && ih < height && iw >= 0 && iw < width) ? plane[(size_t)ih * width + iw] : 0.0f;
               }
            }
         }
      }
   }
}

/* 2-D Conv as emitted by ROperator_Conv.hxx:302-522 for dilation 1 (the reference's dilated path is
 * internally inconsistent and has no fixture; ONNX semantics are used for dilation > 1):
 * per image and group, xcol = Im2col(X); Y[oc][p] = sum_k Wf[oc][k] * xcol[k][p]; then Y += bias[oc].
 * X [N,C,H,W], W [Cout, C/group, kh, kw], bias [Cout] or NULL, Y [N,Cout,oH,oW]. Symmetric pads. */
typedef struct {
   int N, C, H, W, Cout, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, group, relu;
   const float *X, *Wt, *bias;
   float *Y;
} conv2d_f32_args;
static void conv2d_f32_images(long begin, long end, void *ctx)
{
   const conv2d_f32_args *a = (const conv2d_f32_args *)ctx;
   const int C = a->C, H = a->H, W = a->W, Cout = a->Cout, kh = a->kh, kw = a->kw, group = a->group;
   const int oH = (H + 2 * a->pad_h - (a->dil_h * (kh - 1) + 1)) / a->stride_h + 1;
   const int oW = (W + 2 * a->pad_w - (a->dil_w * (kw - 1) + 1)) / a->stride_w + 1;
   const int cg = C / group, og = Cout / group, kk = cg * kh * kw;
   const size_t P = (size_t)oH * oW;
   float *col = (float *)malloc(sizeof(float) * (size_t)kk * P);
   for (long n = begin; n < end; n++) {
      for (int g = 0; g < group; g++) {
         oracle_im2col_f32(a->X + ((size_t)n * C + (size_t)g * cg) * H * W, cg, H, W, kh, kw, a->pad_h, a->pad_w,
                           a->stride_h, a->stride_w, a->dil_h, a->dil_w, col);
         for (int oc = 0; oc < og; oc++) {
            const float *wrow = a->Wt + ((size_t)g * og + oc) * kk;
            float *yrow = a->Y + ((size_t)n * Cout + (size_t)g * og + oc) * P;
            for (size_t p = 0; p < P; p++) {
               double acc = 0.0;
               for (int k = 0; k < kk; k++) acc += (double)wrow[k] * (double)col[(size_t)k * P + p];
               float r = (float)acc;
               if (a->bias) r = r + a->bias[g * og + oc]; /* saxpy_ in fp32, ROperator_Conv.hxx:509-517 */
               if (a->relu) r = (r > 0) ? r : 0;
               yrow[p] = r;
            }
         }
      }
   }
   free(col);
}
ORACLE_API void oracle_conv2d_f32(int N, int C, int H, int W, int Cout, int kh, int kw, int pad_h, int pad_w,
                                  int stride_h, int stride_w, int dil_h, int dil_w, int group, const float *X,
                                  const float *Wt, const float *bias, int relu, float *Y)
{
   conv2d_f32_args a = {N, C, H, W, Cout, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, group, relu, X, Wt, bias, Y};
   oracle_parallel_for(N, conv2d_f32_images, &a);
}

/* ConvTranspose, 2-D, group 1, as emitted by ROperator_ConvTranspose.icc:364-474:
 *   per image   xcol[(oc,r,s)][ih*W+iw] = sum_ic X[ic][ih][iw] * Wt[ic][oc][r][s]      (the sgemm_ at :370-375)
 *               Y_n = col2im(xcol)      scatter-add into the zeroed image, UTILITY::col2im (SOFIE_common.hxx:576-620)
 *   at the end  Y += bias broadcast per output channel                                 (the saxpy_ at :462-471)
 * Output size (ShapeInference :83-90): o = stride*(i-1) + dil*(k-1)+1 + output_padding - 2*pad.
 * The reference's own tests pin dilation 1 only (its emission dilates the filter matrix AND passes the
 * dilation to col2im, :233-262,:380-391); this restates the ONNX definition, which is the same thing at dilation 1. */
typedef struct {
   int N, C, H, W, Cout, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, oH, oW;
   const float *X, *Wt, *bias;
   float *Y;
} convtr_args;
static void conv_transpose2d_images(long n0, long n1, void *ctx)
{
   const convtr_args *a = (const convtr_args *)ctx;
   const size_t in_hw = (size_t)a->H * a->W, out_hw = (size_t)a->oH * a->oW, taps = (size_t)a->kh * a->kw;
   float *col = (float *)malloc(sizeof(float) * a->Cout * taps * in_hw);
   for (long n = n0; n < n1; n++) {
      const float *x = a->X + (size_t)n * a->C * in_hw;
      float *y = a->Y + (size_t)n * a->Cout * out_hw;
      for (size_t j = 0; j < (size_t)a->Cout * taps; j++) { /* j = (oc, r, s) */
         const size_t oc = j / taps, t = j % taps;
         for (size_t p = 0; p < in_hw; p++) {
            float acc = 0.f;
            for (int ic = 0; ic < a->C; ic++) acc += x[(size_t)ic * in_hw + p] * a->Wt[((size_t)ic * a->Cout + oc) * taps + t];
            col[j * in_hw + p] = acc;
         }
      }
      for (size_t i = 0; i < (size_t)a->Cout * out_hw; i++) y[i] = 0.f;
      const float *c = col;
      for (int oc = 0; oc < a->Cout; oc++) {
         float *im = y + (size_t)oc * out_hw;
         for (int r = 0; r < a->kh; r++)
            for (int s = 0; s < a->kw; s++) {
               int row = -a->pad_h + r * a->dil_h;
               for (int ih = 0; ih < a->H; ih++, row += a->stride_h) {
                  if (row < 0 || row >= a->oH) {
                     c += a->W;
                     continue;
                  }
                  int colx = -a->pad_w + s * a->dil_w;
                  for (int iw = 0; iw < a->W; iw++, colx += a->stride_w, c++)
                     if (colx >= 0 && colx < a->oW) im[(size_t)row * a->oW + colx] += *c;
               }
            }
      }
      if (a->bias)
         for (int oc = 0; oc < a->Cout; oc++)
            for (size_t i = 0; i < out_hw; i++) y[(size_t)oc * out_hw + i] += a->bias[oc];
   }
   free(col);
}
ORACLE_API void oracle_conv_transpose2d_f32(int N, int C, int H, int W, int Cout, int kh, int kw, int pad_h, int pad_w,
                                            int stride_h, int stride_w, int dil_h, int dil_w, int outpad_h, int outpad_w,
                                            const float *X, const float *Wt, const float *bias, float *Y)
{
   convtr_args a = {N, C, H, W, Cout, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
                    stride_h * (H - 1) + dil_h * (kh - 1) + 1 + outpad_h - 2 * pad_h,
                    stride_w * (W - 1) + dil_w * (kw - 1) + 1 + outpad_w - 2 * pad_w, X, Wt, bias, Y};
   oracle_parallel_for(N, conv_transpose2d_images, &a);
}

/* Einsum of two operands, the general form the reference emits as nested loops over the output labels and then the
 * summation labels (ROperator_Einsum.hxx:200-274; the matrix-product shapes it hands to sgemm_, :275-332, are the same
 * sum): Y[out] = sum over the non-output labels of A[...] * B[...]. Labels are given by their extents (first the n_out
 * output labels in output order, then the n_sum summed ones) and by the element stride each has in A and in B (0 when the
 * operand does not carry the label). Double accumulator, rounded once. */
ORACLE_API void oracle_einsum_f32(int n_out, int n_sum, const long long *extent, const long long *a_stride, const long long *b_stride,
                                  const float *A, const float *B, float *Y)
{
   long long out_total = 1, sum_total = 1;
   for (int i = 0; i < n_out; i++) out_total *= extent[i];
   for (int i = 0; i < n_sum; i++) sum_total *= extent[n_out + i];
   for (long long o = 0; o < out_total; o++) {
      long long rem = o, a0 = 0, b0 = 0;
      for (int i = n_out - 1; i >= 0; i--) {
         const long long idx = rem % extent[i];
         rem /= extent[i];
         a0 += idx * a_stride[i];
         b0 += idx * b_stride[i];
      }
      double acc = 0.0;
      for (long long q = 0; q < sum_total; q++) {
         long long r2 = q, a = a0, b = b0;
         for (int i = n_sum - 1; i >= 0; i--) {
            const long long idx = r2 % extent[n_out + i];
            r2 /= extent[n_out + i];
            a += idx * a_stride[n_out + i];
            b += idx * b_stride[n_out + i];
         }
         acc += (double)A[a] * (double)B[b];
      }
      Y[o] = (float)acc;
   }
}

/* ROperator_Relu.hxx:54-66 */
ORACLE_API void oracle_relu_f32(const float *X, size_t n, float *Y)
{
   for (size_t i = 0; i < n; i++) Y[i] = (X[i] > 0) ? X[i] : 0;
}

/* 2-D pooling as emitted by ROperator_Pool.hxx:371-416. NC = N*C planes of [H,W].
 * pads = (h_begin, w_begin, h_end, w_end) as in ONNX and in the reference's shape inference
 * (ROperator_Pool.hxx:172-189). The reference's loop bounds read the same vector as
 * (h_begin, h_end, w_begin, w_end) (ROperator_Pool.hxx:283-289); the two readings agree whenever
 * the four pads are equal -- the only padded case the reference handles without writing past its
 * output tensor -- and the shape-inference reading is the one restated here.
 * mode 0 = max (init -INFINITY, out-of-range taps skipped), 1 = average. */
ORACLE_API void oracle_pool2d_f32(int mode, size_t NC, int H, int W, int kh, int kw, const int *pads, int sh, int sw,
                                  int count_include_pad, const float *X, float *Y)
{
   const int hmin = -pads[0], hmax = H + pads[2] - kh + 1;
   const int wmin = -pads[1], wmax = W + pads[3] - kw + 1;
   const int do_pad = pads[0] || pads[1] || pads[2] || pads[3];
   size_t out = 0;
   for (size_t n = 0; n < NC; n++) {
      const float *x = X + n * (size_t)H * W;
      for (int i = hmin; i < hmax; i += sh) {
         for (int j = wmin; j < wmax; j += sw) {
            float value = (mode == 0) ? -INFINITY : 0.0f;
            int nsum = (count_include_pad || !do_pad) ? kh * kw : 0;
            for (int l = i; l < i + kh; l++) {
               if (l < 0 || l >= H) continue;
               for (int m = j; m < j + kw; m++) {
                  if (m < 0 || m >= W) continue;
                  float v = x[(size_t)l * W + m];
                  if (mode == 0) {
                     if (v > value) value = v;
                  } else {
                     value += v;
                     if (!count_include_pad && do_pad) nsum++;
                  }
               }
            }
            if (mode == 1) value /= (float)nsum;
            Y[out++] = value;
         }
      }
   }
}

/* Softmax along one axis as emitted by ROperator_Softmax.hxx:53-184: the tensor is viewed as
 * [outer, axis_len, inner]; per (outer, inner) line: max, exp(x - max) accumulated in fp32, divide. */
ORACLE_API void oracle_softmax_f32(size_t outer, size_t axis_len, size_t inner, const float *X, float *Y)
{
   for (size_t o = 0; o < outer; o++) {
      for (size_t in = 0; in < inner; in++) {
         const float *x = X + o * axis_len * inner + in;
         float *y = Y + o * axis_len * inner + in;
         float vmax = x[0];
         for (size_t i = 1; i < axis_len; i++)
            if (x[i * inner] > vmax) vmax = x[i * inner];
         float sum = 0.f;
         for (size_t i = 0; i < axis_len; i++) {
            y[i * inner] = expf(x[i * inner] - vmax);
            sum += y[i * inner];
         }
         for (size_t i = 0; i < axis_len; i++) y[i * inner] /= sum;
      }
   }
}

/* Unary operators with the expressions of the emitted code (ROperator_Sigmoid.hxx:59,
 * ROperator_Tanh.hxx:60, ROperator_LeakyRelu.hxx:73, ROperator_Selu.hxx:59 -- double constants --,
 * ROperator_Elu.hxx:71 -- `alpha * exp(x) - 1` as written there --, ROperator_BasicUnary.hxx).
 * op: 0 Sigmoid, 1 Tanh, 2 LeakyRelu, 3 Selu, 4 Elu, 5 Neg, 6 Exp, 7 Log, 8 Sqrt, 9 Reciprocal, 10 Abs,
 * 11 Erf (ROperator_Erf.hxx:58), 12 Swish (ROperator_Swish.hxx:59), 13 Cos, 14 Sin. */
ORACLE_API void oracle_unary_f32(int op, float alpha, const float *X, float *Y, size_t n)
{
   for (size_t i = 0; i < n; i++) {
      const float x = X[i];
      float y;
      switch (op) {
      case 0: y = 1 / (1 + expf(-x)); break;
      case 1: y = tanhf(x); break;
      case 2: y = (x >= 0) ? x : alpha * x; break;
      case 3: {
         const double pos = (0.0f > x) ? 0.0f : x;
         const double t = 1.6732632423543772848170429916717 * (expf(x) - 1);
         y = (float)(1.0507009873554804934193349852946 * (pos + (0.0 < t ? 0.0 : t)));
         break;
      }
      case 4: y = (x >= 0) ? x : alpha * expf(x) - 1; break;
      case 5: y = -x; break;
      case 6: y = expf(x); break;
      case 7: y = logf(x); break;
      case 8: y = sqrtf(x); break;
      case 9: y = 1 / x; break;
      case 11: y = erff(x); break;
      case 12: y = x / (1 + expf(-x)); break;
      case 13: y = cosf(x); break;
      case 14: y = sinf(x); break;
      default: y = fabsf(x); break;
      }
      Y[i] = y;
   }
}

/* Binary operators with broadcasting (ROperator_BasicBinary.hxx:18-43): the output has `shape`
 * (rank 4); an operand's element stride is 0 along a broadcast dimension. op: 0 +, 1 -, 2 *, 3 /. */
ORACLE_API void oracle_binary_f32(int op, const int64_t *shape, const int64_t *a_stride, const int64_t *b_stride, const float *A,
                                  const float *B, float *Y)
{
   size_t i = 0;
   for (int64_t c0 = 0; c0 < shape[0]; c0++)
      for (int64_t c1 = 0; c1 < shape[1]; c1++)
         for (int64_t c2 = 0; c2 < shape[2]; c2++)
            for (int64_t c3 = 0; c3 < shape[3]; c3++, i++) {
               const float a = A[c0 * a_stride[0] + c1 * a_stride[1] + c2 * a_stride[2] + c3 * a_stride[3]];
               const float b = B[c0 * b_stride[0] + c1 * b_stride[1] + c2 * b_stride[2] + c3 * b_stride[3]];
               Y[i] = op == 0 ? a + b : (op == 1 ? a - b : (op == 2 ? a * b : a / b));
            }
}

/* BatchNormalization as emitted (ROperator_BatchNormalization.hxx:163-168, 200-226): at Initialize
 * the scale becomes scale * (1. / sqrt(var + epsilon)); at run time y = x, y -= mean, y *= scale,
 * y += bias, optional Relu. X is NCHW viewed as [N, C, HW]. */
ORACLE_API void oracle_batchnorm_f32(int N, int C_, int HW, float epsilon, int relu, const float *X, const float *scale,
                                     const float *bias, const float *mean, const float *var, float *Y)
{
   for (int c = 0; c < C_; c++) {
      float v = var[c] + epsilon;
      float inv = (float)(1. / sqrt(v));
      float s = scale[c] * inv;
      for (int n = 0; n < N; n++) {
         const float *x = X + ((size_t)n * C_ + c) * HW;
         float *y = Y + ((size_t)n * C_ + c) * HW;
         for (int i = 0; i < HW; i++) {
            float t = x[i];
            t = t + (-1.f) * mean[c];
            t *= s;
            t = t + 1.f * bias[c];
            y[i] = relu ? ((t > 0) ? t : 0) : t;
         }
      }
   }
}

/* ------------------------------------------------------------------------------------------ */
/* int8 (ONNX operator definitions; parity unpinned by the reference)                          */
/* ------------------------------------------------------------------------------------------ */

static inline int32_t requant(int32_t acc, float mult, int32_t y_zp, int32_t qmin, int32_t qmax)
{
   float r = nearbyintf((float)acc * mult); /* round half to even under the default rounding mode */
   float lo = (float)(qmin - y_zp), hi = (float)(qmax - y_zp);
   r = r < lo ? lo : (r > hi ? hi : r);
   return (int32_t)r + y_zp;
}

/* The requantisation multiplier, computed in this fixed order in fp32. */
ORACLE_API void oracle_requant_multiplier(float a_scale, const float *w_scale, int n, float y_scale, float *mult)
{
   for (int i = 0; i < n; i++) {
      float t = a_scale * w_scale[i];
      mult[i] = t / y_scale;
   }
}

/* QuantizeLinear to uint8: y = saturate(rne(x / scale) + zp). */
typedef struct { const float *X; float scale; int32_t zp; uint8_t *Y; } quant_args;
static void quantize_u8_range(long begin, long end, void *ctx)
{
   const quant_args *q = (const quant_args *)ctx;
   for (long i = begin; i < end; i++) {
      float r = nearbyintf(q->X[i] / q->scale);
      float lo = (float)(0 - q->zp), hi = (float)(255 - q->zp);
      r = r < lo ? lo : (r > hi ? hi : r);
      q->Y[i] = (uint8_t)((int32_t)r + q->zp);
   }
}
ORACLE_API void oracle_quantize_u8(const float *X, size_t n, float scale, int32_t zp, uint8_t *Y)
{
   quant_args q = {X, scale, zp, Y};
   oracle_parallel_for((long)n, quantize_u8_range, &q);
}

/* DequantizeLinear from uint8: y = (x - zp) * scale. */
ORACLE_API void oracle_dequantize_u8(const uint8_t *X, size_t n, float scale, int32_t zp, float *Y)
{
   for (size_t i = 0; i < n; i++) Y[i] = (float)((int32_t)X[i] - zp) * scale;
}

/* QLinearMatMul: A uint8 [M,K] (scale a_scale, zero point a_zp) times W int8 stored [N,K] when
 * w_is_nk, else [K,N] (per-output-channel scales w_scale[N], zero point 0), optional int32 bias[N],
 * optional Relu on the quantised value (max(q, y_zp)), output uint8 [M,N]. */
typedef struct {
   int M, N, K, relu;
   int32_t a_zp, y_zp;
   const uint8_t *A;
   const int8_t *Wnk;
   const float *mult;
   const int32_t *bias;
   uint8_t *Y;
   int32_t *Acc;
} qmm_args;
static void qlinear_matmul_rows(long begin, long end, void *ctx)
{
   const qmm_args *q = (const qmm_args *)ctx;
   for (long m = begin; m < end; m++) {
      const uint8_t *a = q->A + (size_t)m * q->K;
      for (int n = 0; n < q->N; n++) {
         const int8_t *w = q->Wnk + (size_t)n * q->K;
         int32_t acc = 0;
         for (int k = 0; k < q->K; k++) acc += ((int32_t)a[k] - q->a_zp) * (int32_t)w[k];
         if (q->Acc) {
            q->Acc[(size_t)m * q->N + n] = acc;
            continue;
         }
         if (q->bias) acc += q->bias[n];
         int32_t v = requant(acc, q->mult[n], q->y_zp, 0, 255);
         if (q->relu && v < q->y_zp) v = q->y_zp;
         q->Y[(size_t)m * q->N + n] = (uint8_t)v;
      }
   }
}
ORACLE_API void oracle_qlinear_matmul(int M, int N, int K, const uint8_t *A, float a_scale, int32_t a_zp,
                                      const int8_t *Wt, int w_is_nk, const float *w_scale, const int32_t *bias,
                                      float y_scale, int32_t y_zp, int relu, uint8_t *Y)
{
   float *mult = (float *)malloc(sizeof(float) * N);
   oracle_requant_multiplier(a_scale, w_scale, N, y_scale, mult);
   int8_t *wnk = NULL;
   if (!w_is_nk) { /* transpose once so the inner loop is contiguous */
      wnk = (int8_t *)malloc((size_t)N * K);
      for (int k = 0; k < K; k++)
         for (int n = 0; n < N; n++) wnk[(size_t)n * K + k] = Wt[(size_t)k * N + n];
      Wt = wnk;
   }
   qmm_args q = {M, N, K, relu, a_zp, y_zp, A, Wt, mult, bias, Y, NULL};
   oracle_parallel_for(M, qlinear_matmul_rows, &q);
   free(mult);
   free(wnk);
}

/* Same contraction but the int32 accumulator is dequantised to float: y = acc * (a_scale*w_scale[n])
 * (QLinearMatMul followed by DequantizeLinear collapses to this only when no requantisation happens
 * in between; used for the final layer of the int8 models when they end in DequantizeLinear after
 * a uint8 output, see oracle_dequantize_u8 -- kept for tests of the raw accumulator). */
ORACLE_API void oracle_matmul_u8i8_acc(int M, int N, int K, const uint8_t *A, int32_t a_zp, const int8_t *Wnk,
                                       int32_t *Acc)
{
   qmm_args q = {M, N, K, 0, a_zp, 0, A, Wnk, NULL, NULL, NULL, Acc};
   oracle_parallel_for(M, qlinear_matmul_rows, &q);
}

/* QLinearConv 2-D, NCHW uint8 activations, int8 weights [Cout, C, kh, kw] with per-Cout scales and
 * zero point 0, padding taps contribute (x_zp - x_zp) = 0, optional int32 bias, optional Relu
 * (max(q, y_zp)), group 1, dilation 1. Output uint8 [N,Cout,oH,oW]. */
typedef struct {
   int N, C, H, W, Cout, kh, kw, pad_h, pad_w, stride_h, stride_w, relu;
   int32_t x_zp, y_zp;
   const uint8_t *X;
   const int8_t *Wt;
   const float *mult;
   const int32_t *bias;
   uint8_t *Y;
} qconv_args;
static void qlinear_conv2d_images(long begin, long end, void *ctx)
{
   const qconv_args *a = (const qconv_args *)ctx;
   const int C = a->C, H = a->H, W = a->W, Cout = a->Cout, kh = a->kh, kw = a->kw;
   const int oH = (H + 2 * a->pad_h - kh) / a->stride_h + 1;
   const int oW = (W + 2 * a->pad_w - kw) / a->stride_w + 1;
   for (long n = begin; n < end; n++) {
      for (int oc = 0; oc < Cout; oc++) {
         for (int oh = 0; oh < oH; oh++) {
            for (int ow = 0; ow < oW; ow++) {
               int32_t acc = 0;
               for (int c = 0; c < C; c++) {
                  for (int r = 0; r < kh; r++) {
                     int ih = oh * a->stride_h - a->pad_h + r;
                     if (ih < 0 || ih >= H) continue;
                     for (int s = 0; s < kw; s++) {
                        int iw = ow * a->stride_w - a->pad_w + s;
                        if (iw < 0 || iw >= W) continue;
                        int32_t xv = (int32_t)a->X[(((size_t)n * C + c) * H + ih) * W + iw] - a->x_zp;
                        acc += xv * (int32_t)a->Wt[(((size_t)oc * C + c) * kh + r) * kw + s];
                     }
                  }
               }
               if (a->bias) acc += a->bias[oc];
               int32_t q = requant(acc, a->mult[oc], a->y_zp, 0, 255);
               if (a->relu && q < a->y_zp) q = a->y_zp;
               a->Y[(((size_t)n * Cout + oc) * oH + oh) * oW + ow] = (uint8_t)q;
            }
         }
      }
   }
}
ORACLE_API void oracle_qlinear_conv2d(int N, int C, int H, int W, int Cout, int kh, int kw, int pad_h, int pad_w,
                                      int stride_h, int stride_w, const uint8_t *X, float x_scale, int32_t x_zp,
                                      const int8_t *Wt, const float *w_scale, const int32_t *bias, float y_scale,
                                      int32_t y_zp, int relu, uint8_t *Y)
{
   float *mult = (float *)malloc(sizeof(float) * Cout);
   oracle_requant_multiplier(x_scale, w_scale, Cout, y_scale, mult);
   qconv_args a = {N, C, H, W, Cout, kh, kw, pad_h, pad_w, stride_h, stride_w, relu, x_zp, y_zp, X, Wt, mult, bias, Y};
   oracle_parallel_for(N, qlinear_conv2d_images, &a);
   free(mult);
}

/* MaxPool on uint8, same window rule as oracle_pool2d_f32 with zero pads (integer max). */
ORACLE_API void oracle_maxpool2d_u8(size_t NC, int H, int W, int kh, int kw, int sh, int sw, const uint8_t *X,
                                    uint8_t *Y)
{
   size_t out = 0;
   for (size_t n = 0; n < NC; n++)
      for (int i = 0; i < H - kh + 1; i += sh)
         for (int j = 0; j < W - kw + 1; j += sw) {
            uint8_t v = 0;
            for (int l = i; l < i + kh; l++)
               for (int m = j; m < j + kw; m++) {
                  uint8_t x = X[n * (size_t)H * W + (size_t)l * W + m];
                  if (x > v) v = x;
               }
            Y[out++] = v;
         }
}

/* ------------------------------------------------------------------------------------------ */
/* FP8 E4M3 (the "FN" encoding: no infinities, max finite 448, NaN = S.1111.111) and bf16       */
/* ------------------------------------------------------------------------------------------ */

ORACLE_API float oracle_e4m3_to_f32(uint8_t v)
{
   int s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
   float r;
   if (e == 0xF && m == 7) return NAN;
   if (e == 0) r = ldexpf((float)m, -9);            /* subnormal: m/8 * 2^-6 */
   else r = ldexpf(1.0f + (float)m / 8.0f, e - 7);
   return s ? -r : r;
}

/* float -> E4M3, round to nearest even, saturating to +-448 (NaN stays NaN). */
ORACLE_API uint8_t oracle_f32_to_e4m3(float x)
{
   if (x != x) return 0x7F;
   uint8_t sign = signbit(x) ? 0x80 : 0;
   float a = fabsf(x);
   if (a >= 448.0f) return sign | 0x7E; /* anything above the max finite value saturates */
   if (a < ldexpf(1.0f, -10)) return sign; /* below half the smallest subnormal (2^-9): 0; tie -> even (0) */
   int e;
   (void)frexpf(a, &e); /* a = f * 2^e with f in [0.5,1), i.e. a = (2f) * 2^(e-1) */
   int exp = e - 1;
   if (exp < -6) { /* subnormal range: spacing 2^-9 */
      int m = (int)nearbyintf(ldexpf(a, 9));
      if (m == 8) return sign | 0x08; /* rounds up to the smallest normal */
      return sign | (uint8_t)m;
   }
   int m = (int)nearbyintf(ldexpf(a, 3 - exp)); /* a in units of the spacing at this exponent: [8,16] */
   if (m == 16) {
      m = 8;
      exp += 1;
   }
   int biased = exp + 7;
   if (biased > 15 || (biased == 15 && (m - 8) == 7)) return sign | 0x7E;
   return sign | (uint8_t)(biased << 3) | (uint8_t)(m - 8);
}

static void quantize_e4m3_range(long begin, long end, void *ctx)
{
   const quant_args *q = (const quant_args *)ctx;
   for (long i = begin; i < end; i++) q->Y[i] = oracle_f32_to_e4m3(q->X[i] / q->scale);
}
ORACLE_API void oracle_quantize_e4m3(const float *X, size_t n, float scale, uint8_t *Y)
{
   quant_args q = {X, scale, 0, Y};
   oracle_parallel_for((long)n, quantize_e4m3_range, &q);
}

ORACLE_API uint16_t oracle_f32_to_bf16(float x)
{
   uint32_t u;
   memcpy(&u, &x, 4);
   if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40); /* quiet NaN */
   u += 0x7FFFu + ((u >> 16) & 1u); /* round to nearest even */
   return (uint16_t)(u >> 16);
}

ORACLE_API float oracle_bf16_to_f32(uint16_t v)
{
   uint32_t u = (uint32_t)v << 16;
   float f;
   memcpy(&f, &u, 4);
   return f;
}

/* FP8 Gemm layer: A codes [M,K] (scale a_scale), W codes [N,K] (scale w_scale); the contraction is
 * evaluated on the DEQUANTISED fp32 values with a double accumulator (the "fp32-dequantised
 * reference" the FP8 tolerance is stated against), then * (a_scale*w_scale) + bias, Relu, rounded
 * to bf16 (returned as raw bf16 bits). */
typedef struct {
   int M, N, K, relu;
   const uint8_t *A, *Wnk;
   float scale;
   const float *bias, *lut;
   uint16_t *Y;
} fp8_args;
static void gemm_e4m3_rows(long begin, long end, void *ctx)
{
   const fp8_args *g = (const fp8_args *)ctx;
   for (long m = begin; m < end; m++)
      for (int n = 0; n < g->N; n++) {
         double acc = 0.0;
         for (int k = 0; k < g->K; k++)
            acc += (double)g->lut[g->A[(size_t)m * g->K + k]] * (double)g->lut[g->Wnk[(size_t)n * g->K + k]];
         float y = (float)acc * g->scale;
         if (g->bias) y = y + g->bias[n];
         if (g->relu) y = (y > 0) ? y : 0;
         g->Y[(size_t)m * g->N + n] = oracle_f32_to_bf16(y);
      }
}
ORACLE_API void oracle_gemm_e4m3(int M, int N, int K, const uint8_t *A, float a_scale, const uint8_t *Wnk,
                                 float w_scale, const float *bias, int relu, uint16_t *Ybf16)
{
   float lut[256];
   for (int i = 0; i < 256; i++) lut[i] = oracle_e4m3_to_f32((uint8_t)i);
   fp8_args g = {M, N, K, relu, A, Wnk, a_scale * w_scale, bias, lut, Ybf16};
   oracle_parallel_for(M, gemm_e4m3_rows, &g);
}
