// Memory-bound operators between the contractions: Relu, pooling, softmax, layout changes,
// (de)quantisation and casts. One read and one write per element, 128-bit accesses where the
// pointers allow it, grids sized as a multiple of the SM count.
#include "common.cuh"

#include <cuda_fp8.h>
#include <cfloat>

using namespace sofie;

namespace {

constexpr int kThreads = 256;

inline int grid_for(size_t work_items, int per_block = kThreads, int waves = 8)
{
   size_t blocks = ceil_div<size_t>(work_items, per_block);
   size_t cap = size_t(kNumSMs) * waves;
   if (blocks > cap) blocks = cap;
   if (blocks == 0) blocks = 1;
   return (int)blocks;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------- relu ---------------------------
__global__ void relu_f32_vec4(const float4 *__restrict__ X, float4 *__restrict__ Y, size_t n4)
{
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
      float4 v = X[i];
      v.x = relu_ref(v.x);
      v.y = relu_ref(v.y);
      v.z = relu_ref(v.z);
      v.w = relu_ref(v.w);
      Y[i] = v;
   }
}
__global__ void relu_f32_scalar(const float *__restrict__ X, float *__restrict__ Y, size_t begin, size_t n)
{
   for (size_t i = begin + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
      Y[i] = relu_ref(X[i]);
}

// ---------------------------------------------------------------- pooling ------------------------
template <bool NHWC>
__global__ void pool2d_f32_kernel(sofie_pool2d_desc d, int oH, int oW, const float *__restrict__ X,
                                  float *__restrict__ Y)
{
   const size_t total = (size_t)d.N * d.C * oH * oW;
   const bool do_pad = d.pads[0] || d.pads[1] || d.pads[2] || d.pads[3];
   for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
        idx += (size_t)gridDim.x * blockDim.x) {
      int n, c, oh, ow;
      size_t t = idx;
      if (NHWC) {
         c = t % d.C; t /= d.C;
         ow = t % oW; t /= oW;
         oh = t % oH; n = t / oH;
      } else {
         ow = t % oW; t /= oW;
         oh = t % oH; t /= oH;
         c = t % d.C; n = t / d.C;
      }
      const int i0 = -d.pads[0] + oh * d.stride_h, j0 = -d.pads[1] + ow * d.stride_w;
      float value = d.mode == 0 ? -INFINITY : 0.f;
      int nsum = (d.count_include_pad || !do_pad) ? d.kH * d.kW : 0;
      for (int l = i0; l < i0 + d.kH; l++) {
         if (l < 0 || l >= d.H) continue;
         for (int m = j0; m < j0 + d.kW; m++) {
            if (m < 0 || m >= d.W) continue;
            size_t xi = NHWC ? (((size_t)n * d.H + l) * d.W + m) * d.C + c : (((size_t)n * d.C + c) * d.H + l) * d.W + m;
            float v = X[xi];
            if (d.mode == 0) {
               if (v > value) value = v;
            } else {
               value += v;
               if (!d.count_include_pad && do_pad) nsum++;
            }
         }
      }
      if (d.mode == 1) value /= (float)nsum;
      Y[idx] = value;
   }
}

// The common window: 2 x 2, stride 2, no padding (what every configuration of this path pools with). NCHW: a thread
// reads 16 bytes of two input rows and writes two outputs; NHWC: a thread reads four channels of the four pixels of a
// window as 16-byte loads and writes 16 bytes. 32-bit index arithmetic (the launcher checks the sizes).
template <bool AVG>
__global__ void pool2x2_f32_nchw_kernel(const float *__restrict__ X, float *__restrict__ Y, unsigned planes_rows /* N*C*oH */, int W)
{
   const unsigned qw = (unsigned)W >> 2; // float4 per input row = pairs of outputs per output row
   const unsigned total = planes_rows * qw;
   for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
      const unsigned row = idx / qw, q = idx - row * qw;
      const float4 a = __ldg(reinterpret_cast<const float4 *>(X + (size_t)row * 2 * W) + q);
      const float4 b = __ldg(reinterpret_cast<const float4 *>(X + ((size_t)row * 2 + 1) * W) + q);
      float2 o;
      if (AVG) {
         o.x = (((a.x + a.y) + b.x) + b.y) / 4.f; // the window's elements in the order the reference adds them
         o.y = (((a.z + a.w) + b.z) + b.w) / 4.f;
      } else {
         o.x = -INFINITY;
         if (a.x > o.x) o.x = a.x;
         if (a.y > o.x) o.x = a.y;
         if (b.x > o.x) o.x = b.x;
         if (b.y > o.x) o.x = b.y;
         o.y = -INFINITY;
         if (a.z > o.y) o.y = a.z;
         if (a.w > o.y) o.y = a.w;
         if (b.z > o.y) o.y = b.z;
         if (b.w > o.y) o.y = b.w;
      }
      reinterpret_cast<float2 *>(Y + (size_t)row * (W >> 1))[q] = o;
   }
}
template <bool AVG>
__global__ void pool2x2_f32_nhwc_kernel(const float *__restrict__ X, float *__restrict__ Y, unsigned rows /* N*oH */, int oW, int C)
{
   const unsigned c4 = (unsigned)C >> 2;
   const unsigned total = rows * (unsigned)oW * c4;
   for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
      const unsigned pix = idx / c4, c = idx - pix * c4;
      const unsigned row = pix / (unsigned)oW, ow = pix - row * (unsigned)oW;
      const float4 *p = reinterpret_cast<const float4 *>(X + ((size_t)row * 2 * (2 * oW) + 2 * ow) * C) + c;
      const float4 v00 = __ldg(p), v01 = __ldg(p + c4), v10 = __ldg(p + (size_t)2 * oW * c4), v11 = __ldg(p + (size_t)2 * oW * c4 + c4);
      float4 o;
      auto one = [](float a, float b, float c, float d) {
         if (AVG) return (((a + b) + c) + d) / 4.f;
         float m = -INFINITY;
         if (a > m) m = a;
         if (b > m) m = b;
         if (c > m) m = c;
         if (d > m) m = d;
         return m;
      };
      o.x = one(v00.x, v01.x, v10.x, v11.x);
      o.y = one(v00.y, v01.y, v10.y, v11.y);
      o.z = one(v00.z, v01.z, v10.z, v11.z);
      o.w = one(v00.w, v01.w, v10.w, v11.w);
      reinterpret_cast<float4 *>(Y + (size_t)pix * C)[c] = o;
   }
}

template <bool NHWC>
__global__ void maxpool2d_u8_kernel(int N, int C, int H, int W, int kH, int kW, int sh, int sw, int oH, int oW,
                                    const uint8_t *__restrict__ X, uint8_t *__restrict__ Y)
{
   const size_t total = (size_t)N * C * oH * oW;
   for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
        idx += (size_t)gridDim.x * blockDim.x) {
      int n, c, oh, ow;
      size_t t = idx;
      if (NHWC) {
         c = t % C; t /= C;
         ow = t % oW; t /= oW;
         oh = t % oH; n = t / oH;
      } else {
         ow = t % oW; t /= oW;
         oh = t % oH; t /= oH;
         c = t % C; n = t / C;
      }
      unsigned v = 0;
      for (int l = oh * sh; l < oh * sh + kH; l++)
         for (int m = ow * sw; m < ow * sw + kW; m++) {
            size_t xi = NHWC ? (((size_t)n * H + l) * W + m) * C + c : (((size_t)n * C + c) * H + l) * W + m;
            v = max(v, (unsigned)X[xi]);
         }
      Y[idx] = (uint8_t)v;
   }
}

// ---------------------------------------------------------------- softmax ------------------------
// inner == 1: one warp per row, values kept in registers when the row is short, else re-read.
__global__ void softmax_rows_kernel(const float *__restrict__ X, float *__restrict__ Y, size_t rows, size_t len)
{
   const int lane = threadIdx.x & 31;
   const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
   const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
   for (size_t r = warp; r < rows; r += nwarps) {
      const float *x = X + r * len;
      float *y = Y + r * len;
      float vmax = -INFINITY;
      for (size_t i = lane; i < len; i += 32) vmax = fmaxf(vmax, x[i]);
      for (int o = 16; o; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
      float sum = 0.f;
      for (size_t i = lane; i < len; i += 32) {
         float e = expf(x[i] - vmax);
         y[i] = e;
         sum += e;
      }
      for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      for (size_t i = lane; i < len; i += 32) y[i] = y[i] / sum;
   }
}
// inner == 1, rows of up to 32 * 4 * V4 values that are multiples of 4 long and 16-byte aligned: one warp per row, the
// row read ONCE into registers (16-byte loads), written once.
template <int V4>
__global__ void softmax_rows_reg_kernel(const float *__restrict__ X, float *__restrict__ Y, size_t rows, int len4)
{
   const int lane = threadIdx.x & 31;
   const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
   const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
   for (size_t r = warp; r < rows; r += nwarps) {
      const float4 *x = reinterpret_cast<const float4 *>(X) + r * len4;
      float4 *y = reinterpret_cast<float4 *>(Y) + r * len4;
      float4 v[V4];
      float vmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < V4; i++) {
         const int k = lane + 32 * i;
         if (k < len4) {
            v[i] = __ldg(x + k);
            vmax = fmaxf(vmax, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
         }
      }
      for (int o = 16; o; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < V4; i++) {
         if (lane + 32 * i < len4) {
            v[i].x = expf(v[i].x - vmax);
            v[i].y = expf(v[i].y - vmax);
            v[i].z = expf(v[i].z - vmax);
            v[i].w = expf(v[i].w - vmax);
            sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
         }
      }
      for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
      for (int i = 0; i < V4; i++) {
         const int k = lane + 32 * i;
         if (k < len4) y[k] = make_float4(v[i].x / sum, v[i].y / sum, v[i].z / sum, v[i].w / sum);
      }
   }
}
// inner == 1, rows of at most 32 values (class scores): a block takes 256 consecutive rows, copies them into shared memory
// with coalesced loads (row pitch padded to an odd number of words), one thread works on one row, and the block copies
// the results out coalesced. No division in the copy loops: row and column advance incrementally.
constexpr int kSoftmaxShortRows = 256, kSoftmaxShortMax = 32;
__global__ void __launch_bounds__(kSoftmaxShortRows) softmax_rows_short_kernel(const float *__restrict__ X, float *__restrict__ Y, size_t rows, int len)
{
   __shared__ float s_v[kSoftmaxShortRows * (kSoftmaxShortMax + 1)];
   const int pitch = len | 1;
   const int t = threadIdx.x;
   const int step_row = kSoftmaxShortRows / len, step_col = kSoftmaxShortRows - step_row * len;
   for (size_t r0 = (size_t)blockIdx.x * kSoftmaxShortRows; r0 < rows; r0 += (size_t)gridDim.x * kSoftmaxShortRows) {
      const int nrows = rows - r0 < (size_t)kSoftmaxShortRows ? (int)(rows - r0) : kSoftmaxShortRows;
      const int total = nrows * len;
      const float *x = X + r0 * len;
      float *y = Y + r0 * len;
      int row = t / len, col = t - row * len;
      for (int i = t; i < total; i += kSoftmaxShortRows) {
         s_v[row * pitch + col] = __ldg(x + i);
         row += step_row;
         col += step_col;
         if (col >= len) {
            col -= len;
            row++;
         }
      }
      __syncthreads();
      if (t < nrows) {
         float *v = s_v + t * pitch;
         float vmax = -INFINITY;
         for (int i = 0; i < len; i++) vmax = fmaxf(vmax, v[i]);
         float sum = 0.f;
         for (int i = 0; i < len; i++) {
            const float e = expf(v[i] - vmax);
            v[i] = e;
            sum += e;
         }
         for (int i = 0; i < len; i++) v[i] = v[i] / sum;
      }
      __syncthreads();
      row = t / len;
      col = t - row * len;
      for (int i = t; i < total; i += kSoftmaxShortRows) {
         y[i] = s_v[row * pitch + col];
         row += step_row;
         col += step_col;
         if (col >= len) {
            col -= len;
            row++;
         }
      }
      __syncthreads();
   }
}

// inner > 1: one thread per (outer, inner) line, strided walk; neighbouring threads touch
// neighbouring addresses, so the accesses stay coalesced.
__global__ void softmax_strided_kernel(const float *__restrict__ X, float *__restrict__ Y, size_t outer, size_t len,
                                       size_t inner)
{
   const size_t lines = outer * inner;
   for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < lines;
        idx += (size_t)gridDim.x * blockDim.x) {
      size_t o = idx / inner, in = idx % inner;
      const float *x = X + o * len * inner + in;
      float *y = Y + o * len * inner + in;
      float vmax = x[0];
      for (size_t i = 1; i < len; i++) vmax = fmaxf(vmax, x[i * inner]);
      float sum = 0.f;
      for (size_t i = 0; i < len; i++) {
         float e = expf(x[i * inner] - vmax);
         y[i * inner] = e;
         sum += e;
      }
      for (size_t i = 0; i < len; i++) y[i * inner] = y[i * inner] / sum;
   }
}

// ---------------------------------------------------------------- layout -------------------------
// Tiled transpose of the [C, H*W] plane of every image: NCHW -> NHWC is a [C,P] -> [P,C] transpose.
template <typename T>
__global__ void transpose_batched_kernel(const T *__restrict__ in, T *__restrict__ out, int rows, int cols)
{
   __shared__ T tile[32][33];
   const size_t img = blockIdx.z;
   const T *src = in + img * (size_t)rows * cols;
   T *dst = out + img * (size_t)rows * cols;
   int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
   for (int j = threadIdx.y; j < 32; j += blockDim.y) {
      int r = r0 + j, c = c0 + threadIdx.x;
      if (r < rows && c < cols) tile[j][threadIdx.x] = src[(size_t)r * cols + c];
   }
   __syncthreads();
   for (int j = threadIdx.y; j < 32; j += blockDim.y) {
      int c = c0 + j, r = r0 + threadIdx.x;
      if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[threadIdx.x][j];
   }
}

// NCHW <-> NHWC for float images with few channels (a multiple of 4, at most 64): a thread owns a pixel; its reads (NCHW
// side) are coalesced across the warp plane by plane, its NHWC side is C contiguous floats moved as 16-byte words. The
// tiled transpose above wastes half of each 32 x 32 tile when C = 16.
template <bool TO_NHWC>
__global__ void layout_few_channels_f32_kernel(const float *__restrict__ in, float *__restrict__ out, unsigned images, unsigned P, int C)
{
   const size_t total = (size_t)images * P;
   for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
      const size_t n = idx / P, p = idx - n * P;
      if (TO_NHWC) {
         const float *src = in + n * (size_t)C * P + p;
         float4 *dst = reinterpret_cast<float4 *>(out + idx * C);
         for (int c = 0; c < C; c += 4)
            dst[c >> 2] = make_float4(__ldg(src + (size_t)c * P), __ldg(src + (size_t)(c + 1) * P), __ldg(src + (size_t)(c + 2) * P),
                                      __ldg(src + (size_t)(c + 3) * P));
      } else {
         const float4 *src = reinterpret_cast<const float4 *>(in + idx * C);
         float *dst = out + n * (size_t)C * P + p;
         for (int c = 0; c < C; c += 4) {
            const float4 v = __ldg(src + (c >> 2));
            dst[(size_t)c * P] = v.x;
            dst[(size_t)(c + 1) * P] = v.y;
            dst[(size_t)(c + 2) * P] = v.z;
            dst[(size_t)(c + 3) * P] = v.w;
         }
      }
   }
}
template <bool TO_NHWC>
static bool launch_layout_few_channels(cudaStream_t s, const float *in, float *out, int N, int C, int P)
{
   if (C % 4 != 0 || C > 64 || !aligned16(in) || !aligned16(out)) return false;
   layout_few_channels_f32_kernel<TO_NHWC><<<grid_for((size_t)N * P), kThreads, 0, s>>>(in, out, (unsigned)N, (unsigned)P, C);
   return true;
}

template <typename T>
int launch_transpose(cudaStream_t s, const T *in, T *out, int batch, int rows, int cols)
{
   if (batch <= 0 || rows <= 0 || cols <= 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(batch <= 65535 * 64, "batch too large for transpose");
   // gridDim.z is limited to 65535: fold the batch in chunks
   for (int b0 = 0; b0 < batch; b0 += 65535) {
      int nb = batch - b0 < 65535 ? batch - b0 : 65535;
      dim3 grid(ceil_div(cols, 32), ceil_div(rows, 32), nb), block(32, 8);
      transpose_batched_kernel<T><<<grid, block, 0, s>>>(in + (size_t)b0 * rows * cols, out + (size_t)b0 * rows * cols,
                                                         rows, cols);
   }
   SOFIE_LAUNCH_CHECK("transpose_batched_kernel");
   return SOFIE_CUDA_OK;
}

// ---------------------------------------------------------------- (de)quantise, casts ------------
// q = clamp(rint(x / scale)) + zp with the correctly rounded quotient of the ONNX definition. The IEEE division
// costs about 25 instructions and made this kernel arithmetic bound at a third of the HBM bandwidth, so the
// quotient is first taken as x * (1 / scale): that product is within 2 ulp of the true quotient, hence rounds
// to the same integer unless it lies within a few ulp of a half-integer, and only then (about one element in
// ten thousand, and every value too large to have a fraction) the exact division decides.
__device__ __forceinline__ uint8_t quant_u8(float x, float scale, float inv_scale, int zp)
{
   const float t = __fmul_rn(x, inv_scale);
   float r = rintf(t);
   const float to_half = fabsf(fabsf(t - r) - 0.5f); // distance of t from the nearest half-integer
   if (!(to_half > fabsf(t) * 1e-6f)) r = rintf(__fdiv_rn(x, scale)); // also taken for NaN and for an infinite 1 / scale
   r = fminf(fmaxf(r, (float)(0 - zp)), (float)(255 - zp));
   return (uint8_t)(__float2int_rn(r) + zp);
}

// Sixteen elements per thread and step: four 16-byte loads in flight, one 16-byte store.
__global__ void quantize_u8_vec16_kernel(const float *__restrict__ X, uint8_t *__restrict__ Y, size_t n16, float scale, float inv_scale,
                                         int zp)
{
   griddep_launch_dependents();
   griddep_wait(); // X is the previous kernel's output
   const size_t nthreads = (size_t)gridDim.x * blockDim.x;
#pragma unroll 2
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += nthreads) {
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) v[j] = reinterpret_cast<const float4 *>(X)[4 * i + j];
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; j++)
         w[j] = (uint32_t)quant_u8(v[j].x, scale, inv_scale, zp) | ((uint32_t)quant_u8(v[j].y, scale, inv_scale, zp) << 8) |
                ((uint32_t)quant_u8(v[j].z, scale, inv_scale, zp) << 16) | ((uint32_t)quant_u8(v[j].w, scale, inv_scale, zp) << 24);
      reinterpret_cast<uint4 *>(Y)[i] = make_uint4(w[0], w[1], w[2], w[3]);
   }
}

__global__ void quantize_u8_kernel(const float *__restrict__ X, uint8_t *__restrict__ Y, size_t n, float scale, float inv_scale, int zp,
                                   bool vec)
{
   griddep_launch_dependents();
   griddep_wait(); // X is the previous kernel's output
   const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
   size_t n4 = vec ? n / 4 : 0;
   // several independent 16-byte loads in flight per thread
#pragma unroll 4
   for (size_t i = tid; i < n4; i += nthreads) {
      float4 v = reinterpret_cast<const float4 *>(X)[i];
      uchar4 q = make_uchar4(quant_u8(v.x, scale, inv_scale, zp), quant_u8(v.y, scale, inv_scale, zp), quant_u8(v.z, scale, inv_scale, zp),
                             quant_u8(v.w, scale, inv_scale, zp));
      reinterpret_cast<uchar4 *>(Y)[i] = q;
   }
   for (size_t i = n4 * 4 + tid; i < n; i += nthreads) Y[i] = quant_u8(X[i], scale, inv_scale, zp);
}

__global__ void dequantize_u8_kernel(const uint8_t *__restrict__ X, float *__restrict__ Y, size_t n, float scale,
                                     int zp, bool vec)
{
   griddep_launch_dependents();
   griddep_wait(); // X is the previous kernel's output
   const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
   size_t n4 = vec ? n / 4 : 0;
#pragma unroll 4
   for (size_t i = tid; i < n4; i += nthreads) {
      uchar4 q = reinterpret_cast<const uchar4 *>(X)[i];
      float4 v = make_float4(__fmul_rn((float)((int)q.x - zp), scale), __fmul_rn((float)((int)q.y - zp), scale),
                             __fmul_rn((float)((int)q.z - zp), scale), __fmul_rn((float)((int)q.w - zp), scale));
      reinterpret_cast<float4 *>(Y)[i] = v;
   }
   for (size_t i = n4 * 4 + tid; i < n; i += nthreads) Y[i] = __fmul_rn((float)((int)X[i] - zp), scale);
}

__device__ __forceinline__ uint8_t to_e4m3(float x)
{
   return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// Scalar forms: the tail of a tensor and unaligned tensors.
template <typename In>
__global__ void quantize_e4m3_kernel(const In *__restrict__ X, uint8_t *__restrict__ Y, size_t begin, size_t n, float scale_in,
                                     const float *__restrict__ scale_dev)
{
   const float scale = scale_dev ? *scale_dev : scale_in; // a scale computed on the device by an earlier kernel of the stream
   for (size_t i = begin + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
      float x;
      if constexpr (sizeof(In) == 2) x = bf16_to_f32(X[i]);
      else x = X[i];
      Y[i] = to_e4m3(__fdiv_rn(x, scale));
   }
}

// Eight elements per thread and step: 16- or 32-byte loads, one 8-byte store.
template <typename In>
__global__ void quantize_e4m3_vec8_kernel(const In *__restrict__ X, uint8_t *__restrict__ Y, size_t n8, float scale_in,
                                          const float *__restrict__ scale_dev)
{
   const float scale = scale_dev ? *scale_dev : scale_in;
   const size_t nthreads = (size_t)gridDim.x * blockDim.x;
#pragma unroll 2
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += nthreads) {
      float v[8];
      if constexpr (sizeof(In) == 2) {
         const uint4 p = reinterpret_cast<const uint4 *>(X)[i];
         const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
         for (int j = 0; j < 4; j++) {
            v[2 * j] = __uint_as_float(w[j] << 16);
            v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
         }
      } else {
         const float4 a = reinterpret_cast<const float4 *>(X)[2 * i], b = reinterpret_cast<const float4 *>(X)[2 * i + 1];
         v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
         v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      }
      uint32_t out[2];
#pragma unroll
      for (int h = 0; h < 2; h++) {
         uint16_t lo, hi;
         const float d0 = __fdiv_rn(v[4 * h], scale), d1 = __fdiv_rn(v[4 * h + 1], scale);
         const float d2 = __fdiv_rn(v[4 * h + 2], scale), d3 = __fdiv_rn(v[4 * h + 3], scale);
         asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(d1), "f"(d0));
         asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d3), "f"(d2));
         out[h] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      reinterpret_cast<uint2 *>(Y)[i] = make_uint2(out[0], out[1]);
   }
}

__global__ void cast_bf16_f32_kernel(const uint16_t *__restrict__ X, float *__restrict__ Y, size_t begin, size_t n)
{
   for (size_t i = begin + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
      Y[i] = bf16_to_f32(X[i]);
}
__global__ void cast_bf16_f32_vec8_kernel(const uint16_t *__restrict__ X, float *__restrict__ Y, size_t n8)
{
   const size_t nthreads = (size_t)gridDim.x * blockDim.x;
#pragma unroll 2
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += nthreads) {
      const uint4 p = reinterpret_cast<const uint4 *>(X)[i];
      reinterpret_cast<float4 *>(Y)[2 * i] = make_float4(__uint_as_float(p.x << 16), __uint_as_float(p.x & 0xFFFF0000u),
                                                         __uint_as_float(p.y << 16), __uint_as_float(p.y & 0xFFFF0000u));
      reinterpret_cast<float4 *>(Y)[2 * i + 1] = make_float4(__uint_as_float(p.z << 16), __uint_as_float(p.z & 0xFFFF0000u),
                                                             __uint_as_float(p.w << 16), __uint_as_float(p.w & 0xFFFF0000u));
   }
}
__global__ void cast_f32_bf16_kernel(const float *__restrict__ X, uint16_t *__restrict__ Y, size_t n)
{
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
      Y[i] = f32_to_bf16_rne(X[i]);
}

// |x| as an unsigned integer orders like the float for non-NaN values, so atomicMax on the bit
// pattern gives the exact maximum without a second pass.
__global__ void amax_f32_kernel(const float *__restrict__ X, size_t n, unsigned *__restrict__ out)
{
   unsigned m = 0;
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
      unsigned u = __float_as_uint(X[i]) & 0x7FFFFFFFu;
      if (u <= 0x7F800000u) m = max(m, u);
   }
   for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
   if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

// max |x| of bfloat16 values (as float bit patterns, like amax_f32_kernel)
__global__ void amax_bf16_kernel(const uint16_t *__restrict__ X, size_t n, unsigned *__restrict__ out)
{
   unsigned m = 0;
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
      unsigned u = ((unsigned)X[i] << 16) & 0x7FFFFFFFu;
      if (u <= 0x7F800000u) m = max(m, u);
   }
   for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
   if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}
// scale = amax / 448 (the largest E4M3 value), 1 for an all-zero tensor: in place, one thread
__global__ void e4m3_scale_from_amax_kernel(float *amax_to_scale)
{
   const float a = *amax_to_scale;
   *amax_to_scale = a > 0.f ? __fdiv_rn(a, 448.f) : 1.f;
}

template <typename In>
static int launch_quantize_e4m3(cudaStream_t s, const In *X, uint8_t *Y, size_t n, float scale, const float *scale_dev = nullptr)
{
   size_t done = 0;
   if (aligned16(X) && (reinterpret_cast<uintptr_t>(Y) & 7) == 0 && n >= 8) {
      const size_t n8 = n / 8;
      quantize_e4m3_vec8_kernel<In><<<grid_for(n8), kThreads, 0, s>>>(X, Y, n8, scale, scale_dev);
      SOFIE_LAUNCH_CHECK("quantize_e4m3_vec8_kernel");
      done = n8 * 8;
   }
   if (done < n) {
      quantize_e4m3_kernel<In><<<grid_for(n - done), kThreads, 0, s>>>(X, Y, done, n, scale, scale_dev);
      SOFIE_LAUNCH_CHECK("quantize_e4m3_kernel");
   }
   return SOFIE_CUDA_OK;
}

// Dynamic per-tensor quantisation: scale = max|x| / 448 on the device, then the same rounding as the static form.
template <typename In>
static int dynamic_quantize_e4m3(cudaStream_t s, const In *X, uint8_t *Y, size_t n, float *scale_device)
{
   SOFIE_CUDA_TRY(cudaMemsetAsync(scale_device, 0, sizeof(float), s));
   if (n) {
      if constexpr (sizeof(In) == 2) amax_bf16_kernel<<<grid_for(n), kThreads, 0, s>>>(X, n, reinterpret_cast<unsigned *>(scale_device));
      else amax_f32_kernel<<<grid_for(n), kThreads, 0, s>>>(X, n, reinterpret_cast<unsigned *>(scale_device));
      SOFIE_LAUNCH_CHECK("amax kernel");
   }
   e4m3_scale_from_amax_kernel<<<1, 1, 0, s>>>(scale_device);
   SOFIE_LAUNCH_CHECK("e4m3_scale_from_amax_kernel");
   if (n == 0) return SOFIE_CUDA_OK;
   return launch_quantize_e4m3<In>(s, X, Y, n, 1.f, scale_device);
}
} // namespace

extern "C" {

int sofie_cuda_relu_f32(void *stream, const float *X, float *Y, size_t n)
{
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   if (n == 0) return SOFIE_CUDA_OK;
   cudaStream_t s = as_stream(stream);
   size_t done = 0;
   if (aligned16(X) && aligned16(Y) && n >= 4) {
      size_t n4 = n / 4;
      relu_f32_vec4<<<grid_for(n4), kThreads, 0, s>>>(reinterpret_cast<const float4 *>(X),
                                                       reinterpret_cast<float4 *>(Y), n4);
      done = n4 * 4;
   }
   if (done < n) relu_f32_scalar<<<grid_for(n - done), kThreads, 0, s>>>(X, Y, done, n);
   SOFIE_LAUNCH_CHECK("relu_f32");
   return SOFIE_CUDA_OK;
}

int sofie_cuda_pool2d_f32(void *stream, const sofie_pool2d_desc *d, const float *X, float *Y)
{
   SOFIE_REQUIRE(d && X && Y, "NULL argument");
   SOFIE_REQUIRE(d->mode == 0 || d->mode == 1, "pool mode must be 0 (max) or 1 (average)");
   SOFIE_REQUIRE(d->N >= 0 && d->C > 0 && d->H > 0 && d->W > 0 && d->kH > 0 && d->kW > 0 && d->stride_h > 0 &&
                    d->stride_w > 0,
                 "bad pooling shape");
   // number of window positions, as the reference's shape inference counts them (ROperator_Pool.hxx:172-189)
   const int hspan = d->H + d->pads[0] + d->pads[2] - d->kH + 1, wspan = d->W + d->pads[1] + d->pads[3] - d->kW + 1;
   SOFIE_REQUIRE(hspan > 0 && wspan > 0, "pooling window larger than padded input");
   const int oH = ceil_div(hspan, d->stride_h), oW = ceil_div(wspan, d->stride_w);
   size_t total = (size_t)d->N * d->C * oH * oW;
   if (total == 0) return SOFIE_CUDA_OK;
   cudaStream_t s = as_stream(stream);
   const bool window2x2 = d->kH == 2 && d->kW == 2 && d->stride_h == 2 && d->stride_w == 2 && !d->pads[0] && !d->pads[1] && !d->pads[2] &&
                          !d->pads[3] && d->H % 2 == 0 && d->W % 2 == 0 && aligned16(X) && aligned16(Y) && total < (1u << 31);
   if (window2x2 && d->layout != SOFIE_LAYOUT_NHWC && d->W % 4 == 0) {
      const unsigned rows = (unsigned)((size_t)d->N * d->C * oH);
      if (d->mode == 0) pool2x2_f32_nchw_kernel<false><<<grid_for(total / 2), kThreads, 0, s>>>(X, Y, rows, d->W);
      else pool2x2_f32_nchw_kernel<true><<<grid_for(total / 2), kThreads, 0, s>>>(X, Y, rows, d->W);
   } else if (window2x2 && d->layout == SOFIE_LAYOUT_NHWC && d->C % 4 == 0) {
      const unsigned rows = (unsigned)((size_t)d->N * oH);
      if (d->mode == 0) pool2x2_f32_nhwc_kernel<false><<<grid_for(total / 4), kThreads, 0, s>>>(X, Y, rows, oW, d->C);
      else pool2x2_f32_nhwc_kernel<true><<<grid_for(total / 4), kThreads, 0, s>>>(X, Y, rows, oW, d->C);
   } else if (d->layout == SOFIE_LAYOUT_NHWC)
      pool2d_f32_kernel<true><<<grid_for(total), kThreads, 0, s>>>(*d, oH, oW, X, Y);
   else
      pool2d_f32_kernel<false><<<grid_for(total), kThreads, 0, s>>>(*d, oH, oW, X, Y);
   SOFIE_LAUNCH_CHECK("pool2d_f32_kernel");
   return SOFIE_CUDA_OK;
}

int sofie_cuda_maxpool2d_u8(void *stream, const uint8_t *X, uint8_t *Y, int32_t N, int32_t C, int32_t H, int32_t W,
                            int32_t kH, int32_t kW, int32_t sh, int32_t sw, int32_t layout)
{
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   SOFIE_REQUIRE(N >= 0 && C > 0 && H >= kH && W >= kW && kH > 0 && kW > 0 && sh > 0 && sw > 0, "bad pooling shape");
   const int oH = (H - kH) / sh + 1, oW = (W - kW) / sw + 1;
   size_t total = (size_t)N * C * oH * oW;
   if (total == 0) return SOFIE_CUDA_OK;
   cudaStream_t s = as_stream(stream);
   if (layout == SOFIE_LAYOUT_NHWC)
      maxpool2d_u8_kernel<true><<<grid_for(total), kThreads, 0, s>>>(N, C, H, W, kH, kW, sh, sw, oH, oW, X, Y);
   else
      maxpool2d_u8_kernel<false><<<grid_for(total), kThreads, 0, s>>>(N, C, H, W, kH, kW, sh, sw, oH, oW, X, Y);
   SOFIE_LAUNCH_CHECK("maxpool2d_u8_kernel");
   return SOFIE_CUDA_OK;
}

int sofie_cuda_softmax_f32(void *stream, const float *X, float *Y, size_t outer, size_t axis_len, size_t inner)
{
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   SOFIE_REQUIRE(axis_len > 0, "softmax along an axis with zero elements");
   if (outer == 0 || inner == 0) return SOFIE_CUDA_OK;
   cudaStream_t s = as_stream(stream);
   const bool vec = axis_len % 4 == 0 && aligned16(X) && aligned16(Y);
   if (inner == 1 && axis_len <= (size_t)kSoftmaxShortMax)
      softmax_rows_short_kernel<<<grid_for(outer), kSoftmaxShortRows, 0, s>>>(X, Y, outer, (int)axis_len);
   else if (inner == 1 && vec && axis_len <= 32 * 4 * 2)
      softmax_rows_reg_kernel<2><<<grid_for(outer * 32), kThreads, 0, s>>>(X, Y, outer, (int)(axis_len / 4));
   else if (inner == 1 && vec && axis_len <= 32 * 4 * 8)
      softmax_rows_reg_kernel<8><<<grid_for(outer * 32), kThreads, 0, s>>>(X, Y, outer, (int)(axis_len / 4));
   else if (inner == 1 && vec && axis_len <= 32 * 4 * 16)
      softmax_rows_reg_kernel<16><<<grid_for(outer * 32), kThreads, 0, s>>>(X, Y, outer, (int)(axis_len / 4));
   else if (inner == 1)
      softmax_rows_kernel<<<grid_for(outer * 32), kThreads, 0, s>>>(X, Y, outer, axis_len);
   else
      softmax_strided_kernel<<<grid_for(outer * inner), kThreads, 0, s>>>(X, Y, outer, axis_len, inner);
   SOFIE_LAUNCH_CHECK("softmax");
   return SOFIE_CUDA_OK;
}

int sofie_cuda_transpose_f32(void *stream, const float *in, float *out, int32_t rows, int32_t cols)
{
   SOFIE_REQUIRE(in && out && rows >= 0 && cols >= 0, "bad transpose arguments");
   return launch_transpose<float>(as_stream(stream), in, out, 1, rows, cols);
}
int sofie_cuda_transpose_i8(void *stream, const int8_t *in, int8_t *out, int32_t rows, int32_t cols)
{
   SOFIE_REQUIRE(in && out && rows >= 0 && cols >= 0, "bad transpose arguments");
   return launch_transpose<int8_t>(as_stream(stream), in, out, 1, rows, cols);
}
int sofie_cuda_nchw_to_nhwc_f32(void *stream, const float *X, float *Y, int32_t N, int32_t C, int32_t H, int32_t W)
{
   SOFIE_REQUIRE(X && Y && N >= 0 && C > 0 && H > 0 && W > 0, "bad layout-change arguments");
   if (N > 0 && launch_layout_few_channels<true>(as_stream(stream), X, Y, N, C, H * W)) {
      SOFIE_LAUNCH_CHECK("layout_few_channels_f32_kernel");
      return SOFIE_CUDA_OK;
   }
   return launch_transpose<float>(as_stream(stream), X, Y, N, C, H * W);
}
int sofie_cuda_nhwc_to_nchw_f32(void *stream, const float *X, float *Y, int32_t N, int32_t C, int32_t H, int32_t W)
{
   SOFIE_REQUIRE(X && Y && N >= 0 && C > 0 && H > 0 && W > 0, "bad layout-change arguments");
   if (N > 0 && launch_layout_few_channels<false>(as_stream(stream), X, Y, N, C, H * W)) {
      SOFIE_LAUNCH_CHECK("layout_few_channels_f32_kernel");
      return SOFIE_CUDA_OK;
   }
   return launch_transpose<float>(as_stream(stream), X, Y, N, H * W, C);
}
int sofie_cuda_nchw_to_nhwc_u8(void *stream, const uint8_t *X, uint8_t *Y, int32_t N, int32_t C, int32_t H, int32_t W)
{
   SOFIE_REQUIRE(X && Y && N >= 0 && C > 0 && H > 0 && W > 0, "bad layout-change arguments");
   return launch_transpose<uint8_t>(as_stream(stream), X, Y, N, C, H * W);
}
int sofie_cuda_nhwc_to_nchw_u8(void *stream, const uint8_t *X, uint8_t *Y, int32_t N, int32_t C, int32_t H, int32_t W)
{
   SOFIE_REQUIRE(X && Y && N >= 0 && C > 0 && H > 0 && W > 0, "bad layout-change arguments");
   return launch_transpose<uint8_t>(as_stream(stream), X, Y, N, H * W, C);
}

int sofie_cuda_quantize_u8(void *stream, const float *X, uint8_t *Y, size_t n, float scale, int32_t zp)
{
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   SOFIE_REQUIRE(scale > 0.f && zp >= 0 && zp <= 255, "bad quantisation parameters");
   if (n == 0) return SOFIE_CUDA_OK;
   const float inv_scale = 1.0f / scale;
   if (aligned16(X) && aligned16(Y) && n >= 16) {
      // the bulk sixteen elements at a time, the ragged end (fewer than 16 elements) with the scalar kernel
      const size_t n16 = n / 16;
      SOFIE_CUDA_TRY(launch_dependent(quantize_u8_vec16_kernel, dim3(grid_for(n16)), dim3(kThreads), 0, as_stream(stream), X, Y, n16, scale, inv_scale, (int)zp));
      X += n16 * 16;
      Y += n16 * 16;
      n -= n16 * 16;
      if (n == 0) return SOFIE_CUDA_OK;
   }
   bool vec = aligned16(X) && (reinterpret_cast<uintptr_t>(Y) & 3) == 0;
   SOFIE_CUDA_TRY(launch_dependent(quantize_u8_kernel, dim3(grid_for(vec ? n / 4 + 1 : n)), dim3(kThreads), 0, as_stream(stream), X, Y, n, scale,
                                   inv_scale, (int)zp, vec));
   return SOFIE_CUDA_OK;
}

int sofie_cuda_dequantize_u8(void *stream, const uint8_t *X, float *Y, size_t n, float scale, int32_t zp)
{
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   if (n == 0) return SOFIE_CUDA_OK;
   bool vec = aligned16(Y) && (reinterpret_cast<uintptr_t>(X) & 3) == 0;
   SOFIE_CUDA_TRY(launch_dependent(dequantize_u8_kernel, dim3(grid_for(vec ? n / 4 + 1 : n)), dim3(kThreads), 0, as_stream(stream), X, Y, n, scale,
                                   (int)zp, vec));
   return SOFIE_CUDA_OK;
}

int sofie_cuda_quantize_e4m3_f32(void *stream, const float *X, uint8_t *Y, size_t n, float scale)
{
   SOFIE_REQUIRE(X && Y && scale > 0.f, "bad arguments");
   if (n == 0) return SOFIE_CUDA_OK;
   return launch_quantize_e4m3<float>(as_stream(stream), X, Y, n, scale);
}
int sofie_cuda_quantize_e4m3_bf16(void *stream, const uint16_t *X, uint8_t *Y, size_t n, float scale)
{
   SOFIE_REQUIRE(X && Y && scale > 0.f, "bad arguments");
   if (n == 0) return SOFIE_CUDA_OK;
   return launch_quantize_e4m3<uint16_t>(as_stream(stream), X, Y, n, scale);
}
int sofie_cuda_dynamic_quantize_e4m3_f32(void *stream, const float *X, uint8_t *Y, size_t n, float *scale_device)
{
   SOFIE_REQUIRE((X && Y) || n == 0, "NULL tensor");
   SOFIE_REQUIRE(scale_device != nullptr, "NULL scale");
   return dynamic_quantize_e4m3<float>(as_stream(stream), X, Y, n, scale_device);
}
int sofie_cuda_dynamic_quantize_e4m3_bf16(void *stream, const uint16_t *X, uint8_t *Y, size_t n, float *scale_device)
{
   SOFIE_REQUIRE((X && Y) || n == 0, "NULL tensor");
   SOFIE_REQUIRE(scale_device != nullptr, "NULL scale");
   return dynamic_quantize_e4m3<uint16_t>(as_stream(stream), X, Y, n, scale_device);
}
int sofie_cuda_cast_bf16_f32(void *stream, const uint16_t *X, float *Y, size_t n)
{
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   if (n == 0) return SOFIE_CUDA_OK;
   cudaStream_t s = as_stream(stream);
   size_t done = 0;
   if (aligned16(X) && aligned16(Y) && n >= 8) {
      const size_t n8 = n / 8;
      cast_bf16_f32_vec8_kernel<<<grid_for(n8), kThreads, 0, s>>>(X, Y, n8);
      SOFIE_LAUNCH_CHECK("cast_bf16_f32_vec8_kernel");
      done = n8 * 8;
   }
   if (done < n) {
      cast_bf16_f32_kernel<<<grid_for(n - done), kThreads, 0, s>>>(X, Y, done, n);
      SOFIE_LAUNCH_CHECK("cast_bf16_f32_kernel");
   }
   return SOFIE_CUDA_OK;
}
int sofie_cuda_cast_f32_bf16(void *stream, const float *X, uint16_t *Y, size_t n)
{
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   if (n == 0) return SOFIE_CUDA_OK;
   cast_f32_bf16_kernel<<<grid_for(n), kThreads, 0, as_stream(stream)>>>(X, Y, n);
   SOFIE_LAUNCH_CHECK("cast_f32_bf16_kernel");
   return SOFIE_CUDA_OK;
}
int sofie_cuda_amax_f32(void *stream, const float *X, size_t n, float *amax_device)
{
   SOFIE_REQUIRE(X && amax_device, "NULL tensor");
   cudaStream_t s = as_stream(stream);
   SOFIE_CUDA_TRY(cudaMemsetAsync(amax_device, 0, sizeof(float), s));
   if (n == 0) return SOFIE_CUDA_OK;
   amax_f32_kernel<<<grid_for(n), kThreads, 0, s>>>(X, n, reinterpret_cast<unsigned *>(amax_device));
   SOFIE_LAUNCH_CHECK("amax_f32_kernel");
   return SOFIE_CUDA_OK;
}

} // extern "C"
