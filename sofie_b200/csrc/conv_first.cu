// First-layer convolutions: 3x3, stride 1, pad 1, group 1 with at most 4 input channels (K = 9 C <= 36)
// and at most 64 output channels. With so little K the layer is bound by memory and by the epilogue,
// not by the contraction, so these are plain SIMT kernels built around the data movement:
//   * a block stages the haloed input tile of 16 x 16 (pooled) outputs in shared memory once;
//   * a thread owns one (pooled) output pixel and ALL output channels, so an NHWC output pixel is
//     written with 16-byte stores and neighbouring threads write neighbouring pixels;
//   * weights sit in shared memory, packed for the inner loop, and are read as broadcasts;
//   * with a fused 2x2 MaxPool the maximum is taken over the raw accumulators and bias, Relu and
//     requantisation run once per pooled output: every one of those steps is non-decreasing in
//     the accumulator (the requantisation multiplier is checked to be >= 0), so the stored values
//     are the ones the unfused sequence gives.
// uint8 x int8: the taps of a pixel are packed four to a word and contracted with dp4a; the input
// zero point enters through the padding value and a per-channel correction -zp * sum(w).
#include "contract.cuh"

#include <cstdlib>

namespace sofie {
namespace {

constexpr int kFirstThreads = 256;  // 16 x 16 outputs per block
constexpr int kFirstMaxCout = 64;
constexpr int kFirstF32Threads = 128; // fp32 kernel: 8 x 16 threads, each a 2 x 2 block of outputs
constexpr int kFirstF32UnitsY = 8;

__device__ __forceinline__ int dp4a_u8s8_first(unsigned a, int b, int c)
{
   int d;
   asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
   return d;
}

__device__ __forceinline__ size_t weight_index(const ConvGeom &g, int oc, int c, int r, int t)
{
   return g.w_packed ? (((size_t)oc * 3 + r) * 3 + t) * g.C + c : (((size_t)oc * g.C + c) * 3 + r) * 3 + t;
}

// tile -> image, first (pooled) output row and column
__device__ __forceinline__ void first_tile_origin(const ConvGeom &g, long long tile, int tiles_x, int tiles_y, int &n, int &py0, int &px0)
{
   const int per_image = tiles_x * tiles_y;
   n = (int)(tile / per_image);
   const int rem = (int)(tile % per_image);
   py0 = (rem / tiles_x) * 16;
   px0 = (rem % tiles_x) * 16;
}

// ------------------------------------------------------------------------------------------------
template <int C, int POOL>
__global__ void __launch_bounds__(kFirstThreads)
qconv3x3_first_kernel(ConvGeom g, const uint8_t *__restrict__ X, const int8_t *__restrict__ Wt, const float *__restrict__ mult,
                      const int32_t *__restrict__ bias, int x_zp, int y_zp, uint8_t *__restrict__ Y, long long num_tiles,
                      int tiles_x, int tiles_y)
{
   griddep_launch_dependents(); // the next kernel may set itself up (weights into shared memory) while this one runs
   constexpr int K = 9 * C, KW = (K + 3) / 4;
   constexpr int TS = 16 * POOL + 2;  // side of the haloed input tile
   constexpr int TP = (TS + 3) / 4 * 4;
   constexpr int NPOS = POOL * POOL;
   constexpr int OCC = 8;             // output channels per register pass
   __shared__ uint8_t tile[C][TS][TP];
   __shared__ int s_w[kFirstMaxCout][KW];
   __shared__ float s_mult[kFirstMaxCout];
   __shared__ int s_bias[kFirstMaxCout];
   __shared__ int s_negative;

   const int tid = threadIdx.x;
   if (tid == 0) s_negative = 0;
   __syncthreads();
   // weights: tap k = c * 9 + r * 3 + t of channel oc is byte k % 4 of word k / 4
   for (int i = tid; i < kFirstMaxCout * KW; i += kFirstThreads) {
      const int oc = i / KW, j = i % KW;
      unsigned word = 0;
      if (oc < g.Cout) {
         for (int b = 0; b < 4; b++) {
            const int k = 4 * j + b;
            if (k < K) {
               const int c = k / 9, r = (k % 9) / 3, t = k % 3;
               word |= (unsigned)(uint8_t)Wt[weight_index(g, oc, c, r, t)] << (8 * b);
            }
         }
      }
      s_w[oc][j] = (int)word;
   }
   for (int oc = tid; oc < kFirstMaxCout; oc += kFirstThreads) {
      float m = 0.f;
      int b = 0;
      if (oc < g.Cout) {
         m = mult[oc];
         int wsum = 0;
         for (int k = 0; k < K; k++) wsum += (int)Wt[weight_index(g, oc, k / 9, (k % 9) / 3, k % 3)];
         b = (bias ? bias[oc] : 0) - x_zp * wsum;
         if (!(m >= 0.f)) s_negative = 1;
      }
      s_mult[oc] = m;
      s_bias[oc] = b;
   }
   __syncthreads();
   const bool pool_first = (NPOS > 1) && !s_negative;

   const int ty = tid / 16, tx = tid % 16;
   for (long long tile_id = blockIdx.x; tile_id < num_tiles; tile_id += gridDim.x) {
      int n, py0, px0;
      first_tile_origin(g, tile_id, tiles_x, tiles_y, n, py0, px0);
      const int ih0 = py0 * POOL - 1, iw0 = px0 * POOL - 1;
      constexpr int kLoads = (C * TS * TS + kFirstThreads - 1) / kFirstThreads;
      uint8_t staged[kLoads];
#pragma unroll
      for (int j = 0; j < kLoads; j++) {
         const int i = tid + j * kFirstThreads;
         const int c = i / (TS * TS), rem = i % (TS * TS), r = rem / TS, col = rem % TS;
         const int ih = ih0 + r, iw = iw0 + col;
         uint8_t v = (uint8_t)x_zp;
         if (i < C * TS * TS && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) {
            const size_t xi = g.x_nhwc ? (((size_t)n * g.H + ih) * g.W + iw) * C + c : (((size_t)n * C + c) * g.H + ih) * g.W + iw;
            v = __ldg(X + xi);
         }
         staged[j] = v;
      }
      __syncthreads(); // the previous tile is no longer read
#pragma unroll
      for (int j = 0; j < kLoads; j++) {
         const int i = tid + j * kFirstThreads;
         if (i < C * TS * TS) tile[i / (TS * TS)][(i % (TS * TS)) / TS][i % TS] = staged[j];
      }
      __syncthreads();
      const int ph = py0 + ty, pw = px0 + tx;
      if (ph >= g.pH || pw >= g.pW) continue;
      // packed taps of the NPOS convolution outputs of this thread
      unsigned xw[NPOS][KW];
#pragma unroll
      for (int q = 0; q < NPOS; q++) {
         const int dy = q / POOL, dx = q % POOL;
#pragma unroll
         for (int j = 0; j < KW; j++) {
            unsigned word = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) {
               const int k = 4 * j + b;
               if (k < K) {
                  const int c = k / 9, r = (k % 9) / 3, t = k % 3;
                  word |= (unsigned)tile[c][ty * POOL + dy + r][tx * POOL + dx + t] << (8 * b);
               }
            }
            xw[q][j] = word;
         }
      }
      const size_t opix = ((size_t)n * g.pH + ph) * g.pW + pw;
      for (int oc0 = 0; oc0 < g.Cout; oc0 += OCC) {
         int out[OCC];
#pragma unroll
         for (int o = 0; o < OCC; o++) {
            const int oc = oc0 + o; // < kFirstMaxCout; channels past Cout have zero weights
            int acc[NPOS];
#pragma unroll
            for (int q = 0; q < NPOS; q++) acc[q] = 0;
#pragma unroll
            for (int j = 0; j < KW; j++) {
               const int w = s_w[oc][j];
#pragma unroll
               for (int q = 0; q < NPOS; q++) acc[q] = dp4a_u8s8_first(xw[q][j], w, acc[q]);
            }
            const int b = s_bias[oc];
            const float m = s_mult[oc];
            int v;
            if (pool_first || NPOS == 1) {
               int best = acc[0];
#pragma unroll
               for (int q = 1; q < NPOS; q++) best = max(best, acc[q]);
               v = requant_u8(best + b, m, y_zp, g.relu);
            } else {
               v = requant_u8(acc[0] + b, m, y_zp, g.relu);
#pragma unroll
               for (int q = 1; q < NPOS; q++) v = max(v, requant_u8(acc[q] + b, m, y_zp, g.relu));
            }
            out[o] = v;
         }
         if (g.y_nhwc) {
            uint8_t *y = Y + opix * g.Cout + oc0;
            if (oc0 + OCC <= g.Cout && ((reinterpret_cast<uintptr_t>(y) & 7) == 0)) {
               uint2 pk;
               pk.x = (unsigned)out[0] | ((unsigned)out[1] << 8) | ((unsigned)out[2] << 16) | ((unsigned)out[3] << 24);
               pk.y = (unsigned)out[4] | ((unsigned)out[5] << 8) | ((unsigned)out[6] << 16) | ((unsigned)out[7] << 24);
               *reinterpret_cast<uint2 *>(y) = pk;
            } else {
#pragma unroll
               for (int o = 0; o < OCC; o++)
                  if (oc0 + o < g.Cout) y[o] = (uint8_t)out[o];
            }
         } else {
#pragma unroll
            for (int o = 0; o < OCC; o++)
               if (oc0 + o < g.Cout) Y[(((size_t)n * g.Cout + oc0 + o) * g.pH + ph) * g.pW + pw] = (uint8_t)out[o];
         }
      }
   }
}

// ------------------------------------------------------------------------------------------------
// One input channel with the 2 x 2 pool fused (grey-scale / calorimeter images): the kernel is instruction
// bound, so everything around the 12 dp4a of a pooled output is cut down.
//   * a dp4a takes one ROW of the 4 x 4 input patch under a pooling window as it lies in the image (four
//     consecutive pixels, no repacking of taps); the filter row is stored twice, as (w0,w1,w2,0) for the
//     left output of the window and as (0,w0,w1,w2) for the right one;
//   * the six filter words of a channel, its bias and its multiplier are two 16-byte shared-memory loads;
//   * the input tile is staged with 32-bit loads (the image width is a multiple of 4 and a tile starts on
//     a multiple of 32 columns, so a word is either inside the image or entirely padding) and a thread
//     builds each of its four patch rows from two shared words and one funnel shift.
// Same arithmetic as the general kernel: padding holds the input zero point, bias' = bias - x_zp * sum(w),
// pooling over the raw sums before requantisation when every multiplier is non-negative.
__global__ void __launch_bounds__(kFirstThreads)
qconv3x3_first_c1_pool_kernel(ConvGeom g, const uint8_t *__restrict__ X, const int8_t *__restrict__ Wt, const float *__restrict__ mult,
                              const int32_t *__restrict__ bias, int x_zp, int y_zp, uint8_t *__restrict__ Y, long long num_tiles,
                              int tiles_x, int tiles_y)
{
   griddep_launch_dependents();
   constexpr int TS = 34;     // rows of the haloed tile
   constexpr int TW = 10;     // words per row: image columns px0*2 - 4 .. px0*2 + 35
   constexpr int OCC = 8;
   __shared__ unsigned tile[TS][TW + 1];
   __shared__ uint4 s_wa[kFirstMaxCout]; // filter rows for the left output (w0,w1,w2,0) x 3, bias'
   __shared__ uint4 s_wb[kFirstMaxCout]; // filter rows for the right output (0,w0,w1,w2) x 3, multiplier bits
   __shared__ int s_negative;

   const int tid = threadIdx.x;
   if (tid == 0) s_negative = 0;
   __syncthreads();
   for (int oc = tid; oc < kFirstMaxCout; oc += kFirstThreads) {
      unsigned a[3] = {0, 0, 0}, b[3] = {0, 0, 0};
      float m = 0.f;
      int bb = 0;
      if (oc < g.Cout) {
         int wsum = 0;
         for (int r = 0; r < 3; r++) {
            unsigned w = 0;
            for (int t = 0; t < 3; t++) {
               const int v = (int)Wt[weight_index(g, oc, 0, r, t)];
               wsum += v;
               w |= (unsigned)(uint8_t)v << (8 * t);
            }
            a[r] = w;
            b[r] = w << 8;
         }
         m = mult[oc];
         bb = (bias ? bias[oc] : 0) - x_zp * wsum;
         if (!(m >= 0.f)) s_negative = 1;
      }
      s_wa[oc] = make_uint4(a[0], a[1], a[2], (unsigned)bb);
      s_wb[oc] = make_uint4(b[0], b[1], b[2], __float_as_uint(m));
   }
   __syncthreads();
   const bool pool_first = !s_negative;
   const unsigned pad_word = (unsigned)x_zp * 0x01010101u;
   const int ty = tid / 16, tx = tid % 16;
   const int wcols = g.W >> 2; // words per image row
   for (long long tile_id = blockIdx.x; tile_id < num_tiles; tile_id += gridDim.x) {
      int n, py0, px0;
      first_tile_origin(g, tile_id, tiles_x, tiles_y, n, py0, px0);
      const int ih0 = py0 * 2 - 1, wc0 = (px0 * 2 - 4) >> 2; // first row and first word column of the tile (may be -1)
      const unsigned *img = reinterpret_cast<const unsigned *>(X + (size_t)n * g.H * g.W);
      unsigned staged[2];
#pragma unroll
      for (int j = 0; j < 2; j++) {
         const int i = tid + j * kFirstThreads;
         const int r = i / TW, c = i - r * TW;
         const int ih = ih0 + r, wc = wc0 + c;
         unsigned v = pad_word;
         if (i < TS * TW && ih >= 0 && ih < g.H && wc >= 0 && wc < wcols) v = __ldg(img + (size_t)ih * wcols + wc);
         staged[j] = v;
      }
      __syncthreads(); // the previous tile is no longer read
#pragma unroll
      for (int j = 0; j < 2; j++) {
         const int i = tid + j * kFirstThreads;
         if (i < TS * TW) tile[i / TW][i % TW] = staged[j];
      }
      __syncthreads();
      const int ph = py0 + ty, pw = px0 + tx;
      if (ph >= g.pH || pw >= g.pW) continue;
      // the four rows of the 4 x 4 patch: image columns 2 pw - 1 .. 2 pw + 2 = tile bytes 3 + 2 tx .. 6 + 2 tx
      unsigned row[4];
      {
         const int byte0 = 3 + 2 * tx, w0 = byte0 >> 2, sh = 8 * (byte0 & 3);
#pragma unroll
         for (int r = 0; r < 4; r++) row[r] = __funnelshift_r(tile[2 * ty + r][w0], tile[2 * ty + r][w0 + 1], sh);
      }
      const size_t opix = ((size_t)n * g.pH + ph) * g.pW + pw;
      for (int oc0 = 0; oc0 < g.Cout; oc0 += OCC) {
         int out[OCC];
#pragma unroll
         for (int o = 0; o < OCC; o++) {
            const uint4 wa = s_wa[oc0 + o], wb = s_wb[oc0 + o]; // channels past Cout hold zeros
            int a00 = dp4a_u8s8_first(row[0], (int)wa.x, 0), a01 = dp4a_u8s8_first(row[0], (int)wb.x, 0);
            int a10 = dp4a_u8s8_first(row[1], (int)wa.x, 0), a11 = dp4a_u8s8_first(row[1], (int)wb.x, 0);
            a00 = dp4a_u8s8_first(row[1], (int)wa.y, a00), a01 = dp4a_u8s8_first(row[1], (int)wb.y, a01);
            a10 = dp4a_u8s8_first(row[2], (int)wa.y, a10), a11 = dp4a_u8s8_first(row[2], (int)wb.y, a11);
            a00 = dp4a_u8s8_first(row[2], (int)wa.z, a00), a01 = dp4a_u8s8_first(row[2], (int)wb.z, a01);
            a10 = dp4a_u8s8_first(row[3], (int)wa.z, a10), a11 = dp4a_u8s8_first(row[3], (int)wb.z, a11);
            const int b = (int)wa.w;
            const float m = __uint_as_float(wb.w);
            int v;
            if (pool_first) {
               v = requant_u8(max(max(a00, a01), max(a10, a11)) + b, m, y_zp, g.relu);
            } else {
               v = max(max(requant_u8(a00 + b, m, y_zp, g.relu), requant_u8(a01 + b, m, y_zp, g.relu)),
                       max(requant_u8(a10 + b, m, y_zp, g.relu), requant_u8(a11 + b, m, y_zp, g.relu)));
            }
            out[o] = v;
         }
         if (g.y_nhwc) {
            uint8_t *y = Y + opix * g.Cout + oc0;
            if (oc0 + OCC <= g.Cout && ((reinterpret_cast<uintptr_t>(y) & 7) == 0)) {
               uint2 pk;
               pk.x = (unsigned)out[0] | ((unsigned)out[1] << 8) | ((unsigned)out[2] << 16) | ((unsigned)out[3] << 24);
               pk.y = (unsigned)out[4] | ((unsigned)out[5] << 8) | ((unsigned)out[6] << 16) | ((unsigned)out[7] << 24);
               *reinterpret_cast<uint2 *>(y) = pk;
            } else {
#pragma unroll
               for (int o = 0; o < OCC; o++)
                  if (oc0 + o < g.Cout) y[o] = (uint8_t)out[o];
            }
         } else {
#pragma unroll
            for (int o = 0; o < OCC; o++)
               if (oc0 + o < g.Cout) Y[(((size_t)n * g.Cout + oc0 + o) * g.pH + ph) * g.pW + pw] = (uint8_t)out[o];
         }
      }
   }
}

// ------------------------------------------------------------------------------------------------
// fp32: a thread owns a 2 x 2 block of convolution outputs (the pooling window when the pool is
// fused, four stored pixels otherwise) and 16 output channels at a time. The weights are read from
// shared memory as 16-byte broadcasts; each one feeds four FMAs per output, 16 in all, which keeps
// the shared-memory pipe off the critical path. A block of 128 threads covers 16 rows x 32 columns of
// convolution outputs; blocks are kept that small so that four fit on an SM and the load, compute and
// store phases of different blocks overlap.
// VEC: NCHW input whose width is a multiple of 4 (and a 16-byte aligned base): the tile is staged with 16-byte
// asynchronous copies of whole words of the image rows (a tile starts on a multiple of 32 columns, so a word is
// either inside the image or entirely padding, which the copy zero-fills); the patch then starts at column 3.
template <int C, int POOL, bool VEC>
__global__ void __launch_bounds__(kFirstF32Threads, 4)
conv3x3_first_f32_kernel(ConvGeom g, const float *__restrict__ X, const float *__restrict__ Wt, const float *__restrict__ bias,
                         float *__restrict__ Y, long long num_tiles, int tiles_x, int tiles_y)
{
   griddep_launch_dependents(); // the next kernel may set itself up (weights into shared memory) while this one runs
   constexpr int K = 9 * C;
   constexpr int TSH = 2 * kFirstF32UnitsY + 2, TS = 34; // haloed input tile: 18 rows x 34 columns
   constexpr int OCC = 8;
   constexpr int TW4 = 10;                       // VEC: 16-byte words per tile row, image columns ux0*2 - 4 .. ux0*2 + 35
   constexpr int TSW = VEC ? 4 * TW4 : TS + 1;   // row stride of the tile in floats
   constexpr int COL0 = VEC ? 3 : 0;             // tile column of the patch's first input column
   __shared__ __align__(16) float tile[C][TSH][TSW];
   __shared__ float4 s_w[K][kFirstMaxCout / 4]; // [tap][channel / 4]
   __shared__ float s_bias[kFirstMaxCout];

   const int tid = threadIdx.x;
   const int ty = tid / 16, tx = tid % 16;
   bool weights_staged = false;
   for (long long tile_id = blockIdx.x; tile_id < num_tiles; tile_id += gridDim.x) {
      int n, uy0, ux0; // origin in units of 2 x 2 outputs
      first_tile_origin(g, tile_id, tiles_x, tiles_y, n, uy0, ux0);
      uy0 = uy0 / 16 * kFirstF32UnitsY; // this kernel's tiles are 8 units tall
      const int ih0 = uy0 * 2 - 1, iw0 = ux0 * 2 - 1;
      // all loads of a thread are issued before the first store, so their latencies overlap
      constexpr int kLoads = VEC ? 1 : (C * TSH * TS + kFirstF32Threads - 1) / kFirstF32Threads;
      float staged[kLoads];
      if constexpr (VEC) {
         __syncthreads(); // the previous tile is no longer read: the copies below write the tile directly
         constexpr int kPieces = C * TSH * TW4;
         const int wc0 = (ux0 * 2 - 4) >> 2, wcols = g.W >> 2;
#pragma unroll
         for (int j = 0; j < (kPieces + kFirstF32Threads - 1) / kFirstF32Threads; j++) {
            const int i = tid + j * kFirstF32Threads;
            if (i < kPieces) {
               const int c = i / (TSH * TW4), rem = i % (TSH * TW4), r = rem / TW4, w = rem % TW4;
               const int ih = ih0 + r, wc = wc0 + w;
               const bool ok = ih >= 0 && ih < g.H && wc >= 0 && wc < wcols;
               const float *src = X + (((size_t)n * C + c) * g.H + (ok ? ih : 0)) * g.W + 4 * (ok ? wc : 0);
               const unsigned dst = (unsigned)__cvta_generic_to_shared(&tile[c][r][4 * w]);
               const int bytes = ok ? 16 : 0; // zero-filled when the word lies outside the image
               asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
            }
         }
         staged[0] = 0.f;
      } else {
#pragma unroll
      for (int j = 0; j < kLoads; j++) {
         const int i = tid + j * kFirstF32Threads;
         const int c = i / (TSH * TS), rem = i % (TSH * TS), r = rem / TS, col = rem % TS;
         const int ih = ih0 + r, iw = iw0 + col;
         float v = 0.f;
         if (i < C * TSH * TS && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) {
            const size_t xi = g.x_nhwc ? (((size_t)n * g.H + ih) * g.W + iw) * C + c : (((size_t)n * C + c) * g.H + ih) * g.W + iw;
            v = __ldg(X + xi);
         }
         staged[j] = v;
      }
      }
      if (!weights_staged) {
         // The weights are fetched while the loads of the first tile are still in flight.
         // zero the channels past Cout, then fetch only the K x Cout real weights, a few loads in flight per thread
         for (int i = tid; i < K * kFirstMaxCout; i += kFirstF32Threads)
            if (i % kFirstMaxCout >= g.Cout) reinterpret_cast<float *>(&s_w[0][0])[i] = 0.f;
         const int real = K * g.Cout;
#pragma unroll 4
         for (int i = tid; i < real; i += kFirstF32Threads) {
            const int k = i / g.Cout, oc = i - k * g.Cout;
            reinterpret_cast<float *>(&s_w[k][0])[oc] = __ldg(Wt + weight_index(g, oc, k / 9, (k % 9) / 3, k % 3));
         }
         for (int oc = tid; oc < kFirstMaxCout; oc += kFirstF32Threads) s_bias[oc] = (oc < g.Cout && bias) ? __ldg(bias + oc) : 0.f;
         weights_staged = true;
      }
      if constexpr (VEC) {
         asm volatile("cp.async.wait_all;\n" ::: "memory");
      } else {
         __syncthreads(); // weights staged / the previous tile is no longer read
#pragma unroll
         for (int j = 0; j < kLoads; j++) {
            const int i = tid + j * kFirstF32Threads;
            if (i < C * TSH * TS) tile[i / (TSH * TS)][(i % (TSH * TS)) / TS][i % TS] = staged[j];
         }
      }
      __syncthreads(); // tile and weights are in shared memory
      const int oh0 = (uy0 + ty) * 2, ow0 = (ux0 + tx) * 2; // top-left convolution output of this thread
      if (oh0 >= g.oH || ow0 >= g.oW) continue;
      for (int oc0 = 0; oc0 < g.Cout; oc0 += OCC) {
         float acc[4][OCC];
#pragma unroll
         for (int q = 0; q < 4; q++)
#pragma unroll
            for (int o = 0; o < OCC; o++) acc[q][o] = 0.f;
#pragma unroll
         for (int c = 0; c < C; c++) {
            float win[4][4]; // the 4 x 4 inputs under the 2 x 2 outputs
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
               for (int t = 0; t < 4; t++) win[r][t] = tile[c][ty * 2 + r][COL0 + tx * 2 + t];
#pragma unroll
            for (int rt = 0; rt < 9; rt++) {
               const int r = rt / 3, t = rt % 3;
#pragma unroll
               for (int o4 = 0; o4 < OCC / 4; o4++) {
                  const float4 w = s_w[c * 9 + rt][oc0 / 4 + o4];
#pragma unroll
                  for (int q = 0; q < 4; q++) {
                     const float xv = win[(q >> 1) + r][(q & 1) + t];
                     acc[q][4 * o4 + 0] = fmaf(xv, w.x, acc[q][4 * o4 + 0]);
                     acc[q][4 * o4 + 1] = fmaf(xv, w.y, acc[q][4 * o4 + 1]);
                     acc[q][4 * o4 + 2] = fmaf(xv, w.z, acc[q][4 * o4 + 2]);
                     acc[q][4 * o4 + 3] = fmaf(xv, w.w, acc[q][4 * o4 + 3]);
                  }
               }
            }
         }
         // one stored pixel (pooled) or four
         auto store_pixel = [&](const float *v, int ph, int pw) {
            const size_t opix = ((size_t)n * g.pH + ph) * g.pW + pw;
            if (g.y_nhwc) {
               float *y = Y + opix * g.Cout + oc0;
               if (oc0 + OCC <= g.Cout && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
                  for (int o = 0; o < OCC; o += 4) *reinterpret_cast<float4 *>(y + o) = make_float4(v[o], v[o + 1], v[o + 2], v[o + 3]);
               } else {
#pragma unroll
                  for (int o = 0; o < OCC; o++)
                     if (oc0 + o < g.Cout) y[o] = v[o];
               }
            } else {
#pragma unroll
               for (int o = 0; o < OCC; o++)
                  if (oc0 + o < g.Cout) Y[(((size_t)n * g.Cout + oc0 + o) * g.pH + ph) * g.pW + pw] = v[o];
            }
         };
         if constexpr (POOL == 2) {
            if ((oh0 >> 1) < g.pH && (ow0 >> 1) < g.pW) {
               float best[OCC];
#pragma unroll
               for (int o = 0; o < OCC; o++) {
                  float m = acc[0][o];
#pragma unroll
                  for (int q = 1; q < 4; q++) m = acc[q][o] > m ? acc[q][o] : m;
                  const float v = m + s_bias[oc0 + o];
                  best[o] = g.relu ? relu_ref(v) : v;
               }
               store_pixel(best, oh0 >> 1, ow0 >> 1);
            }
         } else {
#pragma unroll
            for (int q = 0; q < 4; q++) {
               const int oh = oh0 + (q >> 1), ow = ow0 + (q & 1);
               if (oh < g.oH && ow < g.oW) {
#pragma unroll
                  for (int o = 0; o < OCC; o++) {
                     const float v = acc[q][o] + s_bias[oc0 + o];
                     acc[q][o] = g.relu ? relu_ref(v) : v;
                  }
                  store_pixel(acc[q], oh, ow);
               }
            }
         }
      }
   }
}

// SOFIE_CUDA_FIRST_C1=0 keeps single-channel first layers on the general kernel (used to compare the two)
bool first_c1_enabled()
{
   static const bool v = [] { const char *e = getenv("SOFIE_CUDA_FIRST_C1"); return !e || atoi(e) != 0; }();
   return v;
}

bool first_layer_shape(const ConvGeom &g)
{
   return g.kH == 3 && g.kW == 3 && g.pad_h == 1 && g.pad_w == 1 && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1 && g.group == 1 &&
          g.C >= 1 && g.C <= 4 && g.Cout >= 1 && g.Cout <= kFirstMaxCout && (g.pool == 0 || g.pool == 2);
}

struct FirstGrid {
   long long num_tiles;
   int tiles_x, tiles_y, blocks;
};

// units_x x units_y = extent in the units a thread owns (stored pixels for the uint8 kernel, 2 x 2
// blocks of convolution outputs for the fp32 one); a block covers 16 x 16 of them.
FirstGrid first_grid(const ConvGeom &g, int units_x, int units_y, int tile_units_y, int blocks_per_sm)
{
   FirstGrid fg;
   fg.tiles_x = ceil_div(units_x, 16);
   fg.tiles_y = ceil_div(units_y, tile_units_y);
   fg.num_tiles = (long long)g.N * fg.tiles_x * fg.tiles_y;
   const long long cap = (long long)kNumSMs * blocks_per_sm;
   fg.blocks = (int)(fg.num_tiles < cap ? fg.num_tiles : cap);
   return fg;
}

} // namespace

// Both return -1 when the shape is not a first-layer shape (the caller then takes the general kernel).
int launch_qconv2d_first(cudaStream_t s, const ConvGeom &g, const uint8_t *X, const int8_t *W, const float *mult, const int32_t *bias,
                         int x_zp, int y_zp, uint8_t *Y)
{
   if (!first_layer_shape(g)) return -1;
   const FirstGrid fg = first_grid(g, g.pW, g.pH, 16, 8);
   if (fg.num_tiles == 0) return SOFIE_CUDA_OK;
#define SOFIE_FIRST_Q(CC, PP)                                                                                                   \
   qconv3x3_first_kernel<CC, PP><<<fg.blocks, kFirstThreads, 0, s>>>(g, X, W, mult, bias, x_zp, y_zp, Y, fg.num_tiles, fg.tiles_x, \
                                                                     fg.tiles_y)
   const int pp = g.pool == 2 ? 2 : 1;
   if (g.C == 1 && pp == 2 && g.W % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 3) == 0 && first_c1_enabled()) {
      qconv3x3_first_c1_pool_kernel<<<fg.blocks, kFirstThreads, 0, s>>>(g, X, W, mult, bias, x_zp, y_zp, Y, fg.num_tiles, fg.tiles_x, fg.tiles_y);
      SOFIE_LAUNCH_CHECK("qconv3x3_first_c1_pool_kernel");
      set_last_engine(SOFIE_ENGINE_SIMT);
      return SOFIE_CUDA_OK;
   }
   switch (g.C * 10 + pp) {
   case 11: SOFIE_FIRST_Q(1, 1); break;
   case 12: SOFIE_FIRST_Q(1, 2); break;
   case 21: SOFIE_FIRST_Q(2, 1); break;
   case 22: SOFIE_FIRST_Q(2, 2); break;
   case 31: SOFIE_FIRST_Q(3, 1); break;
   case 32: SOFIE_FIRST_Q(3, 2); break;
   case 41: SOFIE_FIRST_Q(4, 1); break;
   default: SOFIE_FIRST_Q(4, 2); break;
   }
#undef SOFIE_FIRST_Q
   SOFIE_LAUNCH_CHECK("qconv3x3_first_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

int launch_conv2d_f32_first(cudaStream_t s, const ConvGeom &g, const float *X, const float *W, const float *bias, float *Y)
{
   if (!first_layer_shape(g)) return -1;
   const FirstGrid fg = first_grid(g, (g.oW + 1) / 2, (g.oH + 1) / 2, kFirstF32UnitsY, 4);
   if (fg.num_tiles == 0) return SOFIE_CUDA_OK;
   static const bool vec_enabled = [] { const char *e = getenv("SOFIE_CUDA_FIRST_VEC"); return !e || atoi(e) != 0; }();
   const bool vec = vec_enabled && !g.x_nhwc && g.W % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0;
#define SOFIE_FIRST_F(CC, PP)                                                                                                      \
   if (vec) conv3x3_first_f32_kernel<CC, PP, true><<<fg.blocks, kFirstF32Threads, 0, s>>>(g, X, W, bias, Y, fg.num_tiles, fg.tiles_x, fg.tiles_y); \
   else conv3x3_first_f32_kernel<CC, PP, false><<<fg.blocks, kFirstF32Threads, 0, s>>>(g, X, W, bias, Y, fg.num_tiles, fg.tiles_x, fg.tiles_y)
   const int pp = g.pool == 2 ? 2 : 1;
   switch (g.C * 10 + pp) {
   case 11: SOFIE_FIRST_F(1, 1); break;
   case 12: SOFIE_FIRST_F(1, 2); break;
   case 21: SOFIE_FIRST_F(2, 1); break;
   case 22: SOFIE_FIRST_F(2, 2); break;
   case 31: SOFIE_FIRST_F(3, 1); break;
   case 32: SOFIE_FIRST_F(3, 2); break;
   case 41: SOFIE_FIRST_F(4, 1); break;
   default: SOFIE_FIRST_F(4, 2); break;
   }
#undef SOFIE_FIRST_F
   SOFIE_LAUNCH_CHECK("conv3x3_first_f32_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

} // namespace sofie
