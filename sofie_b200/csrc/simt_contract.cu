// CUDA-core contraction kernels. They serve every shape the tensor-core (tcgen05) kernels do not
// take -- transposed A, K not a multiple of the TMA alignment, grouped / strided / dilated
// convolutions, the K=27 and K=9 first convolution layers -- and they are the numerical cross-check
// of the tensor-core kernels in the GPU tests. They run on the GPU; there is no CPU path.
#include "contract.cuh"

#include <cuda_fp8.h>
#include <type_traits>

using namespace sofie;

namespace sofie {

// ------------------------------------------------------------------------------------------------
// fp32 GEMM: 64x64 tile, 256 threads, 4x4 outputs per thread, K step 16.
// ------------------------------------------------------------------------------------------------
template <bool TA, bool TB>
__global__ void __launch_bounds__(256)
gemm_f32_simt_kernel(sofie_gemm_f32_desc d, const float *__restrict__ A, const float *__restrict__ B,
                     const float *__restrict__ C, float *__restrict__ Y)
{
   constexpr int BM = 64, BN = 64, BK = 16;
   __shared__ float As[BK][BM + 4];
   __shared__ float Bs[BK][BN + 4];
   const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
   const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
   float acc[4][4] = {};
   for (int k0 = 0; k0 < d.K; k0 += BK) {
      for (int i = tid; i < BM * BK; i += 256) {
         int m, k;
         if (TA) { m = i % BM; k = i / BM; } else { k = i % BK; m = i / BK; }
         int gm = m0 + m, gk = k0 + k;
         float v = 0.f;
         if (gm < d.M && gk < d.K) v = TA ? A[(size_t)gk * d.M + gm] : A[(size_t)gm * d.K + gk];
         As[k][m] = v;
      }
      for (int i = tid; i < BN * BK; i += 256) {
         int n, k;
         if (TB) { k = i % BK; n = i / BK; } else { n = i % BN; k = i / BN; }
         int gn = n0 + n, gk = k0 + k;
         float v = 0.f;
         if (gn < d.N && gk < d.K) v = TB ? B[(size_t)gn * d.K + gk] : B[(size_t)gk * d.N + gn];
         Bs[k][n] = v;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < BK; k++) {
         float a[4], b[4];
#pragma unroll
         for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
         for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
         for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
   }
#pragma unroll
   for (int i = 0; i < 4; i++) {
      int gm = m0 + ty * 4 + i;
      if (gm >= d.M) continue;
#pragma unroll
      for (int j = 0; j < 4; j++) {
         int gn = n0 + tx * 4 + j;
         if (gn >= d.N) continue;
         float y = d.alpha * acc[i][j];
         if (d.bias_kind == 1) y += d.beta * C[gn];
         else if (d.bias_kind == 2) y += d.beta * C[(size_t)gm * d.N + gn];
         if (d.relu) y = relu_ref(y);
         Y[(size_t)gm * d.N + gn] = y;
      }
   }
}

int launch_gemm_f32_simt(cudaStream_t s, const sofie_gemm_f32_desc &d, const float *A, const float *B, const float *C,
                         float *Y)
{
   dim3 grid(ceil_div(d.N, 64), ceil_div(d.M, 64));
   if (d.transA && d.transB) gemm_f32_simt_kernel<true, true><<<grid, 256, 0, s>>>(d, A, B, C, Y);
   else if (d.transA) gemm_f32_simt_kernel<true, false><<<grid, 256, 0, s>>>(d, A, B, C, Y);
   else if (d.transB) gemm_f32_simt_kernel<false, true><<<grid, 256, 0, s>>>(d, A, B, C, Y);
   else gemm_f32_simt_kernel<false, false><<<grid, 256, 0, s>>>(d, A, B, C, Y);
   SOFIE_LAUNCH_CHECK("gemm_f32_simt_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

// ------------------------------------------------------------------------------------------------
// Direct convolution, fp32 and uint8/int8. One thread = one (pooled) output position x OCB output
// channels; the weights of those channels sit in shared memory and are read as broadcasts.
// ------------------------------------------------------------------------------------------------
constexpr int kConvOCB = 16;     // output channels per block
constexpr int kConvThreads = 128;

template <typename TX, typename TW, typename TACC>
__device__ __forceinline__ void conv_accumulate(const ConvGeom &g, const TX *__restrict__ X, const TW *__restrict__ ws,
                                                int n, int cbase, int cg, int oh, int ow, int x_zp, TACC *acc)
{
   for (int c = 0; c < cg; c++) {
      for (int r = 0; r < g.kH; r++) {
         int ih = oh * g.sh - g.pad_h + r * g.dh;
         if (ih < 0 || ih >= g.H) continue;
         for (int t = 0; t < g.kW; t++) {
            int iw = ow * g.sw - g.pad_w + t * g.dw;
            if (iw < 0 || iw >= g.W) continue;
            int cc = cbase + c;
            size_t xi = g.x_nhwc ? (((size_t)n * g.H + ih) * g.W + iw) * g.C + cc
                                 : (((size_t)n * g.C + cc) * g.H + ih) * g.W + iw;
            TACC xv = (TACC)X[xi] - (TACC)x_zp;
            const TW *w = ws + ((c * g.kH + r) * g.kW + t) * kConvOCB;
#pragma unroll
            for (int o = 0; o < kConvOCB; o++) {
               if constexpr (std::is_integral_v<TACC>) acc[o] += xv * (TACC)w[o];
               else acc[o] = fmaf(xv, (TACC)w[o], acc[o]);
            }
         }
      }
   }
}

// Epilogue functors turn the accumulators of one output position into stored values.
struct EpiF32 {
   const float *bias;
   __device__ float operator()(float acc, int oc, int relu) const
   {
      float v = bias ? acc + bias[oc] : acc;
      return relu ? relu_ref(v) : v;
   }
};
struct EpiU8 {
   const float *mult;
   const int32_t *bias;
   int y_zp;
   __device__ uint8_t operator()(int acc, int oc, int relu) const
   {
      if (bias) acc += bias[oc];
      return (uint8_t)requant_u8(acc, mult[oc], y_zp, relu);
   }
};

template <typename TX, typename TW, typename TACC, typename TY, typename Epi>
__global__ void __launch_bounds__(kConvThreads)
conv2d_direct_kernel(ConvGeom g, const TX *__restrict__ X, const TW *__restrict__ Wt, Epi epi, int x_zp,
                     TY *__restrict__ Y)
{
   extern __shared__ __align__(16) unsigned char smem_raw[];
   TW *ws = reinterpret_cast<TW *>(smem_raw);
   const int cg = g.C / g.group, og = g.Cout / g.group;
   const int ocb_per_group = ceil_div(og, kConvOCB);
   const int grp = blockIdx.y / ocb_per_group;
   const int oc0 = grp * og + (blockIdx.y % ocb_per_group) * kConvOCB; // first output channel of this block
   const int oc_end = (grp + 1) * og;
   const int kk = cg * g.kH * g.kW;
   // stage weights as ws[(c,r,t)][o]
   for (int i = threadIdx.x; i < kk * kConvOCB; i += kConvThreads) {
      int o = i % kConvOCB, k = i / kConvOCB;
      int oc = oc0 + o;
      TW v = 0;
      if (oc < oc_end) {
         int t = k % g.kW, r = (k / g.kW) % g.kH, c = k / (g.kW * g.kH);
         size_t wi = g.w_packed ? (((size_t)oc * g.kH + r) * g.kW + t) * cg + c
                                : (((size_t)oc * cg + c) * g.kH + r) * g.kW + t;
         v = Wt[wi];
      }
      ws[i] = v;
   }
   __syncthreads();
   const size_t positions = (size_t)g.N * g.pH * g.pW;
   for (size_t p = blockIdx.x * (size_t)kConvThreads + threadIdx.x; p < positions;
        p += (size_t)gridDim.x * kConvThreads) {
      int pw = p % g.pW, ph = (p / g.pW) % g.pH, n = p / ((size_t)g.pW * g.pH);
      TY best[kConvOCB];
      const int taps = g.pool == 2 ? 4 : 1;
      for (int q = 0; q < taps; q++) {
         int oh = g.pool == 2 ? ph * 2 + (q >> 1) : ph, ow = g.pool == 2 ? pw * 2 + (q & 1) : pw;
         TACC acc[kConvOCB];
#pragma unroll
         for (int o = 0; o < kConvOCB; o++) acc[o] = 0;
         conv_accumulate<TX, TW, TACC>(g, X, ws, n, grp * cg, cg, oh, ow, x_zp, acc);
#pragma unroll
         for (int o = 0; o < kConvOCB; o++) {
            TY v = epi(acc[o], min(oc0 + o, g.Cout - 1), g.relu);
            best[o] = (q == 0 || v > best[o]) ? v : best[o];
         }
      }
#pragma unroll
      for (int o = 0; o < kConvOCB; o++) {
         int oc = oc0 + o;
         if (oc >= oc_end) break;
         size_t yi = g.y_nhwc ? (((size_t)n * g.pH + ph) * g.pW + pw) * g.Cout + oc
                              : (((size_t)n * g.Cout + oc) * g.pH + ph) * g.pW + pw;
         Y[yi] = best[o];
      }
   }
}

template <typename TX, typename TW, typename TACC, typename TY, typename Epi>
int launch_conv_direct(cudaStream_t s, const ConvGeom &g, const TX *X, const TW *Wt, Epi epi, int x_zp, TY *Y)
{
   const int cg = g.C / g.group, og = g.Cout / g.group;
   size_t smem = (size_t)cg * g.kH * g.kW * kConvOCB * sizeof(TW);
   if (smem > 200 * 1024) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "convolution weights slice of %zu bytes exceeds shared memory", smem);
   auto kern = conv2d_direct_kernel<TX, TW, TACC, TY, Epi>;
   if (smem > 48 * 1024) SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
   size_t positions = (size_t)g.N * g.pH * g.pW;
   if (positions == 0) return SOFIE_CUDA_OK;
   int gy = g.group * ceil_div(og, kConvOCB);
   size_t gx = ceil_div<size_t>(positions, kConvThreads);
   size_t cap = (size_t)kNumSMs * 16;
   if (gx > cap) gx = cap;
   kern<<<dim3((unsigned)gx, gy), kConvThreads, smem, s>>>(g, X, Wt, epi, x_zp, Y);
   SOFIE_LAUNCH_CHECK("conv2d_direct_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

int launch_conv2d_f32_simt(cudaStream_t s, const ConvGeom &g, const float *X, const float *W, const float *bias,
                           float *Y)
{
   const int rc = launch_conv2d_f32_first(s, g, X, W, bias, Y);
   if (rc >= 0) return rc;
   return launch_conv_direct<float, float, float, float, EpiF32>(s, g, X, W, EpiF32{bias}, 0, Y);
}
int launch_qconv2d_simt(cudaStream_t s, const ConvGeom &g, const uint8_t *X, const int8_t *W, const float *mult,
                        const int32_t *bias, int x_zp, int y_zp, uint8_t *Y)
{
   const int rc = launch_qconv2d_first(s, g, X, W, mult, bias, x_zp, y_zp, Y);
   if (rc >= 0) return rc;
   return launch_conv_direct<uint8_t, int8_t, int, uint8_t, EpiU8>(s, g, X, W, EpiU8{mult, bias, y_zp}, x_zp, Y);
}

// ------------------------------------------------------------------------------------------------
// uint8 x int8 GEMM with int32 accumulation (dp4a), W as [N,K]. 64x64 tile, K step 64 bytes.
// Computes sum_k a*w (a unsigned); the zero-point term arrives through corr[n].
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ int dp4a_u8s8(unsigned a, int b, int c)
{
   int d;
   asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
   return d;
}

template <bool WNK>
__global__ void __launch_bounds__(256)
qgemm_simt_kernel(sofie_qgemm_desc d, const uint8_t *__restrict__ A, const int8_t *__restrict__ W,
                  const float *__restrict__ mult, const int32_t *__restrict__ corr, uint8_t *__restrict__ Y, float *__restrict__ Yf32,
                  float dq_scale)
{
   constexpr int BM = 64, BN = 64, BK = 64;
   __shared__ unsigned As[BM][BK / 4 + 1];
   __shared__ int Ws[BN][BK / 4 + 1];
   const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
   const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
   int acc[4][4] = {};
   for (int k0 = 0; k0 < d.K; k0 += BK) {
      for (int i = tid; i < BM * BK; i += 256) {
         int k = i % BK, m = i / BK;
         int gm = m0 + m, gk = k0 + k;
         uint8_t v = (gm < d.M && gk < d.K) ? A[(size_t)gm * d.K + gk] : 0;
         reinterpret_cast<uint8_t *>(&As[m][0])[k] = v;
      }
      for (int i = tid; i < BN * BK; i += 256) {
         int n, k;
         if (WNK) { k = i % BK; n = i / BK; } else { n = i % BN; k = i / BN; }
         int gn = n0 + n, gk = k0 + k;
         int8_t v = 0;
         if (gn < d.N && gk < d.K) v = WNK ? W[(size_t)gn * d.K + gk] : W[(size_t)gk * d.N + gn];
         reinterpret_cast<int8_t *>(&Ws[n][0])[k] = v;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < BK / 4; k++) {
         unsigned a[4];
         int b[4];
#pragma unroll
         for (int i = 0; i < 4; i++) a[i] = As[ty * 4 + i][k];
#pragma unroll
         for (int j = 0; j < 4; j++) b[j] = Ws[tx * 4 + j][k];
#pragma unroll
         for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = dp4a_u8s8(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
   }
#pragma unroll
   for (int i = 0; i < 4; i++) {
      int gm = m0 + ty * 4 + i;
      if (gm >= d.M) continue;
#pragma unroll
      for (int j = 0; j < 4; j++) {
         int gn = n0 + tx * 4 + j;
         if (gn >= d.N) continue;
         int a = acc[i][j] + (corr ? corr[gn] : 0);
         const int q = requant_u8(a, mult[gn], d.y_zp, d.relu);
         if (Yf32) Yf32[(size_t)gm * d.N + gn] = __fmul_rn((float)(q - d.y_zp), dq_scale);
         else Y[(size_t)gm * d.N + gn] = (uint8_t)q;
      }
   }
}

int launch_qgemm_simt(cudaStream_t s, const sofie_qgemm_desc &d, const uint8_t *A, const int8_t *W, const float *mult,
                      const int32_t *corr, uint8_t *Y, float *Yf32, float dq_scale)
{
   dim3 grid(ceil_div(d.N, 64), ceil_div(d.M, 64));
   if (d.w_is_nk) qgemm_simt_kernel<true><<<grid, 256, 0, s>>>(d, A, W, mult, corr, Y, Yf32, dq_scale);
   else qgemm_simt_kernel<false><<<grid, 256, 0, s>>>(d, A, W, mult, corr, Y, Yf32, dq_scale);
   SOFIE_LAUNCH_CHECK("qgemm_simt_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

// ------------------------------------------------------------------------------------------------
// E4M3 x E4M3 GEMM on CUDA cores: decode through a 256-entry table, fp32 FMA accumulation.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float e4m3_decode(unsigned v)
{
   unsigned e = (v >> 3) & 0xF, m = v & 7;
   float r;
   if (e == 0) r = (float)m * 0.001953125f; // m * 2^-9
   else r = __uint_as_float(((e + 120u) << 23) | (m << 20));
   if (e == 0xF && m == 7) r = __uint_as_float(0x7FC00000u);
   return (v & 0x80) ? -r : r;
}

__global__ void __launch_bounds__(256)
gemm_e4m3_simt_kernel(sofie_fp8_gemm_desc d, const uint8_t *__restrict__ A, const uint8_t *__restrict__ W,
                      const float *__restrict__ bias, uint16_t *__restrict__ Ybf16, uint8_t *__restrict__ Yq, float *__restrict__ Yf32,
                      const float *__restrict__ a_scale_dev)
{
   constexpr int BM = 64, BN = 64, BK = 16;
   __shared__ float lut[256];
   __shared__ float As[BK][BM + 4];
   __shared__ float Bs[BK][BN + 4];
   const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
   lut[tid] = e4m3_decode(tid);
   __syncthreads();
   const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
   float acc[4][4] = {};
   for (int k0 = 0; k0 < d.K; k0 += BK) {
      for (int i = tid; i < BM * BK; i += 256) {
         int k = i % BK, m = i / BK, gm = m0 + m, gk = k0 + k;
         As[k][m] = (gm < d.M && gk < d.K) ? lut[A[(size_t)gm * d.K + gk]] : 0.f;
      }
      for (int i = tid; i < BN * BK; i += 256) {
         int k = i % BK, n = i / BK, gn = n0 + n, gk = k0 + k;
         Bs[k][n] = (gn < d.N && gk < d.K) ? lut[W[(size_t)gn * d.K + gk]] : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < BK; k++) {
         float a[4], b[4];
#pragma unroll
         for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
         for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
         for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
   }
   const float scale = __fmul_rn(a_scale_dev ? *a_scale_dev : d.a_scale, d.w_scale);
#pragma unroll
   for (int i = 0; i < 4; i++) {
      int gm = m0 + ty * 4 + i;
      if (gm >= d.M) continue;
#pragma unroll
      for (int j = 0; j < 4; j++) {
         int gn = n0 + tx * 4 + j;
         if (gn >= d.N) continue;
         float y = __fmul_rn(acc[i][j], scale);
         if (bias) y = __fadd_rn(y, bias[gn]);
         if (d.relu) y = relu_ref(y);
         uint16_t h = f32_to_bf16_rne(y);
         if (Ybf16) Ybf16[(size_t)gm * d.N + gn] = h;
         if (Yf32) Yf32[(size_t)gm * d.N + gn] = bf16_to_f32(h);
         if (Yq) Yq[(size_t)gm * d.N + gn] =
            (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(bf16_to_f32(h), d.q_scale), __NV_SATFINITE, __NV_E4M3);
      }
   }
}

int launch_gemm_e4m3_simt(cudaStream_t s, const sofie_fp8_gemm_desc &d, const uint8_t *A, const uint8_t *W,
                          const float *bias, uint16_t *Ybf16, uint8_t *Yq, float *Yf32, const float *a_scale_dev)
{
   dim3 grid(ceil_div(d.N, 64), ceil_div(d.M, 64));
   gemm_e4m3_simt_kernel<<<grid, 256, 0, s>>>(d, A, W, bias, Ybf16, Yq, Yf32, a_scale_dev);
   SOFIE_LAUNCH_CHECK("gemm_e4m3_simt_kernel");
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

// Weight repack [Cout, C, kH, kW] -> [Cout, kH, kW, C].
template <typename T>
__global__ void pack_ohwi_kernel(const T *__restrict__ W, T *__restrict__ P, int Cout, int C, int kH, int kW)
{
   size_t total = (size_t)Cout * C * kH * kW;
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      int c = i % C;
      size_t t = i / C;
      int s = t % kW; t /= kW;
      int r = t % kH;
      int oc = t / kH;
      P[i] = W[(((size_t)oc * C + c) * kH + r) * kW + s];
   }
}
template <typename T>
int launch_pack_ohwi(cudaStream_t s, const T *W, T *P, int Cout, int C, int kH, int kW)
{
   size_t total = (size_t)Cout * C * kH * kW;
   if (!total) return SOFIE_CUDA_OK;
   int blocks = (int)(ceil_div<size_t>(total, 256) < 1184 ? ceil_div<size_t>(total, 256) : 1184);
   pack_ohwi_kernel<T><<<blocks, 256, 0, s>>>(W, P, Cout, C, kH, kW);
   SOFIE_LAUNCH_CHECK("pack_ohwi_kernel");
   return SOFIE_CUDA_OK;
}
template int launch_pack_ohwi<float>(cudaStream_t, const float *, float *, int, int, int, int);
template int launch_pack_ohwi<int8_t>(cudaStream_t, const int8_t *, int8_t *, int, int, int, int);

} // namespace sofie
