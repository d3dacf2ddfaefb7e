// Tensor-core implicit-GEMM convolution for sm_100a: 3x3, stride 1, pad 1, group 1, NHWC
// activations, weights packed [Cout][3][3][Cin]. No im2col buffer exists anywhere:
//   GEMM M = 128 output pixels (a tileN x tileH x tileW patch), N = Cout, K = 9 taps x Cin.
// For tap (r,s) the A operand tile is ONE 4-D TMA box {channels, tileW, tileH, tileN} of the input
// at spatial offset (r-1, s-1): with channels innermost the box lands in shared memory as a K-major
// "pixels x channels" tile, and taps that fall outside the image are the TMA zero fill. The B tile
// is a 2-D box of the packed weights. tcgen05.mma accumulates the 9 x (Cin / chunk) stages of a
// tile in TMEM; two TMEM buffers let the epilogue of one tile overlap the MMAs of the next
// (persistent CTAs, one per SM).
//   kTF32: fp32 in / out, 3xTF32 (hi/lo split of both tiles by 4 converter warps), bias, Relu.
//   kI8  : uint8 x int8 -> int32, per-channel requantisation to uint8, Relu = max(q, zp). The input
//          zero point must be 0 (the zero fill of the halo is then exactly the padding value).
// Fused MaxPool 2x2: a warp owns 32 consecutive pixels = two (tileW 16) or four (tileW 8) image
// rows of the patch, so every 2x2 window lives in one warp and is reduced with two shuffles.
#include "umma.cuh"
#include "contract.cuh"

namespace sofie {
namespace umma {

struct ConvEpilogue {
   const float *bias;   // kTF32: per-channel bias or nullptr
   float *Yf;
   const float *mult;   // kI8: per-channel requantisation multiplier
   const int32_t *qbias; // kI8: per-channel int32 bias or nullptr
   int y_zp;
   uint8_t *Yu8;
   int relu, pool;
};

struct ConvTiling {
   int N, H, W, C, Cout;
   int tileW, tileH, tileN;  // patch of 128 pixels
   int tilesW, tilesH;       // patches per image (1 x 1 when tileN > 1)
   int num_tiles;
   int chunks;               // channel chunks per tap
   int stages;               // pipeline depth
};

constexpr int kConvMaxStages = 8;

template <int KIND, int BN, int CB>
__global__ void __launch_bounds__(KIND == kTF32 ? 320 : 192, 1)
umma_conv3x3_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, ConvEpilogue ep,
                    ConvTiling tg, uint32_t *status)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   constexpr int CBE = CB / ES;                         // channels per chunk
   constexpr int A_TILE = 128 * CB, B_TILE = BN * CB;
   constexpr int COPIES = (KIND == kTF32) ? 2 : 1;
   constexpr int STAGE_BYTES = COPIES * (A_TILE + B_TILE);
   constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
   extern __shared__ unsigned char smem_raw[];
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
   __shared__ uint64_t full_bar[kConvMaxStages], conv_bar[kConvMaxStages], empty_bar[kConvMaxStages], tmem_full[2], tmem_empty[2];
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   const int S = tg.stages;
   const int stages_per_tile = 9 * tg.chunks;

   auto a_hi = [&](int s) { return smem + (size_t)s * STAGE_BYTES; };
   auto b_hi = [&](int s) { return smem + (size_t)s * STAGE_BYTES + A_TILE; };
   auto a_lo = [&](int s) { return smem + (size_t)s * STAGE_BYTES + A_TILE + B_TILE; };
   auto b_lo = [&](int s) { return smem + (size_t)s * STAGE_BYTES + 2 * A_TILE + B_TILE; };

   if (threadIdx.x == 0) {
      for (int s = 0; s < kConvMaxStages; s++) {
         mbar_init(&full_bar[s], 1);
         mbar_init(&conv_bar[s], 128);
         mbar_init(&empty_bar[s], 1);
      }
      for (int b = 0; b < 2; b++) {
         mbar_init(&tmem_full[b], 1);
         mbar_init(&tmem_empty[b], 4);
      }
      abort_flag = 0;
      fence_mbar_init();
      prefetch_tensormap(&tmX);
      prefetch_tensormap(&tmW);
   }
   if (warp == 1) {
      tmem_alloc(&tmem_base_holder, TMEM_COLS);
      tmem_relinquish();
   }
   tc_fence_before();
   __syncthreads();
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;

   // tile -> first image, first row, first column of its patch
   auto tile_origin = [&](int tile, int &n0, int &h0, int &w0) {
      const int per_image = tg.tilesH * tg.tilesW;
      const int nb = tile / per_image, rem = tile % per_image;
      n0 = nb * tg.tileN;
      h0 = (rem / tg.tilesW) * tg.tileH;
      w0 = (rem % tg.tilesW) * tg.tileW;
   };

   if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
         int g = 0; // stage counter, continuous over the tiles of this CTA
         for (int tile = blockIdx.x; tile < tg.num_tiles; tile += gridDim.x) {
            int n0, h0, w0;
            tile_origin(tile, n0, h0, w0);
            bool ok = true;
            for (int tap = 0; tap < 9 && ok; tap++) {
               const int r = tap / 3, sx = tap % 3;
               for (int ch = 0; ch < tg.chunks; ch++, g++) {
                  const int s = g % S;
                  const uint32_t ph = (g / S) & 1;
                  if (!mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g)) {
                     ok = false;
                     break;
                  }
                  mbar_expect_tx(&full_bar[s], A_TILE + B_TILE);
                  // x coordinate (channels) is a multiple of CBE, i.e. of 16 bytes; the spatial
                  // coordinates may be -1 or reach H / W: those elements read as zero
                  tma_load_4d(a_hi(s), &tmX, ch * CBE, w0 + sx - 1, h0 + r - 1, n0, &full_bar[s]);
                  tma_load_2d(b_hi(s), &tmW, tap * tg.C + ch * CBE, 0, &full_bar[s]);
               }
            }
            if (!ok) break;
         }
      }
   } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
         constexpr uint32_t idesc = make_idesc<KIND>(128, BN);
         int g = 0, lt = 0;
         bool ok = true;
         for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x, lt++) {
            const int buf = lt & 1;
            if (!mbar_wait(&tmem_empty[buf], ((lt >> 1) & 1) ^ 1, &abort_flag, status, kStatusWaitAccum, 0x2000 + lt)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
            for (int st = 0; st < stages_per_tile; st++, g++) {
               const int s = g % S;
               const uint32_t ph = (g / S) & 1;
               ok = (KIND == kTF32) ? mbar_wait(&conv_bar[s], ph, &abort_flag, status, kStatusWaitConv, g)
                                    : mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g);
               if (!ok) break;
               tc_fence_after();
               const uint64_t da = make_smem_desc(smem_u32(a_hi(s)), CB);
               const uint64_t db = make_smem_desc(smem_u32(b_hi(s)), CB);
#pragma unroll
               for (int k = 0; k < CB / 32; k++) {
                  const uint64_t koff = (uint64_t)(k * 2); // 32 bytes of K = 2 units of 16 bytes
                  const uint32_t accumulate = (st == 0 && k == 0) ? 0u : 1u;
                  if constexpr (KIND == kTF32) {
                     const uint64_t dal = make_smem_desc(smem_u32(a_lo(s)), CB);
                     const uint64_t dbl = make_smem_desc(smem_u32(b_lo(s)), CB);
                     tc_mma<KIND>(d_tmem, dal + koff, db + koff, idesc, accumulate);
                     tc_mma<KIND>(d_tmem, da + koff, dbl + koff, idesc, 1);
                     tc_mma<KIND>(d_tmem, da + koff, db + koff, idesc, 1);
                  } else {
                     tc_mma<KIND>(d_tmem, da + koff, db + koff, idesc, accumulate);
                  }
               }
               tc_commit(&empty_bar[s]);
            }
            if (ok) tc_commit(&tmem_full[buf]);
         }
      }
   } else if (warp >= 6) {
      // ---------------- converter warps 6..9 (kTF32): hi/lo split of each stage ----------------
      if constexpr (KIND == kTF32) {
         const int t = threadIdx.x - 192; // 0..127
         int g = 0;
         bool ok = true;
         for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x) {
            for (int st = 0; st < stages_per_tile; st++, g++) {
               const int s = g % S;
               const uint32_t ph = (g / S) & 1;
               if (!mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g)) {
                  ok = false;
                  break;
               }
               float4 *hi = reinterpret_cast<float4 *>(a_hi(s));
               float4 *lo = reinterpret_cast<float4 *>(a_lo(s));
               constexpr int n4 = (A_TILE + B_TILE) / 16;
#pragma unroll 2
               for (int i = t; i < n4; i += 128) {
                  float4 v = hi[i], h, l;
                  uint32_t u;
                  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.x)); h.x = __uint_as_float(u); l.x = v.x - h.x;
                  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.y)); h.y = __uint_as_float(u); l.y = v.y - h.y;
                  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.z)); h.z = __uint_as_float(u); l.z = v.z - h.z;
                  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.w)); h.w = __uint_as_float(u); l.w = v.w - h.w;
                  hi[i] = h;
                  lo[i] = l;
               }
               fence_proxy_async();
               mbar_arrive(&conv_bar[s]);
            }
         }
      }
   } else {
      // ---------------- epilogue warps 2..5 ----------------
      const int lane_base = (warp & 3) * 32;
      const int pix = lane_base + lane; // pixel of the patch = TMEM lane
      const int ww = pix % tg.tileW, hh = (pix / tg.tileW) % tg.tileH, nn = pix / (tg.tileW * tg.tileH);
      const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
      int lt = 0;
      for (int tile = blockIdx.x; tile < tg.num_tiles; tile += gridDim.x, lt++) {
         const int buf = lt & 1;
         int n0, h0, w0;
         tile_origin(tile, n0, h0, w0);
         if (!mbar_wait(&tmem_full[buf], (lt >> 1) & 1, &abort_flag, status, kStatusWaitAccum, 0x3000 + lt)) break;
         tc_fence_after();
         const int n = n0 + nn, h = h0 + hh, w = w0 + ww;
         const bool valid = n < tg.N;
         // with pooling only the top-left pixel of each 2x2 window stores
         const bool store = valid && (!ep.pool || (((hh | ww) & 1) == 0));
         const int oH = ep.pool ? tg.H / 2 : tg.H, oW = ep.pool ? tg.W / 2 : tg.W;
         const int oh = ep.pool ? h / 2 : h, ow = ep.pool ? w / 2 : w;
         const size_t opix = ((size_t)n * oH + oh) * oW + ow;
#pragma unroll 1
         for (int c0 = 0; c0 < BN; c0 += 32) {
            if (c0 >= tg.Cout) break;
            uint32_t r[32];
            tmem_ld_32x32(t_row + (uint32_t)(buf * BN + c0), r);
            tmem_ld_wait();
            const int ncols = min(32, tg.Cout - c0);
            if constexpr (KIND == kTF32) {
               float v[32];
#pragma unroll
               for (int j = 0; j < 32; j++) {
                  float acc = __uint_as_float(r[j]);
                  if (ep.bias && j < ncols) acc += ep.bias[c0 + j];
                  v[j] = ep.relu ? relu_ref(acc) : acc;
               }
               if (ep.pool) {
#pragma unroll
                  for (int j = 0; j < 32; j++) {
                     float o = __shfl_xor_sync(0xffffffffu, v[j], 1);
                     v[j] = o > v[j] ? o : v[j];
                     o = __shfl_xor_sync(0xffffffffu, v[j], tg.tileW);
                     v[j] = o > v[j] ? o : v[j];
                  }
               }
               if (store) {
                  float *y = ep.Yf + opix * tg.Cout + c0;
                  if (ncols == 32 && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
                     for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(y + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                  } else {
#pragma unroll
                     for (int j = 0; j < 32; j++) if (j < ncols) y[j] = v[j];
                  }
               }
            } else {
               int q[32];
#pragma unroll
               for (int j = 0; j < 32; j++) {
                  q[j] = 0;
                  if (j < ncols) {
                     int acc = (int)r[j] + (ep.qbias ? ep.qbias[c0 + j] : 0);
                     q[j] = requant_u8(acc, ep.mult[c0 + j], ep.y_zp, ep.relu);
                  }
               }
               if (ep.pool) {
#pragma unroll
                  for (int j = 0; j < 32; j++) {
                     q[j] = max(q[j], __shfl_xor_sync(0xffffffffu, q[j], 1));
                     q[j] = max(q[j], __shfl_xor_sync(0xffffffffu, q[j], tg.tileW));
                  }
               }
               if (store) {
                  uint8_t *y = ep.Yu8 + opix * tg.Cout + c0;
                  uint32_t packed[8];
#pragma unroll
                  for (int j = 0; j < 32; j += 4) packed[j >> 2] = (uint32_t)q[j] | ((uint32_t)q[j + 1] << 8) | ((uint32_t)q[j + 2] << 16) | ((uint32_t)q[j + 3] << 24);
                  if (ncols == 32 && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
                     *reinterpret_cast<uint4 *>(y) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                     *reinterpret_cast<uint4 *>(y + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                  } else {
#pragma unroll
                     for (int j = 0; j < 32; j++) if (j < ncols) y[j] = (uint8_t)q[j];
                  }
               }
            }
         }
         // this warp is done with the TMEM buffer: the MMA warp may overwrite it
         tc_fence_before();
         __syncwarp();
         if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      }
   }
   // A wait gives up only after about a second, long after every copy and MMA of this CTA landed.
   tc_fence_before();
   __syncthreads();
   if (warp == 1) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, TMEM_COLS);
   }
}

// ------------------------------------------------------------------------------------------------
template <int KIND, int BN, int CB>
static int launch_conv_one(cudaStream_t s, const CUtensorMap &tmX, const CUtensorMap &tmW, const ConvEpilogue &ep, ConvTiling tg)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   constexpr int COPIES = (KIND == kTF32) ? 2 : 1;
   constexpr int STAGE_BYTES = COPIES * (128 + BN) * CB;
   (void)ES;
   int stages = (200 * 1024) / STAGE_BYTES;
   if (stages > kConvMaxStages) stages = kConvMaxStages;
   if (stages < 2) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "convolution tile does not fit in shared memory");
   tg.stages = stages;
   const int smem = stages * STAGE_BYTES + 1024;
   auto kern = umma_conv3x3_kernel<KIND, BN, CB>;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   uint32_t *status = device_status_word();
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int grid = tg.num_tiles < kNumSMs ? tg.num_tiles : kNumSMs;
   kern<<<grid, KIND == kTF32 ? 320 : 192, smem, s>>>(tmX, tmW, ep, tg, status);
   SOFIE_LAUNCH_CHECK("umma_conv3x3_kernel");
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

template <int KIND, int BN>
static int launch_conv_cb(cudaStream_t s, int cb, const CUtensorMap &tmX, const CUtensorMap &tmW, const ConvEpilogue &ep,
                          const ConvTiling &tg)
{
   switch (cb) {
   case 32: return launch_conv_one<KIND, BN, 32>(s, tmX, tmW, ep, tg);
   case 64: return launch_conv_one<KIND, BN, 64>(s, tmX, tmW, ep, tg);
   default: return launch_conv_one<KIND, BN, 128>(s, tmX, tmW, ep, tg);
   }
}

template <int KIND>
static int launch_conv(cudaStream_t s, const ConvGeom &g, const void *X, const void *Wp, const ConvEpilogue &ep)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   // ---- shape class of this kernel ----
   if (!(g.kH == 3 && g.kW == 3 && g.pad_h == 1 && g.pad_w == 1 && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1 && g.group == 1))
      return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "tensor-core convolution takes 3x3, stride 1, pad 1, group 1");
   if (!g.x_nhwc || !g.y_nhwc || !g.w_packed) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "tensor-core convolution takes NHWC tensors and packed weights");
   const int row_bytes = g.C * ES;
   const int cb = row_bytes >= 128 ? 128 : row_bytes;
   if ((cb != 32 && cb != 64 && cb != 128) || row_bytes % cb != 0)
      return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "channel count %d does not give 32/64/128-byte operand rows", g.C);
   if (g.Cout > 128 || g.Cout < 1) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "tensor-core convolution takes up to 128 output channels");
   ConvTiling tg = {};
   tg.N = g.N; tg.H = g.H; tg.W = g.W; tg.C = g.C; tg.Cout = g.Cout;
   tg.tileW = (g.W % 16 == 0) ? 16 : 8;
   if (g.W % tg.tileW != 0 || g.W < 8) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "image width %d is not a multiple of 8 or 16", g.W);
   tg.tileH = 128 / tg.tileW < g.H ? 128 / tg.tileW : g.H;
   if (g.H % tg.tileH != 0 || (128 % (tg.tileW * tg.tileH)) != 0) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "image height %d does not tile", g.H);
   tg.tileN = 128 / (tg.tileW * tg.tileH);
   if (tg.tileN > 1 && (g.H != tg.tileH || g.W != tg.tileW)) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "patch spans images only for whole images");
   if (g.pool == 2 && ((tg.tileH & 1) || (g.H & 1) || (g.W & 1))) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "fused pooling needs even extents");
   tg.tilesW = g.W / tg.tileW;
   tg.tilesH = g.H / tg.tileH;
   tg.num_tiles = ceil_div(g.N, tg.tileN) * tg.tilesH * tg.tilesW;
   tg.chunks = row_bytes / cb;
   if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(Wp) & 15))
      return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "TMA needs 16-byte aligned tensors");
   const int BN = g.Cout <= 32 ? 32 : (g.Cout <= 64 ? 64 : 128);
   // ---- tensor maps ----
   const CUtensorMapDataType dt = (KIND == kTF32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
   CUtensorMap tmX, tmW;
   uint64_t xdims[4] = {(uint64_t)g.C, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.N};
   uint64_t xstr[3] = {(uint64_t)g.C * ES, (uint64_t)g.W * g.C * ES, (uint64_t)g.H * g.W * g.C * ES};
   uint32_t xbox[4] = {(uint32_t)(cb / ES), (uint32_t)tg.tileW, (uint32_t)tg.tileH, (uint32_t)tg.tileN};
   int rc = make_tensor_map(&tmX, dt, 4, X, xdims, xstr, xbox, cb);
   if (rc) return rc;
   uint64_t wdims[2] = {(uint64_t)9 * g.C, (uint64_t)g.Cout};
   uint64_t wstr[1] = {(uint64_t)9 * g.C * ES};
   uint32_t wbox[2] = {(uint32_t)(cb / ES), (uint32_t)BN};
   rc = make_tensor_map(&tmW, dt, 2, Wp, wdims, wstr, wbox, cb);
   if (rc) return rc;
   switch (BN) {
   case 32: return launch_conv_cb<KIND, 32>(s, cb, tmX, tmW, ep, tg);
   case 64: return launch_conv_cb<KIND, 64>(s, cb, tmX, tmW, ep, tg);
   default: return launch_conv_cb<KIND, 128>(s, cb, tmX, tmW, ep, tg);
   }
}

} // namespace umma

int launch_conv2d_f32_umma(cudaStream_t s, const ConvGeom &g, const float *X, const float *W, const float *bias, float *Y)
{
   umma::ConvEpilogue ep = {};
   ep.bias = bias;
   ep.Yf = Y;
   ep.relu = g.relu;
   ep.pool = g.pool;
   return umma::launch_conv<umma::kTF32>(s, g, X, W, ep);
}

int launch_qconv2d_umma(cudaStream_t s, const ConvGeom &g, const uint8_t *X, const int8_t *W, const float *mult,
                        const int32_t *bias, int x_zp, int y_zp, uint8_t *Y)
{
   if (x_zp != 0) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "tensor-core quantised convolution needs an input zero point of 0");
   umma::ConvEpilogue ep = {};
   ep.mult = mult;
   ep.qbias = bias;
   ep.y_zp = y_zp;
   ep.Yu8 = Y;
   ep.relu = g.relu;
   ep.pool = g.pool;
   return umma::launch_conv<umma::kI8>(s, g, X, W, ep);
}

} // namespace sofie
