// Tensor-core implicit-GEMM convolution for sm_100a: 3x3, stride 1, pad 1, group 1, NHWC
// activations, weights packed [Cout][3][3][Cin]. No im2col buffer exists anywhere:
//   GEMM M = 128 output pixels (a tileN x tileH x tileW patch), N = Cout, K = 9 taps x Cin.
// For tap (r,s) the A operand tile is ONE 4-D TMA box {channels, tileW, tileH, tileN} of the input
// at spatial offset (r-1, s-1): with channels innermost the box lands in shared memory as a K-major
// "pixels x channels" tile, and taps that fall outside the image are the TMA zero fill. The B tile
// is a 2-D box of the packed weights. tcgen05.mma accumulates the 9 x (Cin / chunk) stages of a
// tile in TMEM; two TMEM buffers let the epilogue of one tile overlap the MMAs of the next
// (persistent CTAs, one per SM).
//   kTF32: fp32 in / out, 3xTF32 (hi/lo split of both tiles by 8 converter warps), bias, Relu.
//   kI8  : uint8 x int8 -> int32, per-channel requantisation to uint8, Relu = max(q, zp). The input
//          zero point must be 0 (the zero fill of the halo is then exactly the padding value).
// Fused MaxPool 2x2: a warp owns 32 consecutive pixels = two (tileW 16) or four (tileW 8) image
// rows of the patch, so every 2x2 window lives in one warp and is reduced with two shuffles.
#include "umma.cuh"
#include "contract.cuh"
#include <cstdlib>
#include <type_traits>

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
constexpr int kConvEpilogueWarps = 8;                          // fp32: warps 2..9
constexpr int kConvEpilogueWarpsI8 = 16;                       // int8: warps 2..17 (no converters; requantisation and pooling are the longer epilogue)
constexpr int kConvConverterWarps = 8;                         // fp32 only: warps 10..17
constexpr int kConvIssuerB = 2 + kConvEpilogueWarpsI8;           // int8: warp of the second MMA issuer
constexpr int kConvThreadsI8 = (3 + kConvEpilogueWarpsI8) * 32;
constexpr int kConvThreadsTF32 = (2 + kConvEpilogueWarps + kConvConverterWarps) * 32;

// Walks the tiles start, start + step, ... of an (image groups x tile rows x tile columns) grid with
// adds and compares only: the roles call it once per tile on their critical path.
struct TileWalker {
   int n, th, tw;    // current tile: image group, tile row, tile column
   int dn, dth, dtw; // the stride in the same digits
   int tilesH, tilesW;
   __device__ __forceinline__ void init(int start, int step, int tiles_h, int tiles_w)
   {
      tilesH = tiles_h;
      tilesW = tiles_w;
      const int per_image = tiles_h * tiles_w;
      n = start / per_image;
      th = (start % per_image) / tiles_w;
      tw = start % tiles_w;
      dn = step / per_image;
      dth = (step % per_image) / tiles_w;
      dtw = step % tiles_w;
   }
   __device__ __forceinline__ void next()
   {
      tw += dtw;
      if (tw >= tilesW) {
         tw -= tilesW;
         th++;
      }
      th += dth;
      if (th >= tilesH) {
         th -= tilesH;
         n++;
      }
      n += dn;
   }
};

// The part of the epilogue one warp does for one finished tile: read its 32 TMEM lanes (pixels) for
// its share of the output channels, add the NACC partial accumulators, apply bias / Relu or the
// requantisation, reduce 2x2 windows by shuffles when pooling is fused, and store NHWC.
// EPI_WARPS / 4 warps share a lane quarter and split the channels among them in pieces of at least
// 16; e = index of the epilogue warp, lane_base = first TMEM lane of its quarter.
template <int KIND, int BN, int NACC, int EPI_WARPS>
__device__ __forceinline__ void conv_tile_epilogue(const ConvEpilogue &ep, const ConvTiling &tg, const float *s_bias,
                                                   const float *s_mult, const int *s_qbias, bool pool_first, uint32_t tmem_base,
                                                   int buf, int e, int lane_base, int lane, int nn, int hh, int ww, int n0, int h0,
                                                   int w0)
{
   constexpr int WPQ = EPI_WARPS / 4;                       // warps per lane quarter
   constexpr int CW = BN / WPQ >= 16 ? BN / WPQ : 16;       // channels per warp
   constexpr int CH = CW >= 32 ? 32 : 16;                   // channels per TMEM read
   const int c_begin = (e >> 2) * CW;
   if (c_begin >= BN) return;
   // (nn, hh, ww) = image, row and column inside the patch of the pixel in this thread's TMEM lane
   const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
   const int n = n0 + nn, h = h0 + hh, w = w0 + ww;
   const bool valid = n < tg.N;
   // in the pooling path that keeps all columns only the top-left pixel of each 2x2 window stores
   const bool store = valid && (!ep.pool || (((hh | ww) & 1) == 0));
   const int oH = ep.pool ? tg.H / 2 : tg.H, oW = ep.pool ? tg.W / 2 : tg.W;
   const int oh = ep.pool ? h / 2 : h, ow = ep.pool ? w / 2 : w;
   const size_t opix = ((size_t)n * oH + oh) * oW + ow;
#pragma unroll 1
   for (int c0 = c_begin; c0 < c_begin + CW; c0 += CH) {
      if (c0 >= tg.Cout) break;
      // sum of the NACC partial accumulators of this tile
      uint32_t r[CH];
      tmem_ld_cols<CH>(t_row + (uint32_t)(buf * NACC * BN + c0), r);
      if constexpr (NACC == 2) {
         uint32_t p[CH];
         tmem_ld_cols<CH>(t_row + (uint32_t)((buf * NACC + 1) * BN + c0), p);
         tmem_ld_wait();
#pragma unroll
         for (int j = 0; j < CH; j++) {
            if constexpr (KIND == kTF32) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(p[j]));
            else r[j] = (uint32_t)((int)r[j] + (int)p[j]);
         }
      } else {
         tmem_ld_wait();
#pragma unroll
         for (int a = 1; a < NACC; a++) {
            uint32_t p[CH];
            tmem_ld_cols<CH>(t_row + (uint32_t)((buf * NACC + a) * BN + c0), p);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < CH; j++) {
               if constexpr (KIND == kTF32) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(p[j]));
               else r[j] = (uint32_t)((int)r[j] + (int)p[j]);
            }
         }
      }
      if (ep.pool == 2 && pool_first) {
         // Fused 2x2 MaxPool as a reduce-scatter over the four lanes of a window (lane ^ 1 is the
         // neighbour in the row, lane ^ tileW the one in the next row): each exchange halves the
         // columns a lane keeps, so a lane ends with CH / 4 channels of its window's maximum and
         // bias, Relu and requantisation run on a quarter of the values. Taking the maximum of the
         // raw accumulators first gives the same stored values because every later step is
         // non-decreasing in the accumulator (pool_first is false when a requantisation
         // multiplier is negative; the path below then pools the finished values).
         const bool up1 = lane & 1, up2 = (lane & tg.tileW) != 0;
         uint32_t m1[CH / 2], m2[CH / 4];
#pragma unroll
         for (int i = 0; i < CH / 2; i++) {
            const uint32_t send = up1 ? r[i] : r[CH / 2 + i];
            const uint32_t mine = up1 ? r[CH / 2 + i] : r[i];
            const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 1);
            if constexpr (KIND == kTF32) m1[i] = __uint_as_float(got) > __uint_as_float(mine) ? got : mine;
            else m1[i] = (uint32_t)max((int)got, (int)mine);
         }
#pragma unroll
         for (int i = 0; i < CH / 4; i++) {
            const uint32_t send = up2 ? m1[i] : m1[CH / 4 + i];
            const uint32_t mine = up2 ? m1[CH / 4 + i] : m1[i];
            const uint32_t got = __shfl_xor_sync(0xffffffffu, send, tg.tileW);
            if constexpr (KIND == kTF32) m2[i] = __uint_as_float(got) > __uint_as_float(mine) ? got : mine;
            else m2[i] = (uint32_t)max((int)got, (int)mine);
         }
         const int col = c0 + (up1 ? CH / 2 : 0) + (up2 ? CH / 4 : 0); // first of this lane's CH / 4 channels
         const bool full = col + CH / 4 <= tg.Cout;
         if (valid) {
            if constexpr (KIND == kTF32) {
               float v[CH / 4];
#pragma unroll
               for (int i = 0; i < CH / 4; i++) {
                  const float acc = __uint_as_float(m2[i]) + s_bias[col + i];
                  v[i] = ep.relu ? relu_ref(acc) : acc;
               }
               float *y = ep.Yf + opix * tg.Cout + col;
               if (full && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
                  for (int i = 0; i < CH / 4; i += 4) *reinterpret_cast<float4 *>(y + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
               } else {
#pragma unroll
                  for (int i = 0; i < CH / 4; i++) if (col + i < tg.Cout) y[i] = v[i];
               }
            } else {
               int q[CH / 4];
#pragma unroll
               for (int i = 0; i < CH / 4; i++) q[i] = requant_u8((int)m2[i] + s_qbias[col + i], s_mult[col + i], ep.y_zp, ep.relu);
               uint8_t *y = ep.Yu8 + opix * tg.Cout + col;
               if (full && ((reinterpret_cast<uintptr_t>(y) & 3) == 0)) {
#pragma unroll
                  for (int i = 0; i < CH / 4; i += 4)
                     *reinterpret_cast<uint32_t *>(y + i) = (uint32_t)q[i] | ((uint32_t)q[i + 1] << 8) | ((uint32_t)q[i + 2] << 16) | ((uint32_t)q[i + 3] << 24);
               } else {
#pragma unroll
                  for (int i = 0; i < CH / 4; i++) if (col + i < tg.Cout) y[i] = (uint8_t)q[i];
               }
            }
         }
         continue;
      }
      const int ncols = min(CH, tg.Cout - c0);
      if constexpr (KIND == kTF32) {
         float v[CH];
#pragma unroll
         for (int j = 0; j < CH; j++) {
            float acc = __uint_as_float(r[j]) + s_bias[c0 + j];
            v[j] = ep.relu ? relu_ref(acc) : acc;
         }
         if (ep.pool) {
#pragma unroll
            for (int j = 0; j < CH; j++) {
               float o = __shfl_xor_sync(0xffffffffu, v[j], 1);
               v[j] = o > v[j] ? o : v[j];
               o = __shfl_xor_sync(0xffffffffu, v[j], tg.tileW);
               v[j] = o > v[j] ? o : v[j];
            }
         }
         if (store) {
            float *y = ep.Yf + opix * tg.Cout + c0;
            if (ncols == CH && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
               for (int j = 0; j < CH; j += 4) *reinterpret_cast<float4 *>(y + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
               for (int j = 0; j < CH; j++) if (j < ncols) y[j] = v[j];
            }
         }
      } else {
         int q[CH];
#pragma unroll
         for (int j = 0; j < CH; j++) q[j] = requant_u8((int)r[j] + s_qbias[c0 + j], s_mult[c0 + j], ep.y_zp, ep.relu);
         if (ep.pool) {
#pragma unroll
            for (int j = 0; j < CH; j++) {
               q[j] = max(q[j], __shfl_xor_sync(0xffffffffu, q[j], 1));
               q[j] = max(q[j], __shfl_xor_sync(0xffffffffu, q[j], tg.tileW));
            }
         }
         if (store) {
            uint8_t *y = ep.Yu8 + opix * tg.Cout + c0;
            uint32_t packed[CH / 4];
#pragma unroll
            for (int j = 0; j < CH; j += 4) packed[j >> 2] = (uint32_t)q[j] | ((uint32_t)q[j + 1] << 8) | ((uint32_t)q[j + 2] << 16) | ((uint32_t)q[j + 3] << 24);
            if (ncols == CH && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
               for (int j = 0; j < CH / 4; j += 4) *reinterpret_cast<uint4 *>(y + 4 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
            } else {
#pragma unroll
               for (int j = 0; j < CH; j++) if (j < ncols) y[j] = (uint8_t)q[j];
            }
         }
      }
   }
}

template <int KIND, int BN, int CB, int TPS, bool RW>
__global__ void __launch_bounds__(KIND == kTF32 ? kConvThreadsTF32 : kConvThreadsI8, 1)
umma_conv3x3_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, ConvEpilogue ep,
                    ConvTiling tg, uint32_t *status)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   constexpr int CBE = CB / ES;                         // channels per chunk
   constexpr int A_TILE = 128 * CB, B_TILE = BN * CB;
   constexpr int COPIES = (KIND == kTF32) ? 2 : 1;
   // RW (int8 only): the packed weights of all nine taps stay in shared memory for the life of the CTA and a
   // pipeline stage carries activations alone. Without it every tile fetches the weights again, which for
   // small images (many tiles, few pixels each) is half of all the bytes the kernel moves.
   static_assert(!RW || KIND == kI8, "resident weights: int8 only (the fp32 path would need their lo copies as well)");
   constexpr int SUB_BYTES = RW ? A_TILE : COPIES * (A_TILE + B_TILE); // one (tap, channel chunk): A and B tiles (+ lo copies)
   // A pipeline stage holds TPS such sub-blocks (TPS = 3: the three taps of one kernel row), so the
   // fixed cost of a stage hand-over (barrier round trip, commit) is paid once per TPS taps.
   // fp32: the three MMAs of a K step (lo x hi, hi x lo, hi x hi) rotate over NACC accumulators, which the
   // epilogue adds up, and two such sets double-buffer the tiles. int8: one accumulator per tile and up to
   // four tiles in flight, so a tile's trip through the epilogue and its barriers is hidden behind the MMAs
   // of the next ones.
   constexpr int NACC = KIND == kI8 ? 1 : (256 / BN > 6 ? 6 : 256 / BN);
   constexpr int NBUF = KIND == kI8 ? 4 : 2;
   constexpr uint32_t TMEM_COLS = KIND == kI8 ? NBUF * BN : 512;
   constexpr int EPI_WARPS = KIND == kI8 ? kConvEpilogueWarpsI8 : kConvEpilogueWarps;
   extern __shared__ unsigned char smem_raw[];
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
   __shared__ uint64_t full_bar[kConvMaxStages], conv_bar[kConvMaxStages], empty_bar[kConvMaxStages], tmem_full[NBUF], tmem_empty[NBUF], w_full;
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   __shared__ float s_bias[128], s_mult[128]; // per output channel, zero / one beyond Cout
   __shared__ int s_qbias[128];

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   SOFIE_PROF_DECL
   griddep_launch_dependents(); // the next kernel may set itself up while this one runs
   int negative_mult = 0;
   for (int c = threadIdx.x; c < 128; c += blockDim.x) {
      const bool in = c < tg.Cout;
      s_bias[c] = (KIND == kTF32 && in && ep.bias) ? ep.bias[c] : 0.f;
      s_mult[c] = (KIND == kI8 && in) ? ep.mult[c] : 0.f;
      s_qbias[c] = (KIND == kI8 && in && ep.qbias) ? ep.qbias[c] : 0;
      if (KIND == kI8 && in && !(ep.mult[c] >= 0.f)) negative_mult = 1;
   }
   const int S = tg.stages;
   const int stages_per_tile = 9 * tg.chunks / TPS; // TPS > 1 only when chunks == 1

   unsigned char *w_smem = smem;                                             // RW: 9 * chunks weight tiles
   unsigned char *ring = smem + (RW ? (size_t)9 * tg.chunks * B_TILE : 0);
   auto a_hi = [&](int s, int k) { return ring + (size_t)(s * TPS + k) * SUB_BYTES; };
   auto b_hi = [&](int s, int k) { return ring + (size_t)(s * TPS + k) * SUB_BYTES + A_TILE; };
   auto a_lo = [&](int s, int k) { return ring + (size_t)(s * TPS + k) * SUB_BYTES + A_TILE + B_TILE; };
   auto b_lo = [&](int s, int k) { return ring + (size_t)(s * TPS + k) * SUB_BYTES + 2 * A_TILE + B_TILE; };

   if (threadIdx.x == 0) {
      for (int s = 0; s < kConvMaxStages; s++) {
         mbar_init(&full_bar[s], 1);
         mbar_init(&conv_bar[s], kConvConverterWarps * 32);
         mbar_init(&empty_bar[s], 1);
      }
      for (int b = 0; b < NBUF; b++) {
         mbar_init(&tmem_full[b], 1);
         mbar_init(&tmem_empty[b], EPI_WARPS);
      }
      mbar_init(&w_full, 1);
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
   const bool pool_first = __syncthreads_or(negative_mult) == 0;
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;


   if (warp == 0) {
      // ---------------- TMA producer ----------------
      // Issuing a tensor copy costs the issuing thread a few hundred cycles, so the 2 x TPS copies of
      // a stage are issued by 2 x TPS lanes in parallel; lane 0 waits for the free slot and posts the
      // expected byte count (the phase cannot complete before that arrive, whatever the order).
      if constexpr (RW) {
         // the weights are constants: fetched before the previous kernel's output is waited for
         if (lane == 0) mbar_expect_tx(&w_full, (uint32_t)(9 * tg.chunks * B_TILE));
         __syncwarp();
         for (int item = lane; item < 9 * tg.chunks; item += 32) {
            const int tap = item / tg.chunks, ch = item - tap * tg.chunks;
            tma_load_2d(w_smem + (size_t)item * B_TILE, &tmW, tap * tg.C + ch * CBE, 0, &w_full);
         }
      }
      griddep_wait(); // the activations come after the previous kernel
      int g = 0, s = 0; // stage counter, continuous over the tiles of this CTA, and its ring slot
      uint32_t ph = 0;
      bool ok = true;
      TileWalker tw;
      tw.init(blockIdx.x, gridDim.x, tg.tilesH, tg.tilesW);
      for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x, tw.next()) {
         const int n0 = tw.n * tg.tileN, h0 = tw.th * tg.tileH, w0 = tw.tw * tg.tileW;
         for (int st = 0; st < stages_per_tile; st++, g++, ring_next(s, ph, S)) {
            if (lane == 0) {
               ok = SOFIE_PROF_WAIT(mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g));
               if (ok) mbar_expect_tx(&full_bar[s], TPS * (RW ? A_TILE : A_TILE + B_TILE));
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (RW ? lane < TPS : lane < 2 * TPS) {
               const int k = RW ? lane : lane >> 1;
               const int item = st * TPS + k;
               const int tap = tg.chunks == 1 ? item : item / tg.chunks, ch = tg.chunks == 1 ? 0 : item % tg.chunks;
               const int r = tap / 3, sx = tap - 3 * r;
               // x coordinate (channels) is a multiple of CBE, i.e. of 16 bytes; the spatial
               // coordinates may be -1 or reach H / W: those elements read as zero
               if (!RW && (lane & 1)) tma_load_2d(b_hi(s, k), &tmW, tap * tg.C + ch * CBE, 0, &full_bar[s]);
               else tma_load_4d(a_hi(s, k), &tmX, ch * CBE, w0 + sx - 1, h0 + r - 1, n0, &full_bar[s]);
            }
            __syncwarp();
         }
      }
   } else if (warp == 1 || (KIND == kI8 && warp == kConvIssuerB)) {
      // ---------------- MMA issuers ----------------
      // int8: two threads of different warps take the tiles alternately (an MMA costs the thread that issues
      // it more clocks than it occupies the tensor pipe); fp32: one thread.
      const int issuer = warp == 1 ? 0 : 1;
      if (lane == 0) {
         constexpr uint32_t idesc = make_idesc<KIND>(128, BN);
         int g = 0, lt = 0, s = 0;
         uint32_t ph = 0;
         bool ok = true;
         if constexpr (RW) ok = SOFIE_PROF_WAIT(mbar_wait(&w_full, 0, &abort_flag, status, kStatusWaitFull, 0x4000));
         for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x, lt++) {
            const int buf = lt & (NBUF - 1);
            if (KIND == kI8 && (lt & 1) != issuer) {
               // the other issuer's tile: step over its stages, still seeing each of them become ready (a parity
               // wait tells only the last two phases of a barrier apart, so no phase of a shared slot is skipped)
               for (int st = 0; st < stages_per_tile && ok; st++, g++, ring_next(s, ph, S))
                  ok = SOFIE_PROF_WAIT(mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g));
               continue;
            }
            if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_empty[buf], ((lt / NBUF) & 1) ^ 1, &abort_flag, status, kStatusWaitAccum, 0x2000 + lt))) break;
            tc_fence_after();
            const uint32_t d_base = tmem_base + (uint32_t)(buf * NACC * BN);
            int mma_idx = 0; // MMAs issued for this tile
            for (int st = 0; st < stages_per_tile; st++, g++, ring_next(s, ph, S)) {
               ok = SOFIE_PROF_WAIT((KIND == kTF32) ? mbar_wait(&conv_bar[s], ph, &abort_flag, status, kStatusWaitConv, g)
                                                    : mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g));
               if (!ok) break;
               tc_fence_after();
#pragma unroll
               for (int sub = 0; sub < TPS; sub++) {
                  const uint64_t da = make_smem_desc(smem_u32(a_hi(s, sub)), CB);
                  const uint64_t db = make_smem_desc(smem_u32(RW ? w_smem + (size_t)(st * TPS + sub) * B_TILE : b_hi(s, sub)), CB);
#pragma unroll
                  for (int k = 0; k < CB / 32; k++) {
                     const uint64_t koff = (uint64_t)(k * 2); // 32 bytes of K = 2 units of 16 bytes
                     // the first MMA into each accumulator overwrites it, the later ones add
                     auto issue = [&](uint64_t adesc, uint64_t bdesc) {
                        tc_mma<KIND>(d_base + (uint32_t)((mma_idx % NACC) * BN), adesc, bdesc, idesc, mma_idx >= NACC ? 1u : 0u);
                        mma_idx++;
                     };
                     if constexpr (KIND == kTF32) {
                        const uint64_t dal = make_smem_desc(smem_u32(a_lo(s, sub)), CB);
                        const uint64_t dbl = make_smem_desc(smem_u32(b_lo(s, sub)), CB);
                        issue(dal + koff, db + koff);
                        issue(da + koff, dbl + koff);
                        issue(da + koff, db + koff);
                     } else {
                        issue(da + koff, db + koff);
                     }
                  }
               }
               tc_commit(&empty_bar[s]);
            }
            if (ok) tc_commit(&tmem_full[buf]);
         }
      }
   } else if (KIND == kTF32 && warp >= 2 + EPI_WARPS) {
      // ---------------- converter warps (kTF32): hi/lo split of each stage ----------------
      if constexpr (KIND == kTF32) {
         constexpr int NT = kConvConverterWarps * 32;
         const int t = threadIdx.x - (2 + EPI_WARPS) * 32; // 0..NT-1
         int g = 0, s = 0;
      uint32_t ph = 0;
         bool ok = true;
         for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x) {
            for (int st = 0; st < stages_per_tile; st++, g++, ring_next(s, ph, S)) {
               if (!SOFIE_PROF_WAIT(mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g))) {
                  ok = false;
                  break;
               }
               // The split is elementwise, so the swizzled placement does not matter. All loads of
               // a thread are issued before the first conversion so that their latencies overlap.
               // the TPS sub-blocks of a stage are contiguous: element i of the hi part of sub-block k
               // sits at k*SUB_BYTES + i*16, its lo twin (A_TILE + B_TILE) bytes further
               constexpr int sub4 = (A_TILE + B_TILE) / 16, n4 = TPS * sub4;
               constexpr int PER = (n4 + NT - 1) / NT;
               float4 v[PER];
               auto at = [&](int idx) { return reinterpret_cast<float4 *>(a_hi(s, idx / sub4)) + (idx % sub4); };
#pragma unroll
               for (int i = 0; i < PER; i++)
                  if (t + i * NT < n4) v[i] = *at(t + i * NT);
#pragma unroll
               for (int i = 0; i < PER; i++) {
                  if (t + i * NT < n4) {
                     float4 *p = at(t + i * NT);
                     float4 h, l;
                     uint32_t u;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].x)); h.x = __uint_as_float(u); l.x = v[i].x - h.x;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].y)); h.y = __uint_as_float(u); l.y = v[i].y - h.y;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].z)); h.z = __uint_as_float(u); l.z = v[i].z - h.z;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].w)); h.w = __uint_as_float(u); l.w = v[i].w - h.w;
                     p[0] = h;
                     p[sub4] = l;
                  }
               }
               fence_proxy_async();
               mbar_arrive(&conv_bar[s]);
            }
         }
      }
   } else if (warp < 2 + EPI_WARPS) {
      // ---------------- epilogue warps, from warp 2 on ----------------
      // A warp reads the 32 TMEM lanes (pixels) its id modulo 4 selects; the warps of a lane
      // quarter split the output channels.
      const int e = warp - 2;
      const int lane_base = (warp & 3) * 32;
      const int pix = lane_base + lane; // pixel of the patch = TMEM lane
      const int ww = pix % tg.tileW, hh = (pix / tg.tileW) % tg.tileH, nn = pix / (tg.tileW * tg.tileH);
      TileWalker tw;
      tw.init(blockIdx.x, gridDim.x, tg.tilesH, tg.tilesW);
      int lt = 0;
      for (int tile = blockIdx.x; tile < tg.num_tiles; tile += gridDim.x, lt++, tw.next()) {
         const int buf = lt & (NBUF - 1);
         const int n0 = tw.n * tg.tileN, h0 = tw.th * tg.tileH, w0 = tw.tw * tg.tileW;
         if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_full[buf], (lt / NBUF) & 1, &abort_flag, status, kStatusWaitAccum, 0x3000 + lt))) break;
         tc_fence_after();
         conv_tile_epilogue<KIND, BN, NACC, EPI_WARPS>(ep, tg, s_bias, s_mult, s_qbias, pool_first, tmem_base, buf, e, lane_base, lane, nn, hh, ww, n0, h0, w0);
         // this warp is done with the TMEM buffer: the MMA warp may overwrite it
         tc_fence_before();
         __syncwarp();
         if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      }
   }
   SOFIE_PROF_REPORT(warp == 0 ? "producer" : ((warp == 1 || (KIND == kI8 && warp == kConvIssuerB)) ? "mma" : (warp < 2 + EPI_WARPS ? "epilogue" : "converter")));
   // A wait gives up only after about a second, long after every copy and MMA of this CTA landed.
   tc_fence_before();
   __syncthreads();
   if (warp == 1) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, TMEM_COLS);
   }
}

// ================================================================================================
// Second kernel for the same convolution: one haloed input patch per tile, resident weights.
//
// The kernel above fetches the input tile once per tap (nine overlapping boxes per channel chunk)
// and the weight tile again for every output tile; the TMA issue cost and, for fp32, the hi/lo split
// of all those bytes bound it. Here a tile is 16 rows x 8 columns of one image and its input is
// fetched ONCE, as the 18 x 10 patch including the halo (zero fill outside the image), by one TMA box per
// stage whose rows are the pixels (up to 128 bytes of channels each, the swizzle span; wider pixels are
// streamed in groups of 128 bytes):
//    patch[patch row][patch column][PB bytes of channels]      written with the swizzle of PB-byte rows
// For tap (r,s) the 128 x K operand starts at patch row r, column s: pixel (h, w) of the tile is row
//    (r + h) * 10 + (s + w)
// of that region, so the 8 pixels of one tile row are one 8-row group of the K-major swizzled layout,
// consecutive tile rows are one PATCH row (10 pixels) apart (the stride between 8-row groups), and the
// next 32 bytes of K are 32 bytes further in the row. A tap is therefore only a different start address
// of the same shared-memory bytes. This relies on the swizzle being a function of the absolute
// shared-memory address on both sides (TMA write, MMA read), which holds on B200: a descriptor may start
// at any row and step by any group stride (make_smem_desc_rows). An earlier form kept 16-byte channel
// planes in the no-swizzle layout; its boxes had 16-byte rows, and the copy engine's cost is per row.
// All 9 x C x Cout weights (and their lo parts for fp32) are loaded and split once per CTA and stay
// in shared memory; the launcher falls back to the kernel above when they do not fit.
constexpr int kPatchTileH = 16, kPatchTileW = 8;
constexpr int kPatchH = kPatchTileH + 2, kPatchW = kPatchTileW + 2;
constexpr int kPatchPixels = kPatchH * kPatchW;
constexpr int kPatchMaxStages = 8;

// warps: producer, MMA issuer, 8 epilogue + 8 converter warps (fp32) or 16 epilogue warps (int8), then the further
// MMA issuers from warp 18 on: one for fp32, three for int8 (whose MMAs are shorter than one thread can issue them)
constexpr int kPatchIssuerB = 18;
template <int KIND> constexpr int kPatchIssuers = KIND == kI8 ? 4 : 2;
template <int KIND> constexpr int kPatchThreads = (18 + kPatchIssuers<KIND> - 1) * 32;

struct PatchPlan {
   int chunks;   // weight sub-tiles per tap (rows of cb bytes)
   int cb;       // bytes per weight row chunk: 32, 64 or 128 (selects the swizzle)
   int stages;   // pipeline slots
   uint32_t stage_bytes; // one copy (hi) of a stage: the patch's pixels x the stage's bytes of channels
   uint32_t w_bytes;     // one copy (hi) of all weights
   int issuers;          // 1, 2 or (int8) 4 threads issuing the MMAs, taking the tiles in turn
   int conv_groups;      // fp32: 1 or 2 groups of converter warps (2: slots taken alternately)
};

// KPS = MMAs (32 bytes of K) per tap and stage, G = stages per tile: a stage carries 2 * KPS planes
// of the patch, so a tile with many channels is streamed in G plane groups and a slot stays small
// enough for two of them to fit beside the resident weights.
//
// fp32 (3xTF32): the weight sub-tile of a (tap, chunk) is stored as [hi rows | lo rows], 2 * BN rows
// of one operand, so ONE MMA of width 2 * BN multiplies the hi part of the patch with both (the
// patch, the larger operand, is read once for two of the three products); a second MMA of width BN
// adds lo(patch) x hi(weights). The two halves of the wide accumulator are added in the epilogue.
template <int KIND, int BN, int KPS, int G>
__global__ void __launch_bounds__(kPatchThreads<KIND>, 1)
umma_conv3x3_patch_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, ConvEpilogue ep,
                          ConvTiling tg, PatchPlan pl, uint32_t *status)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   constexpr int COPIES = (KIND == kTF32) ? 2 : 1;
   constexpr int NACC = (KIND == kTF32) ? 2 : 1;
   constexpr int PB = 32 * KPS;                              // bytes of channels per pixel and stage: 32, 64 or 128 = the swizzle span
   static_assert(PB == 32 || PB == 64 || PB == 128, "a stage row is one swizzle span");
   constexpr int KSTEPS = KPS * G;                           // MMAs per tap
   constexpr int CBK = KSTEPS * 32 >= 128 ? 128 : KSTEPS * 32; // bytes per weight row chunk (== pl.cb)
   constexpr int CHUNKS = KSTEPS * 32 / CBK;
   constexpr uint32_t B_TILE = BN * CBK;                     // one copy of a (tap, chunk) weight sub-tile
   // Accumulator buffers in tensor memory: as many tiles as fit in 512 columns, four at most. A tile's trip
   // from its last MMA through the epilogue and back to the issuer is several barrier hand-overs long; with
   // small tiles (few MMAs each) two buffers leave the tensor core waiting for that trip.
   constexpr int NBUF = (512 / (NACC * BN)) >= 4 ? 4 : 2;
   constexpr uint32_t TMEM_COLS = NBUF * NACC * BN;          // 128 ... 512 columns
   constexpr int EPI_WARPS = (KIND == kTF32) ? 8 : 16;
   constexpr int CONV_WARPS = 8;
   extern __shared__ unsigned char smem_raw[];
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
   __shared__ uint64_t full_bar[kPatchMaxStages], conv_bar[kPatchMaxStages], empty_bar[kPatchMaxStages], tmem_full[NBUF], tmem_empty[NBUF];
   __shared__ uint64_t w_full, w_conv;
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   __shared__ float s_bias[128], s_mult[128];
   __shared__ int s_qbias[128];

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   SOFIE_PROF_DECL
   griddep_launch_dependents(); // the next kernel may set itself up while this one runs
   int negative_mult = 0;
   for (int c = threadIdx.x; c < 128; c += blockDim.x) {
      const bool in = c < tg.Cout;
      s_bias[c] = (KIND == kTF32 && in && ep.bias) ? ep.bias[c] : 0.f;
      s_mult[c] = (KIND == kI8 && in) ? ep.mult[c] : 0.f;
      s_qbias[c] = (KIND == kI8 && in && ep.qbias) ? ep.qbias[c] : 0;
      if (KIND == kI8 && in && !(ep.mult[c] >= 0.f)) negative_mult = 1;
   }
   const int S = pl.stages;
   unsigned char *w_smem = smem;                                    // 9 * CHUNKS items of COPIES * B_TILE
   unsigned char *slots = smem + (size_t)COPIES * pl.w_bytes;
   auto slot_hi = [&](int s) { return slots + (size_t)s * COPIES * pl.stage_bytes; };

   if (threadIdx.x == 0) {
      for (int s = 0; s < kPatchMaxStages; s++) {
         mbar_init(&full_bar[s], 1);
         mbar_init(&conv_bar[s], CONV_WARPS * 32 / pl.conv_groups); // the converter threads that split one slot
         mbar_init(&empty_bar[s], 1);
      }
      for (int b = 0; b < NBUF; b++) {
         mbar_init(&tmem_full[b], 1);
         mbar_init(&tmem_empty[b], EPI_WARPS);
      }
      mbar_init(&w_full, 1);
      mbar_init(&w_conv, CONV_WARPS * 32);
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
   const bool pool_first = __syncthreads_or(negative_mult) == 0;
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;


   if (warp == 0) {
      // ---------------- TMA producer ----------------
      // weights: 9 x CHUNKS boxes of BN rows, all on one barrier
      if (lane == 0) mbar_expect_tx(&w_full, pl.w_bytes);
      __syncwarp();
      for (int item = lane; item < 9 * CHUNKS; item += 32) {
         const int tap = item / CHUNKS, ch = item - tap * CHUNKS;
         tma_load_2d(w_smem + (size_t)item * COPIES * B_TILE, &tmW, tap * tg.C + ch * (CBK / ES), 0, &w_full);
      }
      // everything above touched constants only; the activations are the previous kernel's output
      griddep_wait();
      // patches: one box per plane, issued by as many lanes. (A box of 16-byte rows costs the copy engine about
      // as much per row as one of long rows -- some 1.5 clocks --, which bounds this role at int8; copying the
      // pieces with cp.async from four warps instead was slower still: too few copies in flight.)
      int g = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      TileWalker tw;
      tw.init(blockIdx.x, gridDim.x, tg.tilesH, tg.tilesW);
      for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x, tw.next()) {
         const int n0 = tw.n * tg.tileN, h0 = tw.th * tg.tileH, w0 = tw.tw * tg.tileW;
         for (int grp = 0; grp < G; grp++, g++, ring_next(s, ph, S)) {
            if (lane == 0) {
               ok = SOFIE_PROF_WAIT(mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g));
               if (ok) mbar_expect_tx(&full_bar[s], (uint32_t)(kPatchPixels * PB));
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            // ONE box per stage: PB bytes of channels of every pixel of the haloed patch (channel coordinate = a multiple of
            // PB bytes; rows and columns start at -1: zero fill), written with the swizzle of its row length
            if (lane == 0) tma_load_4d(slot_hi(s), &tmX, grp * (PB / ES), w0 - 1, h0 - 1, n0, &full_bar[s]);
            __syncwarp();
         }
      }
   } else if (warp == 1 || warp >= kPatchIssuerB) {
      // ---------------- MMA issuers ----------------
      // Threads of different warps take the tiles of this CTA in turn (the accumulator buffers go round
      // with the tile count): while one waits for its barriers and commits, the others keep the tensor
      // pipe fed, which a single thread cannot -- an MMA costs the thread that issues it more clocks than
      // it occupies the pipe, and its hand-over work between two tiles leaves the pipe idle.
      const int issuer = warp == 1 ? 0 : warp - kPatchIssuerB + 1;
      const int ni = pl.issuers < NBUF ? pl.issuers : NBUF; // a buffer is never shared by two issuers
      if (lane == 0 && issuer < ni) {
         constexpr uint32_t idesc = make_idesc<KIND>(128, BN);
         constexpr uint32_t idesc_wide = make_idesc<KIND>(128, NACC * BN);
         bool ok = SOFIE_PROF_WAIT((KIND == kTF32) ? mbar_wait(&w_conv, 0, &abort_flag, status, kStatusWaitConv, 0x4000)
                                                   : mbar_wait(&w_full, 0, &abort_flag, status, kStatusWaitFull, 0x4000));
         tc_fence_after();
         // The issuing thread is the pacemaker of the whole CTA, so everything that can be is folded
         // at compile time: each MMA costs it one 32-bit add per descriptor. The address field (bits
         // 0..13, in units of 16 bytes) never carries out of its field.
         const uint64_t db0 = make_smem_desc(smem_u32(w_smem), CBK);
         const uint32_t b_hi_word = (uint32_t)(db0 >> 32), b_lo_word = (uint32_t)db0;
         const uint32_t lo16 = pl.stage_bytes >> 4; // hi -> lo copy of a slot, in 16-byte units
         int g = 0, lt = 0, s = 0;
         uint32_t ph = 0;
         for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x, lt++) {
            const int buf = lt & (NBUF - 1);
            if ((lt & (ni - 1)) != issuer) {
               // The other issuer's tile: step over its stages of the ring, but still see each of them
               // become ready. A parity wait only tells the last two phases of a barrier apart, so a
               // thread that skipped a phase of a slot it shares with the other issuer could take an
               // old completion for the one it waits for.
               for (int grp = 0; grp < G && ok; grp++, g++, ring_next(s, ph, S))
                  ok = SOFIE_PROF_WAIT((KIND == kTF32) ? mbar_wait(&conv_bar[s], ph, &abort_flag, status, kStatusWaitConv, g)
                                                       : mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g));
               continue;
            }
            if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_empty[buf], ((lt / NBUF) & 1) ^ 1, &abort_flag, status, kStatusWaitAccum, 0x2000 + lt))) break;
            const uint32_t d = tmem_base + (uint32_t)(buf * NACC * BN);
#pragma unroll
            for (int grp = 0; grp < G; grp++, g++, ring_next(s, ph, S)) {
               ok = SOFIE_PROF_WAIT((KIND == kTF32) ? mbar_wait(&conv_bar[s], ph, &abort_flag, status, kStatusWaitConv, g)
                                                    : mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g));
               if (!ok) break;
               tc_fence_after();
               // K-major rows of PB bytes in the swizzle TMA wrote them with; the eight pixels of a tile row are one 8-row
               // group, the next group is one PATCH row further (not 8 rows: the swizzle is a function of the absolute
               // shared-memory address, so a descriptor may start at any row and step by any number of rows)
               const uint64_t da0 = make_smem_desc_rows(smem_u32(slot_hi(s)), PB, kPatchW * PB);
               const uint32_t a_hi_word = (uint32_t)(da0 >> 32), a_lo_word = (uint32_t)da0;
               auto adesc = [&](uint32_t off16) { return ((uint64_t)a_hi_word << 32) | (uint64_t)(a_lo_word + off16); };
               auto bdesc = [&](uint32_t off16) { return ((uint64_t)b_hi_word << 32) | (uint64_t)(b_lo_word + off16); };
#pragma unroll
               for (int tap = 0; tap < 9; tap++) {
#pragma unroll
                  for (int kk = 0; kk < KPS; kk++) {
                     const int kb = (grp * KPS + kk) * 32; // byte offset in the K row of this tap
                     const uint32_t a16 = (uint32_t)(((tap / 3) * kPatchW + (tap % 3)) * PB + kk * 32) >> 4;
                     const uint32_t b16 = (uint32_t)((tap * CHUNKS + kb / CBK) * (COPIES * B_TILE) + kb % CBK) >> 4;
                     const uint32_t acc = (grp | tap | kk) ? 1u : 0u;
                     if constexpr (KIND == kTF32) {
                        tc_mma<KIND>(d, adesc(a16), bdesc(b16), idesc_wide, acc);     // hi x [hi | lo]
                        tc_mma<KIND>(d, adesc(a16 + lo16), bdesc(b16), idesc, 1u);     // lo x hi
                     } else {
                        tc_mma<KIND>(d, adesc(a16), bdesc(b16), idesc, acc);
                     }
                  }
               }
               tc_commit(&empty_bar[s]);
            }
            if (ok) tc_commit(&tmem_full[buf]);
         }
      }
   } else if (KIND == kTF32 && warp >= 2 + EPI_WARPS && warp < 2 + EPI_WARPS + CONV_WARPS) {
      // ---------------- converter warps (kTF32): hi/lo split, weights once, then each slot ----------------
      if constexpr (KIND == kTF32) {
         // The eight warps work as two groups of four that take the slots of the ring alternately, so
         // two slots are being split at any time: one slot's chain of load, convert, store, proxy
         // fence and arrive is latency, not throughput. The weights are split by all eight together.
         constexpr int NT_ALL = CONV_WARPS * 32, NT_GROUP = NT_ALL / 2;
         const int t_all = threadIdx.x - (2 + EPI_WARPS) * 32;
         const bool two_groups = pl.conv_groups == 2;
         const int group = two_groups ? t_all / NT_GROUP : 0, t_group = two_groups ? t_all % NT_GROUP : t_all;
         // Splits n16 16-byte groups at src in place (hi) and writes the lo parts lo_off bytes further,
         // as thread t of NT. Four independent loads per thread are issued before the first conversion.
         auto split = [&](unsigned char *src, uint32_t n16, uint32_t lo_off, int t, int NT) {
            float4 *base = reinterpret_cast<float4 *>(src);
            const uint32_t lo4 = lo_off / 16;
            for (uint32_t i0 = t; i0 < n16; i0 += 4 * NT) {
               float4 v[4];
#pragma unroll
               for (int i = 0; i < 4; i++)
                  if (i0 + i * NT < n16) v[i] = base[i0 + i * NT];
#pragma unroll
               for (int i = 0; i < 4; i++) {
                  if (i0 + i * NT < n16) {
                     float4 h, l;
                     uint32_t u;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].x)); h.x = __uint_as_float(u); l.x = v[i].x - h.x;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].y)); h.y = __uint_as_float(u); l.y = v[i].y - h.y;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].z)); h.z = __uint_as_float(u); l.z = v[i].z - h.z;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v[i].w)); h.w = __uint_as_float(u); l.w = v[i].w - h.w;
                     base[i0 + i * NT] = h;
                     base[i0 + i * NT + lo4] = l;
                  }
               }
            }
         };
         bool ok = SOFIE_PROF_WAIT(mbar_wait(&w_full, 0, &abort_flag, status, kStatusWaitFull, 0x4000));
         if (ok) {
            for (int item = 0; item < 9 * CHUNKS; item++) split(w_smem + (size_t)item * COPIES * B_TILE, B_TILE / 16, B_TILE, t_all, NT_ALL);
            fence_proxy_async();
            mbar_arrive(&w_conv);
         }
         int g = 0, s = 0;
         uint32_t ph = 0;
         for (int tile = blockIdx.x; tile < tg.num_tiles && ok; tile += gridDim.x) {
            for (int grp = 0; grp < G; grp++, g++, ring_next(s, ph, S)) {
               // every slot's arrival is observed (see the issuers: no phase of a shared barrier is skipped),
               // the other group's slots are then left to it
               if (!SOFIE_PROF_WAIT(mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g))) {
                  ok = false;
                  break;
               }
               if (two_groups && (g & 1) != group) continue;
               split(slot_hi(s), pl.stage_bytes / 16, pl.stage_bytes, t_group, two_groups ? NT_GROUP : NT_ALL);
               fence_proxy_async();
               mbar_arrive(&conv_bar[s]);
            }
         }
      }
   } else if (warp < 2 + EPI_WARPS) {
      // ---------------- epilogue warps, from warp 2 on ----------------
      const int e = warp - 2;
      const int lane_base = (warp & 3) * 32;
      const int pix = lane_base + lane; // pixel of the patch = TMEM lane
      const int ww = pix % tg.tileW, hh = (pix / tg.tileW) % tg.tileH, nn = pix / (tg.tileW * tg.tileH);
      TileWalker tw;
      tw.init(blockIdx.x, gridDim.x, tg.tilesH, tg.tilesW);
      int lt = 0;
      for (int tile = blockIdx.x; tile < tg.num_tiles; tile += gridDim.x, lt++, tw.next()) {
         const int buf = lt & (NBUF - 1);
         const int n0 = tw.n * tg.tileN, h0 = tw.th * tg.tileH, w0 = tw.tw * tg.tileW;
         if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_full[buf], (lt / NBUF) & 1, &abort_flag, status, kStatusWaitAccum, 0x3000 + lt))) break;
         tc_fence_after();
         conv_tile_epilogue<KIND, BN, NACC, EPI_WARPS>(ep, tg, s_bias, s_mult, s_qbias, pool_first, tmem_base, buf, e, lane_base, lane, nn, hh, ww, n0, h0, w0);
         tc_fence_before();
         __syncwarp();
         if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      }
   }
   SOFIE_PROF_REPORT(warp == 0 ? "producer" : ((warp == 1 || warp >= kPatchIssuerB) ? "mma" : (warp < 2 + EPI_WARPS ? "epilogue" : "converter")));
   tc_fence_before();
   __syncthreads();
   if (warp == 1) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, TMEM_COLS);
   }
}

// Launches the patch kernel when the shape belongs to it and the weights fit; returns -1 when the
// caller should use the per-tap kernel instead.
template <int KIND, int BN, int KPS, int G>
static int launch_conv_patch(cudaStream_t s, const ConvGeom &g, const void *X, const void *Wp, const ConvEpilogue &ep)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   constexpr int COPIES = (KIND == kTF32) ? 2 : 1;
   const int row_bytes = g.C * ES;
   PatchPlan pl = {};
   pl.cb = row_bytes >= 128 ? 128 : row_bytes;
   pl.chunks = row_bytes / pl.cb;
   pl.w_bytes = (uint32_t)(9 * pl.chunks * BN * pl.cb);
   // a multiple of 1024, so that every slot (and the lo copy of a slot, which the converters write at the same offset
   // from it) starts on a boundary of the widest swizzle pattern
   pl.stage_bytes = (uint32_t)((kPatchPixels * 32 * KPS + 1023) & ~1023);
   static const int issuers = [] { const char *e = getenv("SOFIE_CUDA_CONV_ISSUERS"); const int v = e ? atoi(e) : 0; return v == 1 || v == 2 || v == 4 ? v : 4; }();
   static const int groups = [] { const char *e = getenv("SOFIE_CUDA_CONV_GROUPS"); return e && atoi(e) == 1 ? 1 : 2; }();
   pl.issuers = issuers < kPatchIssuers<KIND> ? issuers : kPatchIssuers<KIND>;
   pl.conv_groups = groups;
   const long budget = 200 * 1024 - (long)COPIES * pl.w_bytes;
   const long per_stage = (long)COPIES * pl.stage_bytes;
   pl.stages = (int)(budget / per_stage);
   if (pl.stages > kPatchMaxStages) pl.stages = kPatchMaxStages;
   if (pl.stages < 2) return -1;
   ConvTiling tg = {};
   tg.N = g.N; tg.H = g.H; tg.W = g.W; tg.C = g.C; tg.Cout = g.Cout;
   tg.tileW = kPatchTileW; tg.tileH = kPatchTileH; tg.tileN = 1;
   tg.tilesW = g.W / kPatchTileW;
   tg.tilesH = g.H / kPatchTileH;
   tg.num_tiles = g.N * tg.tilesH * tg.tilesW;
   tg.chunks = pl.chunks;
   tg.stages = pl.stages;
   const CUtensorMapDataType dt = (KIND == kTF32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
   CUtensorMap tmX, tmW;
   uint64_t xdims[4] = {(uint64_t)g.C, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.N};
   uint64_t xstr[3] = {(uint64_t)g.C * ES, (uint64_t)g.W * g.C * ES, (uint64_t)g.H * g.W * g.C * ES};
   uint32_t xbox[4] = {(uint32_t)(32 * KPS / ES), (uint32_t)kPatchW, (uint32_t)kPatchH, 1u};
   int rc = make_tensor_map(&tmX, dt, 4, X, xdims, xstr, xbox, 32 * KPS);
   if (rc) return rc;
   uint64_t wdims[2] = {(uint64_t)9 * g.C, (uint64_t)g.Cout};
   uint64_t wstr[1] = {(uint64_t)9 * g.C * ES};
   uint32_t wbox[2] = {(uint32_t)(pl.cb / ES), (uint32_t)BN};
   rc = make_tensor_map(&tmW, dt, 2, Wp, wdims, wstr, wbox, pl.cb);
   if (rc) return rc;
   const int smem = (int)(COPIES * pl.w_bytes + pl.stages * per_stage) + 1024;
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int grid = tg.num_tiles < kNumSMs ? tg.num_tiles : kNumSMs;
   auto kern = umma_conv3x3_patch_kernel<KIND, BN, KPS, G>;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   SOFIE_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(kPatchThreads<KIND>), smem, s, tmX, tmW, ep, tg, pl, status));
   SOFIE_LAUNCH_CHECK("umma_conv3x3_patch_kernel");
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

// A stage carries up to 128 bytes of channels per pixel (one swizzle span); wider pixels are streamed in groups of 128.
template <int KIND, int BN>
static int try_launch_conv_patch_bn(cudaStream_t s, const ConvGeom &g, const void *X, const void *Wp, const ConvEpilogue &ep)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   switch (g.C * ES) {
   case 32: return launch_conv_patch<KIND, BN, 1, 1>(s, g, X, Wp, ep);
   case 64: return launch_conv_patch<KIND, BN, 2, 1>(s, g, X, Wp, ep);
   case 128: {
      // narrower stages when the resident weights leave room for fewer than two of the wide ones
      const int rc = launch_conv_patch<KIND, BN, 4, 1>(s, g, X, Wp, ep);
      return rc != -1 ? rc : launch_conv_patch<KIND, BN, 2, 2>(s, g, X, Wp, ep);
   }
   case 256: {
      const int rc = launch_conv_patch<KIND, BN, 4, 2>(s, g, X, Wp, ep);
      return rc != -1 ? rc : launch_conv_patch<KIND, BN, 2, 4>(s, g, X, Wp, ep);
   }
   default: return -1;
   }
}

template <int KIND>
static int try_launch_conv_patch(cudaStream_t s, const ConvGeom &g, const void *X, const void *Wp, const ConvEpilogue &ep, int BN)
{
   if (g.H % kPatchTileH != 0 || g.W % kPatchTileW != 0) return -1;
   switch (BN) {
   case 32: return try_launch_conv_patch_bn<KIND, 32>(s, g, X, Wp, ep);
   case 64: return try_launch_conv_patch_bn<KIND, 64>(s, g, X, Wp, ep);
   default: return try_launch_conv_patch_bn<KIND, 128>(s, g, X, Wp, ep);
   }
}

// ------------------------------------------------------------------------------------------------
// Weights resident in shared memory (int8, when the nine taps of all channel chunks take at most half
// of it): SOFIE_CUDA_CONV_RESIDENT_W=0 keeps the streamed form (used to compare the two).
static bool conv_resident_weights()
{
   static const bool on = [] { const char *e = getenv("SOFIE_CUDA_CONV_RESIDENT_W"); return !(e && atoi(e) == 0); }();
   return on;
}

template <int KIND, int BN, int CB, int TPS, bool RW>
static int launch_conv_tps_rw(cudaStream_t s, const CUtensorMap &tmX, const CUtensorMap &tmW, const ConvEpilogue &ep, ConvTiling tg)
{
   constexpr int COPIES = (KIND == kTF32) ? 2 : 1;
   constexpr int STAGE_BYTES = RW ? TPS * 128 * CB : TPS * COPIES * (128 + BN) * CB;
   const int w_bytes = RW ? 9 * tg.chunks * BN * CB : 0;
   int stages = (200 * 1024 - w_bytes) / STAGE_BYTES;
   if (stages > kConvMaxStages) stages = kConvMaxStages;
   if (stages < 2) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "convolution tile does not fit in shared memory");
   tg.stages = stages;
   const int smem = w_bytes + stages * STAGE_BYTES + 1024;
   auto kern = umma_conv3x3_kernel<KIND, BN, CB, TPS, RW>;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int grid = tg.num_tiles < kNumSMs ? tg.num_tiles : kNumSMs;
   SOFIE_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(KIND == kTF32 ? kConvThreadsTF32 : kConvThreadsI8), smem, s, tmX, tmW, ep, tg, status));
   SOFIE_LAUNCH_CHECK("umma_conv3x3_kernel");
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

template <int KIND, int BN, int CB, int TPS>
static int launch_conv_tps(cudaStream_t s, const CUtensorMap &tmX, const CUtensorMap &tmW, const ConvEpilogue &ep, const ConvTiling &tg)
{
   if constexpr (KIND == kI8) {
      if (conv_resident_weights() && 9 * tg.chunks * BN * CB <= 100 * 1024 && tg.num_tiles > kNumSMs)
         return launch_conv_tps_rw<KIND, BN, CB, TPS, true>(s, tmX, tmW, ep, tg);
   }
   return launch_conv_tps_rw<KIND, BN, CB, TPS, false>(s, tmX, tmW, ep, tg);
}

template <int KIND, int BN, int CB>
static int launch_conv_one(cudaStream_t s, const CUtensorMap &tmX, const CUtensorMap &tmW, const ConvEpilogue &ep, const ConvTiling &tg)
{
   // three taps per stage when one tap is a single channel chunk and three such stages still fit
   constexpr int COPIES = (KIND == kTF32) ? 2 : 1;
   constexpr bool kFits3 = 3 * 3 * COPIES * (128 + BN) * CB <= 200 * 1024;
   if constexpr (kFits3) {
      if (tg.chunks == 1) return launch_conv_tps<KIND, BN, CB, 3>(s, tmX, tmW, ep, tg);
   }
   return launch_conv_tps<KIND, BN, CB, 1>(s, tmX, tmW, ep, tg);
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

// SOFIE_CUDA_CONV_VARIANT=1 keeps every shape on the per-tap kernel (used to compare the two).
static int conv_variant()
{
   static const int v = [] { const char *e = getenv("SOFIE_CUDA_CONV_VARIANT"); return e ? atoi(e) : 0; }();
   return v;
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
   if (conv_variant() != 1) {
      const int prc = try_launch_conv_patch<KIND>(s, g, X, Wp, ep, BN);
      if (prc >= 0) return prc;
   }
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
   // fused 2x2 pooling on large enough images: the kernel whose TMEM lanes are pooling windows
   const int prc = launch_qconv2d_umma_pooled(s, g, X, W, mult, bias, x_zp, y_zp, Y);
   if (prc >= 0) return prc;
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
