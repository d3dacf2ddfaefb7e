// Quantised 3x3 convolution with the 2x2 MaxPool taken inside tensor memory (sm_100a, tcgen05).
//
// The general tensor-core convolution (umma_conv.cu) maps the 128 TMEM lanes of a tile to 128 output
// pixels, so the four pixels of a pooling window sit in four lanes and its epilogue has to bring them
// together with shuffles before it can requantise: for the small channel counts of a CNN's first
// layers that epilogue, not the MMAs, sets the kernel's time. Here a tile is 32 x 16 output pixels of
// one image = 16 x 8 pooling windows, the TMEM lanes are the 128 WINDOWS, and the four pixels of a
// window are four accumulators side by side in the columns of the same lane:
//     accumulator(position (dy,dx)) [window (py,px)] [channel]  =  conv output at (2py+dy, 2px+dx)
// Each position is an implicit GEMM of its own (M = 128 windows, N = Cout, K = 9 taps x Cin) into its
// own BN columns; a thread of the epilogue reads its lane's four accumulators and the pooling is three
// integer max instructions per channel in registers, followed by one requantisation per POOLED value.
// Consecutive MMAs go to different accumulators (tap-major, position-minor order), so none waits for
// the accumulator of the one before it.
//
// Operand A without im2col: the haloed input patch of a tile (34 rows x 18 columns) is fetched once per
// tile as two TMA boxes, one with the patch's even columns and one with its odd columns (the image is
// addressed as [N][H][W/2][2][C], so a column parity is a coordinate, not a stride). In shared memory a box
// is [patch row][9 columns][C bytes], written with the swizzle of C-byte rows (C = 32 or 64); the eight
// windows of one tile row and one column parity are then eight consecutive rows = one 8-row group of the
// K-major swizzled layout, the next tile row of windows is two patch rows further (the stride between
// 8-row groups), and the next 32 bytes of K are 32 bytes further in the row. For tap (r,s) and position
// (dy,dx) the operand is therefore the SAME bytes read from the start address
//     box((dx+s) & 1) + ((dy+r) * 9 + ((dx+s) >> 1)) * C : 36 addresses, no copies
// (a descriptor may start at any row of a swizzled region: the swizzle is a function of the absolute
// shared-memory address on TMA's side and on the MMA's, see make_smem_desc_rows).
// Taps outside the image are the TMA zero fill (the input zero point must be 0, as in umma_conv.cu).
// All 9 x Cin x Cout weights stay in shared memory. No load uses cluster multicast.
//
// Roles (21 warps, one persistent CTA per SM): warp 0 TMA producer; warps 1, 18, 19, 20 MMA issuers, one per
// window position (an MMA of 64 columns occupies the tensor core for 48 clocks, its 6 KB of operands at 128
// bytes per clock, but costs the thread that issues it 80 to 90: four threads issuing side by side keep
// the pipe full, and all four work on the same tile, so a tile finishes as early as it can); warps 2..17
// epilogue in two groups of eight that take the tiles alternately (group 0 drains TMEM buffer 0 while group 1
// drains buffer 1: the latency of one tile's TMEM reads hides behind the other's arithmetic), two warps per
// lane quarter, 32 channels each. Every wait is bounded (umma::mbar_wait).
#include <type_traits>

#include "umma.cuh"
#include "contract.cuh"
#include <cstdlib>

namespace sofie {
namespace umma {

namespace {

constexpr int kPoolTileH = 32, kPoolTileW = 16;          // output pixels per tile (one image region)
constexpr int kPoolRows = kPoolTileH + 2;                // patch rows including the halo
constexpr int kPoolCols = 9;                             // columns of one parity in the patch
constexpr int kPoolBoxPixels = kPoolRows * kPoolCols;    // pixels one box (one column parity of the patch) delivers
// bytes between the two boxes of a stage: a multiple of 1024, the period of the widest swizzle pattern
__host__ __device__ constexpr int pool_box_stride(int pixel_bytes) { return (kPoolBoxPixels * pixel_bytes + 1023) / 1024 * 1024; }
constexpr int kPoolMaxStages = 4;
constexpr int kPoolThreads = 21 * 32;
constexpr int kPoolEpiWarps = 16;              // warps 2..17, two groups of eight
constexpr int kPoolFirstExtraIssuer = 18;      // warps 18, 19, 20 issue positions 1, 2, 3 (warp 1 issues position 0)

// Tiles start, start + step, ... of an (images x tile rows x tile columns) grid, walked with adds and compares only.
struct PoolTileWalker {
   int n, th, tw, dn, dth, dtw, tilesH, tilesW;
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

struct PoolConvParams {
   int N, H, W, C, Cout;
   int tilesH, tilesW, num_tiles;
   int stages;
   uint32_t w_bytes;      // all weights
   uint32_t stage_bytes;  // one patch: the boxes of its two column parities
   const float *mult;
   const int32_t *qbias;
   int y_zp, relu;
   uint8_t *Y;            // [N][H/2][W/2][Cout]
};

// Requantisation to a zero point of 0: q = clamp(rne(acc * mult), 0, 255) is ONE conversion with round-to-nearest-even and
// saturation to the uint8 range (the lower bound 0 is also the Relu of a quantised value, so `relu` changes nothing here).
// Same value as requant_u8(acc, mult, 0, relu), three instructions instead of seven.
__device__ __forceinline__ uint32_t requant_u8_zp0(int acc, float mult)
{
   uint32_t q;
   asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(__fmul_rn(__int2float_rn(acc), mult)));
   return q;
}

// The epilogue of both kernels of this file: the sixteen epilogue warps form NBUF groups that take the tiles in turn,
// group g draining TMEM buffer g (NBUF = 2: eight warps per group, two per lane quarter, BN / 2 channels each; NBUF = 4,
// possible when a tile's four accumulators are 128 columns: four warps per group, one per lane quarter, all BN
// channels). More buffers in flight hide more of the fixed latency of a tile's trip through the barriers, which is
// what bounds a kernel whose tiles carry little arithmetic. lane = pooling window; its four accumulators lie BN
// columns apart.
template <int BN, int NBUF>
__device__ __forceinline__ void pool_epilogue_warp(const PoolConvParams &p, const float *s_mult, const int *s_qbias, bool pool_first,
                                                   uint32_t tmem_base, uint64_t *tmem_full, uint64_t *tmem_empty,
                                                   volatile uint32_t *abort_flag, uint32_t *status, int warp, int lane)
{
   constexpr int WPG = kPoolEpiWarps / NBUF;        // warps per group: 8 or 4
   constexpr int CW = BN / (WPG / 4);               // channels per warp
   const int e = warp - 2;
   const int group = e / WPG;                       // which tiles (and TMEM buffer) this warp drains
   const int half = (e % WPG) >> 2;                 // which CW channels of the lane's row
   const int lane_base = (warp & 3) * 32;
   const int win = lane_base + lane;
   const int px = win & 7, py = win >> 3;
   const int oH = p.H / 2, oW = p.W / 2;
   PoolTileWalker tw;
   tw.init(blockIdx.x + group * gridDim.x, NBUF * gridDim.x, p.tilesH, p.tilesW);
   int lt = group;
   for (int tile = blockIdx.x + group * gridDim.x; tile < p.num_tiles; tile += NBUF * gridDim.x, lt += NBUF, tw.next()) {
      const int buf = group;
      if (!mbar_wait(&tmem_full[buf], (lt / NBUF) & 1, abort_flag, status, kStatusWaitAccum, 0x3000 + lt)) break;
      tc_fence_after();
      const int oh = tw.th * (kPoolTileH / 2) + py, ow = tw.tw * (kPoolTileW / 2) + px;
      uint8_t *yrow = p.Y + (((size_t)tw.n * oH + oh) * oW + ow) * p.Cout;
#pragma unroll
      for (int piece = 0; piece < CW / 16; piece++) {
         const int c0 = half * CW + piece * 16;
         if (c0 >= p.Cout) break;
         const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(buf * 4 * BN + c0);
         int q[16];
         if (pool_first) {
            uint32_t a[16], b[16];
            tmem_ld_32x16(t_row, a);
            tmem_ld_32x16(t_row + BN, b);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j++) a[j] = (uint32_t)max((int)a[j], (int)b[j]);
            uint32_t c[16];
            tmem_ld_32x16(t_row + 2 * BN, b);
            tmem_ld_32x16(t_row + 3 * BN, c);
            tmem_ld_wait();
            // four channels at a time: their multipliers (and biases) are one 16-byte shared load each (c0 is a multiple of 16)
            // four copies of the loop, chosen by two uniform branches outside it: a layer without bias does not pay an addition
            // per value, and the choice between the two requantisation forms is not made (or both computed) per value
            auto finish = [&](auto with_bias, auto zero_point_0) {
#pragma unroll
               for (int j4 = 0; j4 < 4; j4++) {
                  const float4 m4 = reinterpret_cast<const float4 *>(s_mult + c0)[j4];
                  const float mu[4] = {m4.x, m4.y, m4.z, m4.w};
                  int bi[4] = {0, 0, 0, 0};
                  if constexpr (decltype(with_bias)::value) {
                     const int4 b4 = reinterpret_cast<const int4 *>(s_qbias + c0)[j4];
                     bi[0] = b4.x; bi[1] = b4.y; bi[2] = b4.z; bi[3] = b4.w;
                  }
#pragma unroll
                  for (int t = 0; t < 4; t++) {
                     const int j = 4 * j4 + t;
                     int m = __vimax3_s32((int)a[j], (int)b[j], (int)c[j]);
                     if constexpr (decltype(with_bias)::value) m += bi[t];
                     if constexpr (decltype(zero_point_0)::value) q[j] = (int)requant_u8_zp0(m, mu[t]);
                     else q[j] = requant_u8(m, mu[t], p.y_zp, p.relu);
                  }
               }
            };
            if (p.y_zp == 0) {
               if (p.qbias != nullptr) finish(std::true_type{}, std::true_type{});
               else finish(std::false_type{}, std::true_type{});
            } else {
               if (p.qbias != nullptr) finish(std::true_type{}, std::false_type{});
               else finish(std::false_type{}, std::false_type{});
            }
         } else {
            // a negative multiplier reverses the order: requantise the four pixels, then take the maximum
#pragma unroll
            for (int pos = 0; pos < 4; pos++) {
               uint32_t a[16];
               tmem_ld_32x16(t_row + pos * BN, a);
               tmem_ld_wait();
#pragma unroll
               for (int j = 0; j < 16; j++) {
                  const int v = requant_u8((int)a[j] + s_qbias[c0 + j], s_mult[c0 + j], p.y_zp, p.relu);
                  q[j] = pos ? max(q[j], v) : v;
               }
            }
         }
         uint32_t w4[4];
#pragma unroll
         for (int j = 0; j < 4; j++)
            w4[j] = (uint32_t)q[4 * j] | ((uint32_t)q[4 * j + 1] << 8) | ((uint32_t)q[4 * j + 2] << 16) | ((uint32_t)q[4 * j + 3] << 24);
         *reinterpret_cast<uint4 *>(yrow + c0) = make_uint4(w4[0], w4[1], w4[2], w4[3]);   // Cout % 16 == 0: aligned
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
   }
}

// BN = accumulator columns per position (32 or 64 >= Cout), KPS = MMAs (32 bytes of K) per tap = Cin / 32.
template <int BN, int KPS>
__global__ void __launch_bounds__(kPoolThreads, 1)
umma_qconv3x3_pool_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, PoolConvParams p,
                          uint32_t *status)
{
   constexpr int PB = 32 * KPS;                             // bytes of channels per pixel (C of int8): a box row, one swizzle span
   static_assert(PB == 32 || PB == 64 || PB == 128, "a pixel is one swizzle span");
   constexpr uint32_t BOX_STRIDE = pool_box_stride(PB);
   constexpr int CBK = KPS * 32 >= 128 ? 128 : KPS * 32;    // bytes of one weight row chunk (selects the swizzle)
   constexpr int CHUNKS = KPS * 32 / CBK;
   constexpr uint32_t B_TILE = BN * CBK;
   constexpr uint32_t TMEM_COLS = 8 * BN;                   // two buffers of four accumulators
   extern __shared__ unsigned char smem_raw[];
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
   __shared__ uint64_t full_bar[kPoolMaxStages], empty_bar[kPoolMaxStages], tmem_full[2], tmem_empty[2], w_full;
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   __shared__ __align__(16) float s_mult[64];
   __shared__ __align__(16) int s_qbias[64];

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   griddep_launch_dependents();
   int negative_mult = 0;
   for (int c = threadIdx.x; c < 64; c += blockDim.x) {
      const bool in = c < p.Cout;
      s_mult[c] = in ? p.mult[c] : 0.f;
      s_qbias[c] = (in && p.qbias) ? p.qbias[c] : 0;
      if (in && !(p.mult[c] >= 0.f)) negative_mult = 1;
   }
   const int S = p.stages;
   unsigned char *w_smem = smem;
   unsigned char *slots = smem + p.w_bytes;

   if (threadIdx.x == 0) {
      for (int s = 0; s < kPoolMaxStages; s++) {
         mbar_init(&full_bar[s], 1);
         mbar_init(&empty_bar[s], 4);   // one commit per issuer
      }
      for (int b = 0; b < 2; b++) {
         mbar_init(&tmem_full[b], 4);   // one commit per issuer
         mbar_init(&tmem_empty[b], kPoolEpiWarps / 2);
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
   // Pooling the raw sums first is exact when every later step is non-decreasing in the sum: all multipliers >= 0.
   const bool pool_first = __syncthreads_or(negative_mult) == 0;
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;
   const int per_image = p.tilesH * p.tilesW;

   if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0) mbar_expect_tx(&w_full, p.w_bytes);
      __syncwarp();
      for (int item = lane; item < 9 * CHUNKS; item += 32) {
         const int tap = item / CHUNKS, ch = item - tap * CHUNKS;
         tma_load_2d(w_smem + (size_t)item * B_TILE, &tmW, tap * p.C + ch * CBK, 0, &w_full);
      }
      griddep_wait(); // the activations are the previous kernel's output
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x, g = 0; tile < p.num_tiles && ok; tile += gridDim.x, g++, ring_next(s, ph, S)) {
         const int n = tile / per_image, rem = tile - n * per_image;
         const int h0 = (rem / p.tilesW) * kPoolTileH, w0 = (rem % p.tilesW) * kPoolTileW;
         if (lane == 0) {
            ok = mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g);
            if (ok) mbar_expect_tx(&full_bar[s], (uint32_t)(2 * kPoolBoxPixels * PB));
         }
         ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
         if (!ok) break;
         if (lane < 2) {
            // box b = 0: patch columns w0-1, w0+1, ... (odd image columns, from pair w0/2 - 1);
            // box b = 1: patch columns w0, w0+2, ...   (even image columns, from pair w0/2).
            // A box row is one pixel with all its PB bytes of channels, written with the swizzle of that row length.
            const int b = lane;
            asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                         ::"r"(smem_u32(slots + (size_t)s * p.stage_bytes + (size_t)b * BOX_STRIDE)),
                         "l"(&tmX), "r"(0), "r"(b ? 0 : 1), "r"(b ? w0 / 2 : w0 / 2 - 1), "r"(h0 - 1), "r"(n),
                         "r"(smem_u32(&full_bar[s]))
                         : "memory");
         }
         __syncwarp();
      }
   } else if (warp == 1 || warp >= kPoolFirstExtraIssuer) {
      // ---------------- MMA issuers: thread `pos` issues the nine taps of window position pos of every tile ----------------
      const int pos = warp == 1 ? 0 : warp - kPoolFirstExtraIssuer + 1;
      if (lane == 0) {
         constexpr uint32_t idesc = make_idesc<kI8>(128, BN);
         bool ok = mbar_wait(&w_full, 0, &abort_flag, status, kStatusWaitFull, 0x4000);
         tc_fence_after();
         const uint64_t db0 = make_smem_desc(smem_u32(w_smem), CBK);
         const uint32_t b_hi_word = (uint32_t)(db0 >> 32), b_lo_word = (uint32_t)db0;
         // start of this position's operand for tap (r,s), in 16-byte units: box (dx+s) & 1, patch row dy+r, column (dx+s) >> 1
         uint32_t a_off[9];
#pragma unroll
         for (int tap = 0; tap < 9; tap++) {
            const int row = (pos >> 1) + tap / 3, e = (pos & 1) + tap % 3;
            a_off[tap] = (uint32_t)((e & 1) * BOX_STRIDE + (row * kPoolCols + (e >> 1)) * PB) >> 4;
         }
         int s = 0, lt = 0;
         uint32_t ph = 0;
         for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, lt++, ring_next(s, ph, S)) {
            const int buf = lt & 1;
            ok = mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, lt);
            if (!ok) break;
            if (!mbar_wait(&tmem_empty[buf], ((lt >> 1) & 1) ^ 1, &abort_flag, status, kStatusWaitAccum, 0x2000 + lt)) break;
            tc_fence_after();
            const uint32_t d = tmem_base + (uint32_t)(buf * 4 * BN + pos * BN);
            // swizzled K-major rows of PB bytes; the eight windows of a tile row are eight consecutive pixels of a box row, the
            // next tile row of windows is two patch rows further (make_smem_desc_rows: any start row, any group stride)
            const uint64_t da0 = make_smem_desc_rows(smem_u32(slots + (size_t)s * p.stage_bytes), PB, 2 * kPoolCols * PB);
            const uint32_t a_hi_word = (uint32_t)(da0 >> 32), a_lo_word = (uint32_t)da0;
#pragma unroll
            for (int tap = 0; tap < 9; tap++) {
#pragma unroll
               for (int kk = 0; kk < KPS; kk++) {
                  const int kb = kk * 32;
                  const uint32_t b16 = (uint32_t)((tap * CHUNKS + kb / CBK) * B_TILE + kb % CBK) >> 4;
                  const uint64_t bdesc = ((uint64_t)b_hi_word << 32) | (uint64_t)(b_lo_word + b16);
                  const uint64_t adesc = ((uint64_t)a_hi_word << 32) | (uint64_t)(a_lo_word + a_off[tap] + (uint32_t)(kk * 2));
                  tc_mma<kI8>(d, adesc, bdesc, idesc, (tap | kk) ? 1u : 0u);
               }
            }
            tc_commit(&empty_bar[s]);
            tc_commit(&tmem_full[buf]);
         }
      }
   } else if (warp < 2 + kPoolEpiWarps) {
      pool_epilogue_warp<BN, 2>(p, s_mult, s_qbias, pool_first, tmem_base, tmem_full, tmem_empty, &abort_flag, status, warp, lane);
   }
   tc_fence_before();
   __syncthreads();
   if (warp == 1) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, TMEM_COLS);
   }
}


// ================================================================================================
// First layer (ONE input channel) of the same shape class, on the same tensor-memory pooling: with C = 1 a tap is a
// single byte, far below the 16 bytes of K a shared-memory operand row needs, so here -- and only here -- the operand is
// written out: four builder warps (one thread per pooling window) read the window's 4 x 4 input bytes from the staged
// input rows and store, for each of the four window positions, the 9 taps of that position as one 16-byte operand row
// (bytes 9..15 zero). K = 32 for 8-bit MMAs: the upper 16 bytes of every row of A and of the weights are ONE shared block
// of zeros that each descriptor's leading byte offset points at. A tile is four MMAs (128 windows x BN channels x 32),
// issued by one thread; its epilogue is the one above. The input rows of a tile (34 x 48 bytes: the tile's 18 columns
// start at byte 15 so that the TMA box starts on a 16-byte boundary of the image row, as the copy engine requires)
// arrive by one TMA box per tile; out-of-image bytes are the zero fill = the padding value (input zero point 0).
// Two threads issue (even and odd tiles): a tile's two waits, four MMAs and two commits cost one thread about as long as
// the tile's epilogue takes, and the thread that issues is the pacemaker of everything behind it.
//   warp 0 producer | warps 1 and 26 MMA issuers | warps 2..17 epilogue | warps 18..25 operand builders (two groups of four)
constexpr int kFirstRawPitch = 48;                                  // bytes per staged input row
constexpr int kFirstRawBytes = kPoolRows * kFirstRawPitch;          // 1632
constexpr int kFirstRawStride = (kFirstRawBytes + 127) / 128 * 128; // 1664
constexpr int kFirstABytes = 4 * 2048;                              // four positions x 128 rows x 16 bytes
constexpr int kFirstStages = 4;
constexpr int kFirstBuilderGroups = 2;   // groups of four builder warps that take the tiles alternately
constexpr int kFirstThreads = (19 + 4 * kFirstBuilderGroups) * 32;
constexpr int kFirstBuilderWarp0 = 18;
constexpr int kFirstIssuerB = 18 + 4 * kFirstBuilderGroups;

template <int BN>
__global__ void __launch_bounds__(kFirstThreads, 1)
umma_qconv3x3_first_pool_kernel(const __grid_constant__ CUtensorMap tmX, const int8_t *__restrict__ W, PoolConvParams p, uint32_t *status)
{
   constexpr int NBUF = 512 / (4 * BN);                // tiles in flight in tensor memory: 4 (BN = 32) or 2 (BN = 64)
   constexpr uint32_t TMEM_COLS = 512;
   extern __shared__ unsigned char smem_raw[];
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
   // layout: [A slots: S x 8 KB][raw slots: S x 1664][weights: BN x 16][zeros: 2 KB]
   unsigned char *a_slots = smem;
   unsigned char *raw_slots = a_slots + kFirstStages * kFirstABytes;
   unsigned char *w_smem = raw_slots + kFirstStages * kFirstRawStride;
   unsigned char *zeros = w_smem + 1024;
   __shared__ uint64_t raw_full[kFirstStages], raw_empty[kFirstStages], a_full[kFirstStages], a_empty[kFirstStages], tmem_full[4], tmem_empty[4];
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   __shared__ __align__(16) float s_mult[64];
   __shared__ __align__(16) int s_qbias[64];

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   griddep_launch_dependents();
   int negative_mult = 0;
   for (int c = threadIdx.x; c < 64; c += blockDim.x) {
      const bool in = c < p.Cout;
      s_mult[c] = in ? p.mult[c] : 0.f;
      s_qbias[c] = (in && p.qbias) ? p.qbias[c] : 0;
      if (in && !(p.mult[c] >= 0.f)) negative_mult = 1;
   }
   // weights: row n = its nine taps and seven zeros (no-swizzle K-major: 8 rows of 16 bytes per core matrix); zero block
   for (int i = threadIdx.x; i < BN * 16; i += blockDim.x) {
      const int n = i >> 4, k = i & 15;
      w_smem[i] = (n < p.Cout && k < 9) ? (unsigned char)W[n * 9 + k] : 0;
   }
   for (int i = threadIdx.x; i < 2048 / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(zeros)[i] = 0u;
   if (threadIdx.x == 0) {
      for (int s = 0; s < kFirstStages; s++) {
         mbar_init(&raw_full[s], 1);
         mbar_init(&raw_empty[s], 4);      // one arrival per builder warp
         mbar_init(&a_full[s], 4);
         mbar_init(&a_empty[s], 1);        // the commit of the issuer that read the slot
      }
      for (int b = 0; b < NBUF; b++) {
         mbar_init(&tmem_full[b], 1);
         mbar_init(&tmem_empty[b], kPoolEpiWarps / NBUF);
      }
      abort_flag = 0;
      fence_mbar_init();
      prefetch_tensormap(&tmX);
   }
   if (warp == 1) {
      tmem_alloc(&tmem_base_holder, TMEM_COLS);
      tmem_relinquish();
   }
   fence_proxy_async(); // the weights and the zeros were written by ordinary stores; the MMAs read them through the async proxy
   tc_fence_before();
   const bool pool_first = __syncthreads_or(negative_mult) == 0;
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;
   constexpr int S = kFirstStages;

   if (warp == 0) {
      // ---------------- TMA producer: the 34 input rows of a tile ----------------
      griddep_wait(); // the input is the previous kernel's output
      if (lane == 0) {
         PoolTileWalker tw;
         tw.init(blockIdx.x, gridDim.x, p.tilesH, p.tilesW);
         int s = 0;
         uint32_t ph = 0;
         for (int tile = blockIdx.x, g = 0; tile < p.num_tiles; tile += gridDim.x, g++, ring_next(s, ph, S), tw.next()) {
            if (!mbar_wait(&raw_empty[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g)) break;
            mbar_expect_tx(&raw_full[s], kFirstRawBytes);
            // box {48 bytes, 34 rows, 1 image} from column w0 - 16 (a 16-byte boundary), row h0 - 1
            asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                         ::"r"(smem_u32(raw_slots + (size_t)s * kFirstRawStride)), "l"(&tmX), "r"(tw.tw * kPoolTileW - 16),
                         "r"(tw.th * kPoolTileH - 1), "r"(tw.n), "r"(smem_u32(&raw_full[s]))
                         : "memory");
         }
      }
   } else if (warp == 1 || warp == kFirstIssuerB) {
      // ---------------- MMA issuers: four MMAs per tile, one per window position; even tiles warp 1, odd tiles warp 22 ----------------
      // (an even number of operand slots and of TMEM buffers: each of them always meets the same issuer)
      if (lane == 0) {
         constexpr uint32_t idesc = make_idesc<kI8>(128, BN);
         const uint32_t zero_addr = smem_u32(zeros);
         const uint64_t bdesc = make_smem_desc_noswizzle(smem_u32(w_smem), zero_addr - smem_u32(w_smem), 128);
         // descriptor of the operand at a_slots (slot 0, position 0); one at `off` bytes further has its address field
         // (bits 0-13, 16-byte units) larger and its leading byte offset (bits 16-29: the distance to the zero block) smaller
         const uint64_t da0 = make_smem_desc_noswizzle(smem_u32(a_slots), zero_addr - smem_u32(a_slots), 128);
         const uint32_t a_hi_word = (uint32_t)(da0 >> 32), a_lo_word = (uint32_t)da0;
         for (int lt = (warp == 1 ? 0 : 1); blockIdx.x + (long long)lt * gridDim.x < p.num_tiles; lt += 2) {
            const int s = lt % S, buf = lt % NBUF;
            if (!mbar_wait(&a_full[s], (uint32_t)(lt / S) & 1u, &abort_flag, status, kStatusWaitFull, lt)) break;
            if (!mbar_wait(&tmem_empty[buf], (((uint32_t)(lt / NBUF)) & 1u) ^ 1u, &abort_flag, status, kStatusWaitAccum, 0x2000 + lt)) break;
            tc_fence_after();
            const uint32_t d = tmem_base + (uint32_t)(buf * 4 * BN);
            const uint32_t lo_slot = a_lo_word + (uint32_t)(s * (kFirstABytes >> 4)) * (1u - 65536u);
#pragma unroll
            for (int pos = 0; pos < 4; pos++) {
               const uint32_t lo = lo_slot + (uint32_t)(pos * (2048 >> 4)) * (1u - 65536u);
               tc_mma<kI8>(d + (uint32_t)(pos * BN), ((uint64_t)a_hi_word << 32) | lo, bdesc, idesc, 0u);
            }
            tc_commit(&a_empty[s]);
            tc_commit(&tmem_full[buf]);
         }
      }
   } else if (warp < 2 + kPoolEpiWarps) {
      pool_epilogue_warp<BN, NBUF>(p, s_mult, s_qbias, pool_first, tmem_base, tmem_full, tmem_empty, &abort_flag, status, warp, lane);
   } else {
      // ---------------- operand builders: thread = pooling window (py, px) of the tile ----------------
      // Two groups of four warps take the tiles alternately (the number of slots is even: a slot always meets the same group):
      // a group's chain of wait, load, permute, store, proxy fence and arrive is the one serial stage of a tile's way through
      // this kernel, and two tiles are in it at any time.
      const int bt = threadIdx.x - kFirstBuilderWarp0 * 32;
      const int group = bt >> 7, t = bt & 127;
      const int px = t & 7, py = t >> 3;
      // the window's 4 x 4 input bytes: patch rows 2py .. 2py+3, patch columns 2px .. 2px+3; patch column c is byte 15 + c of a staged row
      const int byte0 = 15 + 2 * px, word0 = byte0 >> 2, shift = byte0 & 3;   // shift is 1 or 3
      const uint32_t sel_row = shift == 1 ? 0x4321u : 0x6543u;                 // four bytes starting at byte `shift` of a word pair
      static_assert(kFirstStages % kFirstBuilderGroups == 0, "a slot always meets the same builder group");
      for (int g = group; blockIdx.x + (long long)g * gridDim.x < p.num_tiles; g += kFirstBuilderGroups) {
         const int s = g % S;
         const uint32_t ph = (uint32_t)(g / S) & 1u;
         if (!mbar_wait(&raw_full[s], ph, &abort_flag, status, kStatusWaitFull, 0x6000 + g)) break;
         const uint32_t *raw = reinterpret_cast<const uint32_t *>(raw_slots + (size_t)s * kFirstRawStride);
         uint32_t r[4];
#pragma unroll
         for (int i = 0; i < 4; i++) {
            const uint32_t *row = raw + (2 * py + i) * (kFirstRawPitch / 4) + word0;
            r[i] = __byte_perm(row[0], row[1], sel_row);
         }
         __syncwarp();
         if (lane == 0) mbar_arrive(&raw_empty[s]);   // the staged rows are in registers
         if (!mbar_wait(&a_empty[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, 0x7000 + g)) break;
         unsigned char *a_slot = a_slots + (size_t)s * kFirstABytes + t * 16;
#pragma unroll
         for (int pos = 0; pos < 4; pos++) {
            const int dy = pos >> 1, dx = pos & 1;
            // taps (r,s) in the order r*3+s: rows dy..dy+2 of the window, columns dx..dx+2
            // k = 0..3: columns dx, dx+1, dx+2 of window row dy, column dx of row dy+1
            const uint32_t w0 = __byte_perm(r[dy], r[dy + 1], dx ? 0x5321u : 0x4210u);
            // k = 4..7: columns dx+1, dx+2 of row dy+1, columns dx, dx+1 of row dy+2
            const uint32_t w1 = __byte_perm(r[dy + 1], r[dy + 2], dx ? 0x6532u : 0x5421u);
            // k = 8: column dx+2 of row dy+2; k = 9..15 are zero
            const uint32_t w2 = (r[dy + 2] >> (8 * (dx + 2))) & 0xffu;
            *reinterpret_cast<uint4 *>(a_slot + pos * 2048) = make_uint4(w0, w1, w2, 0u);
         }
         fence_proxy_async();
         __syncwarp();
         if (lane == 0) mbar_arrive(&a_full[s]);
      }
   }
   tc_fence_before();
   __syncthreads();
   if (warp == 1) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, TMEM_COLS);
   }
}

template <int BN>
int launch_first_pool_conv(cudaStream_t s, const ConvGeom &g, const uint8_t *X, const int8_t *W, const float *mult, const int32_t *bias,
                           int y_zp, uint8_t *Y)
{
   PoolConvParams p = {};
   p.N = g.N; p.H = g.H; p.W = g.W; p.C = 1; p.Cout = g.Cout;
   p.tilesH = g.H / kPoolTileH;
   p.tilesW = g.W / kPoolTileW;
   p.num_tiles = g.N * p.tilesH * p.tilesW;
   p.stages = kFirstStages;
   p.mult = mult; p.qbias = bias; p.y_zp = y_zp; p.relu = g.relu; p.Y = Y;
   CUtensorMap tmX;
   uint64_t xdims[3] = {(uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.N};
   uint64_t xstr[2] = {(uint64_t)g.W, (uint64_t)g.H * g.W};
   uint32_t xbox[3] = {(uint32_t)kFirstRawPitch, (uint32_t)kPoolRows, 1u};
   int rc = make_tensor_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, X, xdims, xstr, xbox, 0);
   if (rc) return rc;
   const int smem = kFirstStages * (kFirstABytes + kFirstRawStride) + 1024 + 2048 + 1024;
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int grid = p.num_tiles < kNumSMs ? p.num_tiles : kNumSMs;
   auto kern = umma_qconv3x3_first_pool_kernel<BN>;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   SOFIE_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(kFirstThreads), smem, s, tmX, W, p, status));
   SOFIE_LAUNCH_CHECK("umma_qconv3x3_first_pool_kernel");
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

template <int BN, int KPS>
int launch_pool_conv(cudaStream_t s, const ConvGeom &g, const uint8_t *X, const int8_t *Wp, const float *mult, const int32_t *bias,
                     int y_zp, uint8_t *Y)
{
   constexpr int CBK = KPS * 32 >= 128 ? 128 : KPS * 32;
   constexpr int CHUNKS = KPS * 32 / CBK;
   PoolConvParams p = {};
   p.N = g.N; p.H = g.H; p.W = g.W; p.C = g.C; p.Cout = g.Cout;
   p.tilesH = g.H / kPoolTileH;
   p.tilesW = g.W / kPoolTileW;
   p.num_tiles = g.N * p.tilesH * p.tilesW;
   p.w_bytes = (uint32_t)(9 * CHUNKS * BN * CBK);
   p.stage_bytes = (uint32_t)(2 * pool_box_stride(32 * KPS));
   p.stages = (int)((200 * 1024 - (long)p.w_bytes) / (long)p.stage_bytes);
   if (p.stages > kPoolMaxStages) p.stages = kPoolMaxStages;
   if (p.stages < 2) return -1;
   p.mult = mult; p.qbias = bias; p.y_zp = y_zp; p.relu = g.relu; p.Y = Y;
   CUtensorMap tmX, tmW;
   // the image as [N][H][W/2][2][C]: the parity of a column is a coordinate of its own
   uint64_t xdims[5] = {(uint64_t)g.C, 2u, (uint64_t)g.W / 2, (uint64_t)g.H, (uint64_t)g.N};
   uint64_t xstr[4] = {(uint64_t)g.C, (uint64_t)2 * g.C, (uint64_t)g.W * g.C, (uint64_t)g.H * g.W * g.C};
   uint32_t xbox[5] = {(uint32_t)(32 * KPS), 1u, (uint32_t)kPoolCols, (uint32_t)kPoolRows, 1u};
   int rc = make_tensor_map(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, X, xdims, xstr, xbox, 32 * KPS);
   if (rc) return rc;
   uint64_t wdims[2] = {(uint64_t)9 * g.C, (uint64_t)g.Cout};
   uint64_t wstr[1] = {(uint64_t)9 * g.C};
   uint32_t wbox[2] = {(uint32_t)CBK, (uint32_t)BN};
   rc = make_tensor_map(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, Wp, wdims, wstr, wbox, CBK);
   if (rc) return rc;
   const int smem = (int)(p.w_bytes + p.stages * p.stage_bytes) + 1024;
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int grid = p.num_tiles < kNumSMs ? p.num_tiles : kNumSMs;
   auto kern = umma_qconv3x3_pool_kernel<BN, KPS>;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   SOFIE_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(kPoolThreads), smem, s, tmX, tmW, p, status));
   SOFIE_LAUNCH_CHECK("umma_qconv3x3_pool_kernel");
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

} // namespace
} // namespace umma

// Quantised 3x3 / stride 1 / pad 1 convolution with fused Relu and MaxPool 2x2 on the pooled-window kernel.
// Returns -1 when the shape is not this kernel's (the caller then takes the general tensor-core kernel).
int launch_qconv2d_umma_pooled(cudaStream_t s, const ConvGeom &g, const uint8_t *X, const int8_t *W, const float *mult,
                               const int32_t *bias, int x_zp, int y_zp, uint8_t *Y)
{
   static const bool enabled = [] { const char *e = getenv("SOFIE_CUDA_CONV_POOLED"); return !e || atoi(e) != 0; }();
   if (!enabled || x_zp != 0 || g.pool != 2) return -1;
   if (!(g.kH == 3 && g.kW == 3 && g.pad_h == 1 && g.pad_w == 1 && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1 && g.group == 1)) return -1;
   if (g.C == 1 ? !g.y_nhwc : (!g.x_nhwc || !g.y_nhwc || !g.w_packed)) return -1;
   if (g.H % umma::kPoolTileH != 0 || g.W % umma::kPoolTileW != 0) return -1;
   if (g.Cout % 16 != 0 || g.Cout > 64) return -1;
   if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(Y) & 15)) return -1;
   const bool wide = g.Cout > 32;
   if (g.C == 1) {
      // one input channel: NCHW and NHWC are the same bytes, ONNX and packed weights too; rows must be TMA-addressable
      static const bool first = [] { const char *e = getenv("SOFIE_CUDA_FIRST_TC"); return !e || atoi(e) != 0; }();
      if (!first) return -1;
      return wide ? umma::launch_first_pool_conv<64>(s, g, X, W, mult, bias, y_zp, Y) : umma::launch_first_pool_conv<32>(s, g, X, W, mult, bias, y_zp, Y);
   }
   switch (g.C) {
   case 32: return wide ? umma::launch_pool_conv<64, 1>(s, g, X, W, mult, bias, y_zp, Y) : umma::launch_pool_conv<32, 1>(s, g, X, W, mult, bias, y_zp, Y);
   case 64: return wide ? umma::launch_pool_conv<64, 2>(s, g, X, W, mult, bias, y_zp, Y) : umma::launch_pool_conv<32, 2>(s, g, X, W, mult, bias, y_zp, Y);
   default: return -1;
   }
}

} // namespace sofie
