// Tensor-core GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T with both operands K-major in global
// memory, TMA-tiled into 128B-swizzled shared memory, multiplied by tcgen05.mma into a TMEM
// accumulator and finished by a fused epilogue. Three instantiations share one main loop:
//   kTF32 : fp32 in / fp32 out. Each operand tile is split on chip into hi = tf32(x) and
//           lo = x - hi, and the product is accumulated as lo*hi + hi*lo + hi*hi in fp32 (3xTF32).
//   kI8   : uint8 x int8 -> int32, epilogue requantises to uint8.
//   kF8   : E4M3 x E4M3 -> fp32, epilogue scales, adds bias, Relu, writes bf16 and/or E4M3.
//
// Persistent CTAs (one per SM). Warp 0 issues TMA, warp 1 allocates TMEM and issues MMA; kI8 / kF8
// have 16 epilogue warps (warps 2-17: each owns the 32 TMEM lanes its warp id modulo 4 selects and
// every fourth 32-column chunk); kTF32 has 4 epilogue warps (2-5) and 8 converter warps (6-13) that split
// every stage into hi / lo. Two TMEM accumulator buffers overlap epilogue and MMAs.
#include <cstring>

#include "umma.cuh"
#include <cstdlib>
#include "contract.cuh"

#include <cuda_fp8.h>
#include <mutex>

namespace sofie {
namespace umma {

EncodeTiledFn encode_tiled_fn()
{
   static EncodeTiledFn fn = nullptr;
   static std::once_flag once;
   std::call_once(once, [] {
      void *p = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
          q == cudaDriverEntryPointSuccess)
         fn = reinterpret_cast<EncodeTiledFn>(p);
      else
         cudaGetLastError();
   });
   return fn;
}

// A tensor map is a pure function of these arguments, and the launchers ask for the same few maps over and over (every
// eager launch of a layer: the input parts of a pipelined upload, Sessions with a run-time batch, calls from Python). A
// small per-thread table keyed by the arguments saves the driver call; a captured graph never comes back here.
namespace {
struct TensorMapKey {
   uint64_t base, dims[5], strides[4];
   uint32_t box[5];
   int32_t dtype, rank, swizzle;
   bool operator==(const TensorMapKey &o) const { return std::memcmp(this, &o, sizeof(*this)) == 0; }
};
struct TensorMapSlot {
   bool used = false;
   TensorMapKey key;
   CUtensorMap map;
};
constexpr int kTensorMapSlots = 128;
} // namespace

int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, int swizzle_bytes)
{
   EncodeTiledFn fn = encode_tiled_fn();
   if (!fn) return fail(SOFIE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
   if (rank < 1 || rank > 5) return fail(SOFIE_CUDA_ERR_INVALID, "tensor map of rank %d", rank);
   TensorMapKey key;
   std::memset(&key, 0, sizeof(key)); // padding included: the key is compared bytewise
   key.base = reinterpret_cast<uint64_t>(base);
   key.dtype = (int32_t)dtype, key.rank = rank, key.swizzle = swizzle_bytes;
   uint64_t h = key.base * 0x9E3779B97F4A7C15ull + (uint64_t)dtype * 31 + (uint64_t)swizzle_bytes;
   for (int i = 0; i < rank; i++) {
      key.dims[i] = dims[i];
      key.box[i] = box[i];
      if (i > 0) key.strides[i - 1] = strides_bytes[i - 1];
      h = (h ^ (dims[i] + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2))) * 1099511628211ull + box[i];
   }
   thread_local TensorMapSlot table[kTensorMapSlots];
   TensorMapSlot &slot = table[(h >> 17) % kTensorMapSlots];
   if (slot.used && slot.key == key) {
      *map = slot.map;
      return SOFIE_CUDA_OK;
   }
   cuuint64_t gdims[5], gstrides[5];
   cuuint32_t gbox[5], estrides[5];
   for (int i = 0; i < rank; i++) {
      gdims[i] = dims[i];
      gbox[i] = box[i];
      estrides[i] = 1;
      if (i > 0) gstrides[i - 1] = strides_bytes[i - 1];
   }
   CUtensorMapSwizzle sw = swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                           : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                           : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                 : CU_TENSOR_MAP_SWIZZLE_NONE;
   CUresult r = fn(map, dtype, (cuuint32_t)rank, const_cast<void *>(base), gdims, gstrides, gbox, estrides,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
   if (r != CUDA_SUCCESS) return fail(SOFIE_CUDA_ERR_INVALID, "cuTensorMapEncodeTiled failed with code %d", (int)r);
   slot.used = true;
   slot.key = key;
   slot.map = *map;
   return SOFIE_CUDA_OK;
}

// ------------------------------------------------------------------------------------------------
struct GemmEpilogue {
   // kTF32
   float alpha, beta;
   const float *C;
   int bias_kind;
   float *Yf;
   // kI8
   const float *mult;
   const int32_t *corr;
   int y_zp;
   uint8_t *Yu8;
   // kF8
   float scale, q_scale, q_inv; // q_inv = 1 / q_scale rounded to fp32
   const float *a_scale_dev;    // kF8: the activation scale lies in device memory (dynamic quantisation); scale = *a_scale_dev * w_scale
   float w_scale;
   const float *bias;
   uint16_t *Ybf16;
   uint8_t *Yq;
   // all
   int relu;
};

constexpr int kBM = 128;        // rows of the output tile = TMEM lanes
constexpr int kStageK = 128;    // bytes of K per pipeline stage = one 128B swizzle row
constexpr int kMmaK = 32;       // bytes of K per tcgen05.mma

template <int KIND, int BN>
struct GemmSmem {
   static constexpr int kATile = kBM * kStageK;                  // 16 KB
   static constexpr int kBTile = BN * kStageK;
   static constexpr int kCopies = (KIND == kTF32) ? 2 : 1;       // hi and lo
   static constexpr int kStageBytes = kCopies * (kATile + kBTile);
   static constexpr int stages(int budget) { return budget / kStageBytes; }
};

// x / scale for a value that is rounded to E4M3 next. The stored byte must be the one the correctly
// rounded fp32 quotient gives. x * (1 / scale) is within two units in the last place of that
// quotient, and the two can only round to different E4M3 values when they lie on different sides of
// (or on) a rounding boundary of E4M3; every such boundary, in the normal and the subnormal range,
// is an fp32 number whose low 19 mantissa bits are zero. So the product is used unless its low 19
// bits are within a few units of zero (about one value in 10^5), where the real division runs.
__device__ __forceinline__ float div_for_e4m3(float x, float scale, float inv_scale)
{
   const float q = __fmul_rn(x, inv_scale);
   if (((__float_as_uint(q) + 4u) & 0x7FFFFu) < 9u) return __fdiv_rn(x, scale);
   return q;
}

// Epilogue of 32 consecutive columns of one output row: r[j] is the raw accumulator of column
// col0 + j (fp32 bits, or int32 for kI8). The per-column constants (bias, multiplier, correction) are
// fetched once per chunk, one column per lane, and handed round through `cf`, 64 floats of shared
// memory private to the calling warp, so the loop reads them as 16-byte broadcasts instead of one
// global load per output. Vector stores when the row chunk is full and aligned. `row_ok` is false
// for the rows past M (their lanes still take part in the hand-over).
template <int KIND>
__device__ __forceinline__ void store_row_chunk(const GemmEpilogue &ep, const uint32_t (&r)[32], int row, bool row_ok, int col0, int N,
                                                float *cf, int lane)
{
   const int ncols = min(32, N - col0);
   const bool col_ok = lane < ncols;
   __syncwarp(); // the previous chunk's constants are no longer read
   if constexpr (KIND == kTF32) {
      cf[lane] = (col_ok && ep.bias_kind == 1) ? ep.C[col0 + lane] : 0.f;
   } else if constexpr (KIND == kI8) {
      cf[lane] = col_ok ? ep.mult[col0 + lane] : 0.f;
      cf[32 + lane] = __int_as_float((col_ok && ep.corr) ? ep.corr[col0 + lane] : 0);
   } else {
      cf[lane] = (col_ok && ep.bias) ? ep.bias[col0 + lane] : 0.f;
   }
   __syncwarp();
   if (!row_ok) return;
   const float4 *cf4 = reinterpret_cast<const float4 *>(cf);
   if constexpr (KIND == kTF32) {
      float *y = ep.Yf + (size_t)row * N + col0;
      float v[32];
#pragma unroll
      for (int j4 = 0; j4 < 8; j4++) {
         const float4 c = cf4[j4];
         const float cc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
         for (int t = 0; t < 4; t++) {
            const int j = 4 * j4 + t;
            float acc = ep.alpha * __uint_as_float(r[j]);
            if (ep.bias_kind == 1) acc += ep.beta * cc[t];
            else if (ep.bias_kind == 2 && j < ncols) acc += ep.beta * ep.C[(size_t)row * N + col0 + j];
            v[j] = ep.relu ? relu_ref(acc) : acc;
         }
      }
      if (ncols == 32 && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
         for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4 *>(y + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      } else {
#pragma unroll
         for (int j = 0; j < 32; j++) if (j < ncols) y[j] = v[j];
      }
   } else if constexpr (KIND == kI8) {
      if (ep.Yf) {
         // DequantizeLinear of the requantised value in the same pass: y = (q - y_zp) * scale, the float a separate
         // dequantise kernel would compute from the uint8 tensor
         float *yf = ep.Yf + (size_t)row * N + col0;
         const bool vec = ncols == 32 && ((reinterpret_cast<uintptr_t>(yf) & 15) == 0);
#pragma unroll
         for (int j4 = 0; j4 < 8; j4++) {
            const float4 m = cf4[j4], c = cf4[8 + j4];
            float4 o;
            o.x = __fmul_rn((float)(requant_u8((int)r[4 * j4 + 0] + __float_as_int(c.x), m.x, ep.y_zp, ep.relu) - ep.y_zp), ep.scale);
            o.y = __fmul_rn((float)(requant_u8((int)r[4 * j4 + 1] + __float_as_int(c.y), m.y, ep.y_zp, ep.relu) - ep.y_zp), ep.scale);
            o.z = __fmul_rn((float)(requant_u8((int)r[4 * j4 + 2] + __float_as_int(c.z), m.z, ep.y_zp, ep.relu) - ep.y_zp), ep.scale);
            o.w = __fmul_rn((float)(requant_u8((int)r[4 * j4 + 3] + __float_as_int(c.w), m.w, ep.y_zp, ep.relu) - ep.y_zp), ep.scale);
            if (vec) {
               *reinterpret_cast<float4 *>(yf + 4 * j4) = o;
            } else {
               const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
               for (int t = 0; t < 4; t++)
                  if (4 * j4 + t < ncols) yf[4 * j4 + t] = ov[t];
            }
         }
         return;
      }
      uint8_t *y = ep.Yu8 + (size_t)row * N + col0;
      uint32_t packed[8];
#pragma unroll
      for (int j4 = 0; j4 < 8; j4++) {
         const float4 m = cf4[j4], c = cf4[8 + j4];
         const int q0 = requant_u8((int)r[4 * j4 + 0] + __float_as_int(c.x), m.x, ep.y_zp, ep.relu);
         const int q1 = requant_u8((int)r[4 * j4 + 1] + __float_as_int(c.y), m.y, ep.y_zp, ep.relu);
         const int q2 = requant_u8((int)r[4 * j4 + 2] + __float_as_int(c.z), m.z, ep.y_zp, ep.relu);
         const int q3 = requant_u8((int)r[4 * j4 + 3] + __float_as_int(c.w), m.w, ep.y_zp, ep.relu);
         packed[j4] = (uint32_t)q0 | ((uint32_t)q1 << 8) | ((uint32_t)q2 << 16) | ((uint32_t)q3 << 24);
      }
      if (ncols == 32 && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
         *reinterpret_cast<uint4 *>(y) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
         *reinterpret_cast<uint4 *>(y + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      } else {
#pragma unroll
         for (int j = 0; j < 32; j++) if (j < ncols) y[j] = (uint8_t)(packed[j >> 2] >> (8 * (j & 3)));
      }
   } else {
      // y = acc * scale (+ bias) (Relu) -> bf16 (round to nearest even) -> optional E4M3 of bf16(y) / q_scale.
      // Both conversions use the paired hardware instructions (two values per instruction).
      uint32_t hb[16], qb[8];
      const float scale = ep.a_scale_dev ? __fmul_rn(__ldg(ep.a_scale_dev), ep.w_scale) : ep.scale;
#pragma unroll
      for (int j4 = 0; j4 < 8; j4++) {
         const float4 c = cf4[j4];
         const float cc[4] = {c.x, c.y, c.z, c.w};
         float yv[4];
#pragma unroll
         for (int t = 0; t < 4; t++) {
            float y = __fmul_rn(__uint_as_float(r[4 * j4 + t]), scale);
            if (ep.bias) y = __fadd_rn(y, cc[t]);
            yv[t] = ep.relu ? relu_ref(y) : y;
         }
         // cvt packs {hi, lo}: the first source lands in the upper half
         asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hb[2 * j4]) : "f"(yv[1]), "f"(yv[0]));
         asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hb[2 * j4 + 1]) : "f"(yv[3]), "f"(yv[2]));
         if (ep.Yq) {
            const float d0 = div_for_e4m3(__uint_as_float(hb[2 * j4] << 16), ep.q_scale, ep.q_inv);
            const float d1 = div_for_e4m3(__uint_as_float(hb[2 * j4] & 0xFFFF0000u), ep.q_scale, ep.q_inv);
            const float d2 = div_for_e4m3(__uint_as_float(hb[2 * j4 + 1] << 16), ep.q_scale, ep.q_inv);
            const float d3 = div_for_e4m3(__uint_as_float(hb[2 * j4 + 1] & 0xFFFF0000u), ep.q_scale, ep.q_inv);
            uint16_t lo, hi;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(d1), "f"(d0));
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d3), "f"(d2));
            qb[j4] = (uint32_t)lo | ((uint32_t)hi << 16);
         }
      }
      if (ep.Ybf16) {
         uint16_t *y = ep.Ybf16 + (size_t)row * N + col0;
         if (ncols == 32 && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 4; j++)
               reinterpret_cast<uint4 *>(y)[j] = make_uint4(hb[4 * j], hb[4 * j + 1], hb[4 * j + 2], hb[4 * j + 3]);
         } else {
#pragma unroll
            for (int j = 0; j < 32; j++) if (j < ncols) y[j] = (uint16_t)(hb[j >> 1] >> (16 * (j & 1)));
         }
      }
      if (ep.Yf) {
         // the bf16 result widened to fp32 in the same pass (a Cast behind the last layer of a chain): the low
         // 16 bits of every float are zero, the value is exactly what a separate bf16 -> float kernel would write
         float *y = ep.Yf + (size_t)row * N + col0;
         if (ncols == 32 && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 8; j++)
               reinterpret_cast<uint4 *>(y)[j] = make_uint4(hb[2 * j] << 16, hb[2 * j] & 0xFFFF0000u, hb[2 * j + 1] << 16, hb[2 * j + 1] & 0xFFFF0000u);
         } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
               if (j < ncols) y[j] = __uint_as_float((j & 1) ? (hb[j >> 1] & 0xFFFF0000u) : (hb[j >> 1] << 16));
         }
      }
      if (ep.Yq) {
         uint8_t *y = ep.Yq + (size_t)row * N + col0;
         if (ncols == 32 && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
            *reinterpret_cast<uint4 *>(y) = make_uint4(qb[0], qb[1], qb[2], qb[3]);
            *reinterpret_cast<uint4 *>(y + 16) = make_uint4(qb[4], qb[5], qb[6], qb[7]);
         } else {
#pragma unroll
            for (int j = 0; j < 32; j++) if (j < ncols) y[j] = (uint8_t)(qb[j >> 2] >> (8 * (j & 3)));
         }
      }
   }
}

// fp32 only: the tensor core adds into its accumulator with truncation, so a long K drifts (about
// 3e-5 of the result at K = 4096). The fp32 kernel therefore accumulates at most kPromoteKB stages
// (256 elements of K) in one TMEM buffer, and the epilogue warps add that partial sum into fp32
// registers with round-to-nearest while the tensor core fills the other TMEM buffer.
constexpr int kPromoteKB = 8;
constexpr int kGemmConverterWarps = 8;   // kTF32: warps 6..13 split the stages into hi / lo
constexpr int kGemmEpilogueWarps8 = 16;  // kI8 / kF8: warps 2..17 drain the accumulator
constexpr int kGemmMaxStages = 8;

template <int KIND> constexpr int gemm_threads() { return KIND == kTF32 ? (6 + kGemmConverterWarps) * 32 : (2 + kGemmEpilogueWarps8) * 32; }

// Persistent kernel: each CTA walks output tiles (N fastest, so CTAs running together share A rows
// and all of B through L2). Work is handed between the roles in "units": one unit = what is
// accumulated in one TMEM buffer before the epilogue warps drain it -- a whole tile for kI8 / kF8,
// kPromoteKB stages of a tile for kTF32. Two TMEM buffers: the MMAs of unit u+1 overlap the drain
// of unit u.
template <int KIND, int BN>
__global__ void __launch_bounds__(gemm_threads<KIND>(), 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmEpilogue ep,
                 int M, int N, int K, int S, uint32_t *status)
{
   using L = GemmSmem<KIND, BN>;
   constexpr int ES = (KIND == kTF32) ? 4 : 1;           // element size in bytes
   constexpr int KE = kStageK / ES;                      // elements of K per stage
   constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
   constexpr int EPI_WARPS = (KIND == kTF32) ? 4 : kGemmEpilogueWarps8;
   extern __shared__ unsigned char smem_raw[];
   // 1024-byte alignment: the 128B swizzle pattern repeats every 1024 bytes and is address based.
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
   __shared__ uint64_t full_bar[kGemmMaxStages], conv_bar[kGemmMaxStages], empty_bar[kGemmMaxStages], tmem_full[2], tmem_empty[2];
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   __shared__ __align__(16) float s_cf[18][64]; // per-warp hand-over of the per-column epilogue constants

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   SOFIE_PROF_DECL
   griddep_launch_dependents(); // the next kernel may set itself up while this one runs
   const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + kBM - 1) / kBM;
   const int num_tiles = tiles_m * tiles_n;
   const int num_kb = (K * ES + kStageK - 1) / kStageK;
   const int chunk_kb = (KIND == kTF32) ? kPromoteKB : num_kb; // stages accumulated in TMEM per unit
   const int units_per_tile = (num_kb + chunk_kb - 1) / chunk_kb;

   auto a_hi = [&](int s) { return smem + (size_t)s * L::kStageBytes; };
   auto b_hi = [&](int s) { return smem + (size_t)s * L::kStageBytes + L::kATile; };
   auto a_lo = [&](int s) { return smem + (size_t)s * L::kStageBytes + L::kATile + L::kBTile; };
   auto b_lo = [&](int s) { return smem + (size_t)s * L::kStageBytes + 2 * L::kATile + L::kBTile; };

   if (threadIdx.x == 0) {
      for (int s = 0; s < kGemmMaxStages; s++) {
         mbar_init(&full_bar[s], 1);
         mbar_init(&conv_bar[s], kGemmConverterWarps * 32);
         mbar_init(&empty_bar[s], 1);
      }
      for (int b = 0; b < 2; b++) {
         mbar_init(&tmem_full[b], 1);
         mbar_init(&tmem_empty[b], EPI_WARPS);
      }
      abort_flag = 0;
      fence_mbar_init();
      prefetch_tensormap(&tmA);
      prefetch_tensormap(&tmB);
   }
   if (warp == 1) {
      tmem_alloc(&tmem_base_holder, TMEM_COLS);
      tmem_relinquish();
   }
   tc_fence_before();
   __syncthreads();
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;

   if (warp == 0) {
      // ---------------- TMA producer ----------------
      // lane 0 waits for the free slot and posts the byte count; lanes 0 and 1 issue the A and the B
      // copy in parallel (issuing a tensor copy costs the issuing thread a few hundred cycles)
      griddep_wait(); // A is the previous kernel's output
      int g = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
         const int m0 = (tile / tiles_n) * kBM, n0 = (tile % tiles_n) * BN;
         for (int kb = 0; kb < num_kb; kb++, g++, ring_next(s, ph, S)) {
            if (lane == 0) {
               ok = SOFIE_PROF_WAIT(mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g));
               if (ok) mbar_expect_tx(&full_bar[s], L::kATile + L::kBTile);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) tma_load_2d(a_hi(s), &tmA, kb * KE, m0, &full_bar[s]);
            else if (lane == 1) tma_load_2d(b_hi(s), &tmB, kb * KE, n0, &full_bar[s]);
            __syncwarp();
         }
      }
   } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
         constexpr uint32_t idesc = make_idesc<KIND>(kBM, BN);
         int g = 0, u = 0, s = 0;
         uint32_t ph = 0;
         bool ok = true;
         for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int c = 0; c < units_per_tile && ok; c++, u++) {
               const int buf = u & 1;
               if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_empty[buf], ((u >> 1) & 1) ^ 1, &abort_flag, status, kStatusWaitAccum, 0x1000 + u))) {
                  ok = false;
                  break;
               }
               tc_fence_after();
               const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
               const int kb_end = min(num_kb, (c + 1) * chunk_kb);
               for (int kb = c * chunk_kb; kb < kb_end; kb++, g++, ring_next(s, ph, S)) {
                  ok = SOFIE_PROF_WAIT((KIND == kTF32) ? mbar_wait(&conv_bar[s], ph, &abort_flag, status, kStatusWaitConv, g)
                                                       : mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g));
                  if (!ok) break;
                  tc_fence_after();
                  const uint64_t da = make_smem_desc(smem_u32(a_hi(s)), kStageK);
                  const uint64_t db = make_smem_desc(smem_u32(b_hi(s)), kStageK);
#pragma unroll
                  for (int k = 0; k < kStageK / kMmaK; k++) {
                     // advancing K inside the swizzle row: +32 bytes = +2 in the (>>4) address field
                     const uint64_t koff = (uint64_t)(k * (kMmaK >> 4));
                     const uint32_t accumulate = (kb == c * chunk_kb && k == 0) ? 0u : 1u;
                     if constexpr (KIND == kTF32) {
                        const uint64_t dal = make_smem_desc(smem_u32(a_lo(s)), kStageK);
                        const uint64_t dbl = make_smem_desc(smem_u32(b_lo(s)), kStageK);
                        tc_mma<KIND>(d_tmem, dal + koff, db + koff, idesc, accumulate);
                        tc_mma<KIND>(d_tmem, da + koff, dbl + koff, idesc, 1);
                        tc_mma<KIND>(d_tmem, da + koff, db + koff, idesc, 1);
                     } else {
                        tc_mma<KIND>(d_tmem, da + koff, db + koff, idesc, accumulate);
                     }
                  }
                  tc_commit(&empty_bar[s]); // the stage is free once these MMAs have read it
               }
               if (ok) tc_commit(&tmem_full[buf]);
            }
         }
      }
   } else if (warp >= 2 + EPI_WARPS) {
      // ---------------- converter warps (kTF32): hi / lo split of every stage ----------------
      if constexpr (KIND == kTF32) {
         constexpr int NT = kGemmConverterWarps * 32;
         const int t = threadIdx.x - (2 + EPI_WARPS) * 32;
         int g = 0, s = 0;
      uint32_t ph = 0;
         bool ok = true;
         for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; kb++, g++, ring_next(s, ph, S)) {
               if (!SOFIE_PROF_WAIT(mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g))) {
                  ok = false;
                  break;
               }
               // The split is elementwise, so the swizzled placement does not matter: the lo tile is
               // written at the same offsets as the hi tile (A and B tiles are contiguous). All loads
               // of a thread are issued before the first conversion so that their latencies overlap.
               float4 *hi = reinterpret_cast<float4 *>(a_hi(s));
               float4 *lo = reinterpret_cast<float4 *>(a_lo(s));
               constexpr int n4 = (L::kATile + L::kBTile) / 16;
               constexpr int PER = (n4 + NT - 1) / NT;
               float4 v[PER];
#pragma unroll
               for (int i = 0; i < PER; i++)
                  if (t + i * NT < n4) v[i] = hi[t + i * NT];
#pragma unroll
               for (int i = 0; i < PER; i++) {
                  if (t + i * NT < n4) {
                     float4 h, l;
                     uint32_t w;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(w) : "f"(v[i].x)); h.x = __uint_as_float(w); l.x = v[i].x - h.x;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(w) : "f"(v[i].y)); h.y = __uint_as_float(w); l.y = v[i].y - h.y;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(w) : "f"(v[i].z)); h.z = __uint_as_float(w); l.z = v[i].z - h.z;
                     asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(w) : "f"(v[i].w)); h.w = __uint_as_float(w); l.w = v[i].w - h.w;
                     hi[t + i * NT] = h;
                     lo[t + i * NT] = l;
                  }
               }
               fence_proxy_async(); // make the generic-proxy writes visible to the tensor-core (async) proxy
               mbar_arrive(&conv_bar[s]);
            }
         }
      }
   } else {
      // ---------------- epilogue warps ----------------
      // TMEM lanes a warp may read are fixed by (warp id mod 4); with 8 epilogue warps two warps
      // share a lane quarter and split the columns.
      const int lane_base = (warp & 3) * 32;
      const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
      // the EPI_WARPS / 4 warps of a lane quarter take the 32-column chunks of the tile round-robin
      constexpr int GROUPS = EPI_WARPS / 4;
      const int group = (warp - 2) >> 2;
      int u = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
         const int m0 = (tile / tiles_n) * kBM, n0 = (tile % tiles_n) * BN;
         const int row = m0 + lane_base + lane;
         if constexpr (KIND == kTF32) {
            float acc[BN];
#pragma unroll
            for (int j = 0; j < BN; j++) acc[j] = 0.f;
            for (int c = 0; c < units_per_tile; c++, u++) {
               const int buf = u & 1;
               if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_full[buf], (u >> 1) & 1, &abort_flag, status, kStatusWaitAccum, 0x3000 + u))) {
                  ok = false;
                  break;
               }
               tc_fence_after();
#pragma unroll
               for (int c0 = 0; c0 < BN; c0 += 32) {
                  uint32_t r[32];
                  tmem_ld_32x32(t_row + (uint32_t)(buf * BN + c0), r);
                  tmem_ld_wait();
#pragma unroll
                  for (int j = 0; j < 32; j++) acc[c0 + j] += __uint_as_float(r[j]);
               }
               tc_fence_before();
               __syncwarp();
               if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            }
            if (ok) {
#pragma unroll
               for (int c0 = 0; c0 < BN; c0 += 32) {
                  if (n0 + c0 < N) {
                     uint32_t r[32];
#pragma unroll
                     for (int j = 0; j < 32; j++) r[j] = __float_as_uint(acc[c0 + j]);
                     store_row_chunk<KIND>(ep, r, row, row < M, n0 + c0, N, s_cf[warp], lane);
                  }
               }
            }
         } else {
            const int buf = u & 1;
            if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_full[buf], (u >> 1) & 1, &abort_flag, status, kStatusWaitAccum, 0x3000 + u))) break;
            tc_fence_after();
#pragma unroll 1
            for (int c0 = group * 32; c0 < BN; c0 += GROUPS * 32) {
               if (n0 + c0 >= N) break;
               uint32_t r[32];
               tmem_ld_32x32(t_row + (uint32_t)(buf * BN + c0), r);
               tmem_ld_wait();
               store_row_chunk<KIND>(ep, r, row, row < M, n0 + c0, N, s_cf[warp], lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            u++;
         }
      }
   }
   SOFIE_PROF_REPORT(warp == 0 ? "producer" : (warp == 1 ? "mma" : (warp < 2 + EPI_WARPS ? "epilogue" : "converter")));
   // A wait only gives up after about a second, long after every copy and MMA this CTA issued has
   // landed, so nothing is in flight when the TMEM columns are released below.
   tc_fence_before();
   __syncthreads();
   if (warp == 1) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, TMEM_COLS);
   }
}

// ================================================================================================
// Pair kernel for the 8-bit kinds: a cluster of two CTAs (one TPC) computes a 256 x 256 output tile
// with `tcgen05.mma.cta_group::2`. CTA r of the pair keeps rows [128 r, 128 r + 128) of the A tile,
// rows [128 r, 128 r + 128) of the B tile and the same rows of the accumulator in its own TMEM, so a
// stage is 32 KB per CTA for 4 MMAs of 128 clocks each: 64 bytes per clock and SM, where the 128 x 256
// single-CTA tile needs 96 and the copy engine delivers about 48. No load is a multicast load.
//   Protocol (leader = cluster rank 0; every barrier exists in both CTAs):
//   full[s]      leader's only: 1 arrival (its producer, with the byte count of BOTH CTAs' copies);
//                both producers' copies complete on it (the peer's through the cluster address).
//   empty[s]     each CTA's own: the leader's commit arrives on both (multicast of the commit).
//   tmem_full[b] each CTA's own: committed on both after the last stage of a tile.
//   tmem_empty[b] leader's only: 2 x 16 arrivals, one per epilogue warp of either CTA.
// The CTAs meet at a cluster barrier after initialising their barriers and before releasing TMEM,
// which every thread reaches (a wait that gives up only leaves its loop).
constexpr int kPairBN = 256;      // columns of the pair's tile
constexpr int kPairStages = 6;    // 6 x 32 KB per CTA
constexpr int kPairStageBytes = 2 * kBM * kStageK;

template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((2 + kGemmEpilogueWarps8) * 32, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmEpilogue ep,
                      int M, int N, int K, uint32_t *status)
{
   constexpr int S = kPairStages;
   constexpr uint32_t TMEM_COLS = 2 * kPairBN;
   constexpr int EPI_WARPS = kGemmEpilogueWarps8;
   extern __shared__ unsigned char smem_raw[];
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
   __shared__ uint64_t full_bar[S], empty_bar[S], tmem_full[2], tmem_empty[2];
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   __shared__ __align__(16) float s_cf[18][64]; // per-warp hand-over of the per-column epilogue constants

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   SOFIE_PROF_DECL
   griddep_launch_dependents(); // the next kernel may set itself up while this one runs
   const uint32_t rank = cluster_ctarank();
   const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
   const int tiles_n = (N + kPairBN - 1) / kPairBN, tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
   const int num_tiles = tiles_m * tiles_n;
   const int num_kb = (K + kStageK - 1) / kStageK;

   auto a_tile = [&](int s) { return smem + (size_t)s * kPairStageBytes; };
   auto b_tile = [&](int s) { return smem + (size_t)s * kPairStageBytes + kBM * kStageK; };

   if (threadIdx.x == 0) {
      for (int s = 0; s < S; s++) {
         mbar_init(&full_bar[s], 1);
         mbar_init(&empty_bar[s], 1);
      }
      for (int b = 0; b < 2; b++) {
         mbar_init(&tmem_full[b], 1);
         mbar_init(&tmem_empty[b], 2 * EPI_WARPS);
      }
      abort_flag = 0;
      fence_mbar_init();
      prefetch_tensormap(&tmA);
      prefetch_tensormap(&tmB);
   }
   if (warp == 1) {
      tmem_alloc_pair(&tmem_base_holder, TMEM_COLS);
      tmem_relinquish_pair();
   }
   tc_fence_before();
   __syncthreads();
   cluster_sync_all(); // the peer's barriers exist before anything arrives on them
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;

   if (warp == 0) {
      // ---------------- TMA producer (both CTAs) ----------------
      griddep_wait(); // A is the previous kernel's output
      int g = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
         const int m0 = (tile / tiles_n) * (2 * kBM) + (int)rank * kBM;
         const int n0 = (tile % tiles_n) * kPairBN + (int)rank * kBM;
         for (int kb = 0; kb < num_kb; kb++, g++, ring_next(s, ph, S)) {
            if (lane == 0) {
               ok = SOFIE_PROF_WAIT(mbar_wait(&empty_bar[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g));
               if (ok && rank == 0) mbar_expect_tx(&full_bar[s], 2 * kPairStageBytes);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const uint32_t full_leader = mapa_shared(smem_u32(&full_bar[s]), 0);
            if (lane == 0) tma_load_2d_pair(a_tile(s), &tmA, kb * kStageK, m0, full_leader);
            else if (lane == 1) tma_load_2d_pair(b_tile(s), &tmB, kb * kStageK, n0, full_leader);
            __syncwarp();
         }
      }
   } else if (warp == 1) {
      // ---------------- MMA issuer (leader CTA only) ----------------
      if (lane == 0 && rank == 0) {
         constexpr uint32_t idesc = make_idesc<KIND>(2 * kBM, kPairBN);
         int g = 0, u = 0, s = 0;
         uint32_t ph = 0;
         bool ok = true;
         for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, u++) {
            const int buf = u & 1;
            if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_empty[buf], ((u >> 1) & 1) ^ 1, &abort_flag, status, kStatusWaitAccum, 0x1000 + u))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kPairBN);
            for (int kb = 0; kb < num_kb; kb++, g++, ring_next(s, ph, S)) {
               ok = SOFIE_PROF_WAIT(mbar_wait(&full_bar[s], ph, &abort_flag, status, kStatusWaitFull, g));
               if (!ok) break;
               tc_fence_after();
               const uint64_t da = make_smem_desc(smem_u32(a_tile(s)), kStageK);
               const uint64_t db = make_smem_desc(smem_u32(b_tile(s)), kStageK);
#pragma unroll
               for (int k = 0; k < kStageK / kMmaK; k++) {
                  const uint64_t koff = (uint64_t)(k * (kMmaK >> 4));
                  tc_mma_pair<KIND>(d_tmem, da + koff, db + koff, idesc, (kb == 0 && k == 0) ? 0u : 1u);
               }
               tc_commit_pair(&empty_bar[s], 3); // both CTAs' slots are free once these MMAs have read them
            }
            if (ok) tc_commit_pair(&tmem_full[buf], 3);
         }
      }
   } else {
      // ---------------- epilogue warps 2..17 (both CTAs) ----------------
      const int lane_base = (warp & 3) * 32;
      const uint32_t t_row = tmem_base + ((uint32_t)lane_base << 16);
      constexpr int GROUPS = EPI_WARPS / 4;
      const int group = (warp - 2) >> 2;
      int u = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs, u++) {
         const int m0 = (tile / tiles_n) * (2 * kBM) + (int)rank * kBM, n0 = (tile % tiles_n) * kPairBN;
         const int row = m0 + lane_base + lane;
         const int buf = u & 1;
         if (!SOFIE_PROF_WAIT(mbar_wait(&tmem_full[buf], (u >> 1) & 1, &abort_flag, status, kStatusWaitAccum, 0x3000 + u))) break;
         tc_fence_after();
#pragma unroll 1
         for (int c0 = group * 32; c0 < kPairBN; c0 += GROUPS * 32) {
            if (n0 + c0 >= N) break;
            uint32_t r[32];
            tmem_ld_32x32(t_row + (uint32_t)(buf * kPairBN + c0), r);
            tmem_ld_wait();
            store_row_chunk<KIND>(ep, r, row, row < M, n0 + c0, N, s_cf[warp], lane);
         }
         tc_fence_before();
         __syncwarp();
         if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[buf]), 0));
      }
   }
   SOFIE_PROF_REPORT(warp == 0 ? "producer" : (warp == 1 ? "mma" : "epilogue"));
   // Nothing of this CTA may be released while the peer can still touch it (the leader's MMAs write
   // the peer's TMEM and its commits arrive on the peer's barriers).
   tc_fence_before();
   __syncthreads();
   cluster_sync_all();
   if (warp == 1) {
      tc_fence_after();
      tmem_dealloc_pair(tmem_base, TMEM_COLS);
   }
}

template <int KIND>
static int launch_pair(cudaStream_t s, const CUtensorMap &tmA, const CUtensorMap &tmB, const GemmEpilogue &ep, int M, int N, int K)
{
   const int smem = kPairStages * kPairStageBytes + 1024;
   auto kern = umma_gemm_pair_kernel<KIND>;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int tiles = ceil_div(N, kPairBN) * ceil_div(M, 2 * kBM);
   const int pairs = tiles < kNumSMs / 2 ? tiles : kNumSMs / 2;
   SOFIE_CUDA_TRY(launch_dependent(kern, dim3(2 * pairs), dim3((2 + kGemmEpilogueWarps8) * 32), smem, s, tmA, tmB, ep, M, N, K, status));
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

// SOFIE_CUDA_GEMM_PAIR=0 keeps every shape on the single-CTA kernel (used to compare the two).
static bool pair_enabled()
{
   static const bool v = [] { const char *e = getenv("SOFIE_CUDA_GEMM_PAIR"); return !e || atoi(e) != 0; }();
   return v;
}

// ------------------------------------------------------------------------------------------------
template <int KIND, int BN>
static int launch_one(cudaStream_t s, const CUtensorMap &tmA, const CUtensorMap &tmB, const GemmEpilogue &ep, int M,
                      int N, int K)
{
   using L = GemmSmem<KIND, BN>;
   int stages = (200 * 1024) / L::kStageBytes;
   if (stages > kGemmMaxStages) stages = kGemmMaxStages;
   const int smem = stages * L::kStageBytes + 1024;
   auto kern = umma_gemm_kernel<KIND, BN>;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int tiles = ceil_div(N, BN) * ceil_div(M, kBM);
   const int grid = tiles < kNumSMs ? tiles : kNumSMs;
   SOFIE_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(gemm_threads<KIND>()), smem, s, tmA, tmB, ep, M, N, K, stages, status));
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

template <int KIND>
static int launch_umma_gemm(cudaStream_t s, const void *A, const void *B, const GemmEpilogue &ep, int M, int N, int K)
{
   constexpr int ES = (KIND == kTF32) ? 4 : 1;
   if (M <= 0 || N <= 0 || K <= 0) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "empty GEMM");
   if (((size_t)K * ES) % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
      return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "TMA needs 16-byte aligned rows (K*%d %% 16 == 0) and bases", ES);
   // fp32 keeps the tile's running sum in registers (promotion), which bounds its width at 64 columns
   int BN = N <= 32 ? 32 : ((N <= 64 || KIND == kTF32) ? 64 : (N <= 128 ? 128 : 256));
   // wide tiles are the efficient ones, but not when they leave most SMs without a tile
   while (BN > 64 && (long long)ceil_div(M, kBM) * ceil_div(N, BN) < (kNumSMs * 4) / 5) BN /= 2;
   CUtensorMap tmA, tmB;
   const CUtensorMapDataType dt = (KIND == kTF32) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
   uint64_t dimsA[2] = {(uint64_t)K, (uint64_t)M}, dimsB[2] = {(uint64_t)K, (uint64_t)N};
   uint64_t stride[1] = {(uint64_t)K * ES};
   uint32_t boxA[2] = {(uint32_t)(kStageK / ES), (uint32_t)kBM}, boxB[2] = {(uint32_t)(kStageK / ES), (uint32_t)BN};
   int rc = make_tensor_map(&tmA, dt, 2, A, dimsA, stride, boxA, 128);
   if (rc) return rc;
   rc = make_tensor_map(&tmB, dt, 2, B, dimsB, stride, boxB, 128);
   if (rc) return rc;
   if constexpr (KIND != kTF32) {
      // wide outputs with enough 256 x 256 tiles to keep every pair of SMs busy for several rounds: with one or two
      // tiles per pair the fill of the deeper pipeline and the uneven last round cost more than the pair saves
      if (pair_enabled() && N >= 256 && ceil_div(N, kPairBN) * ceil_div(M, 2 * kBM) >= 4 * (kNumSMs / 2)) {
         CUtensorMap tmBh;
         uint32_t boxBh[2] = {(uint32_t)kStageK, (uint32_t)kBM};
         rc = make_tensor_map(&tmBh, dt, 2, B, dimsB, stride, boxBh, 128);
         if (rc) return rc;
         return launch_pair<KIND>(s, tmA, tmBh, ep, M, N, K);
      }
   }
   if constexpr (KIND == kTF32) {
      if (BN == 32) return launch_one<KIND, 32>(s, tmA, tmB, ep, M, N, K);
      return launch_one<KIND, 64>(s, tmA, tmB, ep, M, N, K);
   } else {
      switch (BN) {
      case 32: return launch_one<KIND, 32>(s, tmA, tmB, ep, M, N, K);
      case 64: return launch_one<KIND, 64>(s, tmA, tmB, ep, M, N, K);
      case 128: return launch_one<KIND, 128>(s, tmA, tmB, ep, M, N, K);
      default: return launch_one<KIND, 256>(s, tmA, tmB, ep, M, N, K);
      }
   }
}

} // namespace umma

// Entry points used by api.cu. Each returns SOFIE_CUDA_ERR_UNSUPPORTED when the shape does not fit
// the tensor-core kernel, and the caller then takes the CUDA-core kernel.
int launch_gemm_f32_umma(cudaStream_t s, const sofie_gemm_f32_desc &d, const float *A, const float *B, const float *C,
                         float *Y)
{
   if (d.transA || !d.transB) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "tensor-core GEMM takes A[M,K] and B[N,K]");
   umma::GemmEpilogue ep = {};
   ep.alpha = d.alpha;
   ep.beta = d.beta;
   ep.C = C;
   ep.bias_kind = d.bias_kind;
   ep.Yf = Y;
   ep.relu = d.relu;
   return umma::launch_umma_gemm<umma::kTF32>(s, A, B, ep, d.M, d.N, d.K);
}

int launch_qgemm_umma(cudaStream_t s, const sofie_qgemm_desc &d, const uint8_t *A, const int8_t *W, const float *mult,
                      const int32_t *corr, uint8_t *Y, float *Yf32, float dq_scale)
{
   if (!d.w_is_nk) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "tensor-core GEMM takes W as [N,K]");
   umma::GemmEpilogue ep = {};
   ep.mult = mult;
   ep.corr = corr;
   ep.y_zp = d.y_zp;
   ep.Yu8 = Y;
   ep.Yf = Yf32;
   ep.scale = dq_scale;
   ep.relu = d.relu;
   return umma::launch_umma_gemm<umma::kI8>(s, A, W, ep, d.M, d.N, d.K);
}

int launch_gemm_e4m3_umma(cudaStream_t s, const sofie_fp8_gemm_desc &d, const uint8_t *A, const uint8_t *W,
                          const float *bias, uint16_t *Ybf16, uint8_t *Yq, float *Yf32, const float *a_scale_dev)
{
   umma::GemmEpilogue ep = {};
   ep.scale = d.a_scale * d.w_scale;
   ep.a_scale_dev = a_scale_dev;
   ep.w_scale = d.w_scale;
   ep.q_scale = d.q_scale;
   ep.q_inv = d.q_scale != 0.f ? (float)(1.0 / (double)d.q_scale) : 0.f;
   ep.bias = bias;
   ep.Ybf16 = Ybf16;
   ep.Yq = Yq;
   ep.Yf = Yf32;
   ep.relu = d.relu;
   return umma::launch_umma_gemm<umma::kF8>(s, A, W, ep, d.M, d.N, d.K);
}

} // namespace sofie
