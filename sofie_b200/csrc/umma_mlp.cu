// Fused chain of small Gemm layers on the tensor cores: y = act(... act(x W0^T + b0) ... W_{L-1}^T + b_{L-1}).
// Replaces, for one launch, the chain of sgemm_ calls plus bias and Relu loops that the reference emits per layer
// (ROperator_Gemm.hxx:292-390, ROperator_Relu.hxx:55-60).
//
// A CTA owns slabs of 128 rows. The activations of a slab never leave the SM: a layer's accumulators go from tensor
// memory through registers (bias, Relu, split into a tf32 "hi" part and the fp32 remainder "lo") straight back into
// shared memory as the next layer's A operand. The weights are split the same way while they are staged, K chunk by
// K chunk, through a small ring; fp32 accuracy comes from three tf32 products per K step, issued as two MMAs:
//
//    D[:, 0:Np)    = A_hi x W_hi      D[:, Np:2Np) = A_hi x W_lo      (one MMA of width 2 Np over the rows [W_hi; W_lo])
//    D[:, 0:Np)   += A_lo x W_hi                                      (one MMA of width Np)
//
// and the epilogue adds the two halves. Operand layout (both operands, no swizzle): 16-byte groups of four consecutive
// K values; group j of row r lives at j * LBO + r * 16, so eight consecutive rows of a group are the 128 contiguous
// bytes the MMA calls a core matrix, and 32 threads that hold 32 consecutive rows write 512 contiguous bytes. LBO is
// padded by 64 bytes so that the staging threads, which read four rows x 128 contiguous bytes per warp from global
// memory, also write without bank conflicts.
//
// Roles: warps 0-7 activations (a thread = a row = a tensor-memory lane; the two warps of a lane quarter split the
// columns), warps 8-15 weight staging, warp 16 the thread that issues the MMAs. Global loads are issued two stages
// (weights) or one slab (input rows) ahead of the shared-memory stores that consume them, so their latency is hidden
// behind the MMAs. The operands are written with ordinary stores (generic proxy) and read by the MMAs through the
// async proxy: the proxy fence between the two is executed by the issuing thread, after its wait on the barrier the
// writers arrived on and before the MMA -- a fence in a writing thread would also wait for that thread's prefetches in
// flight and put their latency back on the critical path (measured: 4 k clocks per stage). Every wait is bounded (umma.cuh).
#include "umma.cuh"
#include "contract.cuh"

namespace sofie {
namespace umma {

constexpr int kMlpTcMaxLayers = 4;
constexpr int kMlpActWarps = 8, kMlpLoadWarps = 8;
constexpr int kMlpTcThreads = (kMlpActWarps + kMlpLoadWarps + 1) * 32;
constexpr int kMlpKC = 32;              // K values per weight stage (four MMA K steps of 8)
constexpr int kMlpMaxStages = 3;
constexpr uint32_t kMlpPad = 64;        // bytes added to each LBO (see above)

struct MlpTcPlan {
   int M, layers;
   int K[kMlpTcMaxLayers], N[kMlpTcMaxLayers], Np[kMlpTcMaxLayers]; // Np: N rounded up to 16
   int relu[kMlpTcMaxLayers], nk[kMlpTcMaxLayers];
   const float *W[kMlpTcMaxLayers];
   const float *B[kMlpTcMaxLayers];
   uint32_t a_lbo;        // bytes between K groups of the activation operand (128 rows x 16 + pad)
   uint32_t a_bytes;      // one copy (hi) of the activation operand
   uint32_t stage_bytes;  // one weight stage: 8 K groups x (2 Np_max x 16 + pad)
   int stages;
   uint32_t tmem_cols;
};

__device__ __forceinline__ void split_tf32(const float4 v, float4 &h, float4 &l)
{
   uint32_t u;
   asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.x)); h.x = __uint_as_float(u); l.x = v.x - h.x;
   asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.y)); h.y = __uint_as_float(u); l.y = v.y - h.y;
   asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.z)); h.z = __uint_as_float(u); l.z = v.z - h.z;
   asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v.w)); h.w = __uint_as_float(u); l.w = v.w - h.w;
}

// Read-only global loads as volatile asm: the compiler keeps them where they are written (a plain __ldg may be sunk to
// its first use, past the barrier waits in between, which puts the load latency back on the critical path).
__device__ __forceinline__ float4 ld_nc_f4(const float *p)
{
   float4 v;
   asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
   return v;
}
__device__ __forceinline__ float ld_nc_f1(const float *p)
{
   float v;
   asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
   return v;
}

// Staging of `rows` rows x `groups` K groups (of four floats) of a matrix into the operand layout, in two halves so
// that the loads of a later block can be in flight while an earlier one is stored: item i of a thread (thread t of NT)
// is element i * NT + t of the block. Row-major source (src[r * ld + k]): a warp takes four rows x eight groups, 128
// contiguous bytes per row; K-major source (src[k * ld + r], `transposed`): 32 rows of one group, four coalesced loads.
// Rows at or beyond rows_valid and K values at or beyond k_valid read as zero.
struct StageGeom {
   const float *src;
   size_t ld;
   int rows, rows_valid, k0, groups, k_valid;
   bool transposed, vec;
};
__device__ __forceinline__ bool stage_item(const StageGeom &g, int i, int &r, int &j)
{
   if (!g.transposed) {
      const int gb = (g.groups + 7) >> 3;
      const int lane = i & 31, blk = i >> 5;
      r = (blk / gb) * 4 + (lane >> 3);
      j = (blk % gb) * 8 + (lane & 7);
   } else {
      const int rpad = (g.rows + 31) & ~31;
      j = i / rpad;
      r = i - j * rpad;
   }
   return r < g.rows && j < g.groups;
}
template <int NT, int ITEMS>
__device__ __forceinline__ void stage_load(const StageGeom &g, int t, int first, float4 (&v)[ITEMS])
{
   if (g.vec && !g.transposed) {
      // the common case: every load is issued, unconditionally (an item outside the block reads the block's first
      // 16 bytes and is dropped when it is stored), so that nothing between here and the store waits for the data
#pragma unroll
      for (int q = 0; q < ITEMS; q++) {
         int r, j;
         const bool in = stage_item(g, (first + q) * NT + t, r, j) && r < g.rows_valid;
         v[q] = ld_nc_f4(in ? g.src + (size_t)r * g.ld + (g.k0 + 4 * j) : g.src);
      }
      return;
   }
#pragma unroll
   for (int q = 0; q < ITEMS; q++) {
      int r, j;
      v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (!stage_item(g, (first + q) * NT + t, r, j) || r >= g.rows_valid) continue;
      const int k = g.k0 + 4 * j;
      const float *p = g.transposed ? g.src + (size_t)k * g.ld + r : g.src + (size_t)r * g.ld + k;
      const size_t step = g.transposed ? g.ld : 1;
      if (k < g.k_valid) v[q].x = ld_nc_f1(p);
      if (k + 1 < g.k_valid) v[q].y = ld_nc_f1(p + step);
      if (k + 2 < g.k_valid) v[q].z = ld_nc_f1(p + 2 * step);
      if (k + 3 < g.k_valid) v[q].w = ld_nc_f1(p + 3 * step);
   }
}
// hi part at dst + j * lbo + r * 16, lo part lo_off bytes further
template <int NT, int ITEMS>
__device__ __forceinline__ void stage_store(const StageGeom &g, int t, int first, const float4 (&v)[ITEMS], unsigned char *dst, uint32_t lbo,
                                            uint32_t lo_off)
{
#pragma unroll
   for (int q = 0; q < ITEMS; q++) {
      int r, j;
      if (!stage_item(g, (first + q) * NT + t, r, j)) continue;
      float4 h, l;
      split_tf32(r < g.rows_valid ? v[q] : make_float4(0.f, 0.f, 0.f, 0.f), h, l);
      unsigned char *p = dst + (size_t)j * lbo + (size_t)r * 16;
      *reinterpret_cast<float4 *>(p) = h;
      *reinterpret_cast<float4 *>(p + lo_off) = l;
   }
}
__device__ __forceinline__ int stage_items(const StageGeom &g)
{
   return g.transposed ? g.groups * ((g.rows + 31) & ~31) : ((g.rows + 3) >> 2) * ((g.groups + 7) >> 3) * 32;
}

__global__ void __launch_bounds__(kMlpTcThreads, 1)
umma_mlp_kernel(MlpTcPlan pl, const float *__restrict__ X, float *__restrict__ Y, int x_vec, uint32_t *status)
{
   extern __shared__ unsigned char smem_raw[];
   unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
   unsigned char *a_hi = smem;                              // activations: hi copy, lo copy a_bytes further
   unsigned char *ring = smem + 2 * (size_t)pl.a_bytes;     // weight stages
   __shared__ uint64_t act_ready, acc_full, w_full[kMlpMaxStages], w_empty[kMlpMaxStages];
   __shared__ uint32_t tmem_base_holder;
   __shared__ volatile uint32_t abort_flag;
   __shared__ float s_bias[kMlpTcMaxLayers][128];

   const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
   SOFIE_PROF_DECL
   griddep_launch_dependents();
   for (int i = threadIdx.x; i < kMlpTcMaxLayers * 128; i += blockDim.x) {
      const int l = i >> 7, n = i & 127;
      s_bias[l][n] = (l < pl.layers && n < pl.N[l] && pl.B[l]) ? pl.B[l][n] : 0.f;
   }
   if (threadIdx.x == 0) {
      mbar_init(&act_ready, kMlpActWarps * 32);
      mbar_init(&acc_full, 1);
      for (int s = 0; s < kMlpMaxStages; s++) {
         mbar_init(&w_full[s], kMlpLoadWarps * 32);
         mbar_init(&w_empty[s], 1);
      }
      abort_flag = 0;
      fence_mbar_init();
   }
   if (warp == kMlpActWarps + kMlpLoadWarps) {
      tmem_alloc(&tmem_base_holder, pl.tmem_cols);
      tmem_relinquish();
   }
   tc_fence_before();
   __syncthreads();
   tc_fence_after();
   const uint32_t tmem_base = tmem_base_holder;
   const int slabs = (pl.M + 127) >> 7;
   const int S = pl.stages;

   if (warp < kMlpActWarps) {
      // ---------------- activation warps ----------------
      const int q = warp & 3, half = warp >> 2;
      const int r = q * 32 + lane;                       // row of the slab = tensor-memory lane
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
      const int t = threadIdx.x;                          // 0..255
      uint32_t acc_ph = 0;
      constexpr int NTA = kMlpActWarps * 32, XPRE = 8; // the first XPRE items of a thread are fetched one slab ahead
      auto x_geom = [&](int slab) {
         StageGeom g;
         const int row0 = slab << 7;
         g.src = slab < slabs ? X + (size_t)row0 * pl.K[0] : X; // beyond the last slab nothing is valid: every item reads X[0..3]
         g.ld = (size_t)pl.K[0];
         g.rows = 128;
         g.rows_valid = slab < slabs ? (pl.M - row0 < 128 ? pl.M - row0 : 128) : 0;
         g.k0 = 0;
         g.groups = pl.K[0] >> 2;
         g.k_valid = pl.K[0];
         g.transposed = false;
         g.vec = x_vec != 0;
         return g;
      };
      griddep_wait(); // X is the previous kernel's output
      float4 xv[XPRE];
      stage_load<NTA, XPRE>(x_geom(blockIdx.x), t, 0, xv);
      for (int slab = blockIdx.x; slab < slabs; slab += gridDim.x) {
         const int row0 = slab << 7;
         const int valid = pl.M - row0 < 128 ? pl.M - row0 : 128;
         // layer 0's operand: the slab of X (the previous slab's last accumulators have been read: its MMAs are done)
         {
            const StageGeom g = x_geom(slab);
            stage_store<NTA, XPRE>(g, t, 0, xv, a_hi, pl.a_lbo, pl.a_bytes);
            const int per_thread = (stage_items(g) + NTA - 1) / NTA;
            for (int first = XPRE; first < per_thread; first += XPRE) {
               stage_load<NTA, XPRE>(g, t, first, xv);
               stage_store<NTA, XPRE>(g, t, first, xv, a_hi, pl.a_lbo, pl.a_bytes);
            }
         }
         mbar_arrive(&act_ready);
         // the next slab's rows, in flight during this slab's layers
         stage_load<NTA, XPRE>(x_geom(slab + (int)gridDim.x), t, 0, xv);
         bool ok = true;
         for (int l = 0; l < pl.layers && ok; l++) {
            ok = SOFIE_PROF_WAIT(mbar_wait(&acc_full, acc_ph, &abort_flag, status, kStatusWaitAccum, 0x5000 + l));
            acc_ph ^= 1;
            if (!ok) break;
            tc_fence_after();
            const int Np = pl.Np[l], N = pl.N[l];
            const bool last = l + 1 == pl.layers;
            const bool relu = pl.relu[l] != 0;
            // chunks of 16 columns, taken alternately by the two warps of this lane quarter
            for (int c0 = half * 16; c0 < Np; c0 += 32) {
               uint32_t hi[16], lo[16];
               tmem_ld_32x16(t_row + (uint32_t)c0, hi);
               tmem_ld_32x16(t_row + (uint32_t)(Np + c0), lo);
               tmem_ld_wait();
               float v[16];
#pragma unroll
               for (int i = 0; i < 16; i++) {
                  v[i] = (__uint_as_float(hi[i]) + __uint_as_float(lo[i])) + s_bias[l][c0 + i];
                  if (relu) v[i] = v[i] > 0.f ? v[i] : 0.f; // NaN -> 0, as the reference's (x > 0) ? x : 0
               }
               if (last) {
                  if (r < valid) {
                     float *y = Y + (size_t)(row0 + r) * N + c0;
                     if (c0 + 16 <= N && ((reinterpret_cast<uintptr_t>(y) & 15) == 0)) {
#pragma unroll
                        for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4 *>(y + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                     } else {
#pragma unroll
                        for (int i = 0; i < 16; i++)
                           if (c0 + i < N) y[i] = v[i];
                     }
                  }
               } else {
#pragma unroll
                  for (int i = 0; i < 16; i += 4) {
                     float4 h, lw;
                     split_tf32(make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]), h, lw);
                     unsigned char *p = a_hi + (size_t)((c0 + i) >> 2) * pl.a_lbo + (size_t)r * 16;
                     *reinterpret_cast<float4 *>(p) = h;
                     *reinterpret_cast<float4 *>(p + pl.a_bytes) = lw;
                  }
               }
            }
            tc_fence_before(); // the accumulators have been read: the next layer may overwrite them
            if (!last) mbar_arrive(&act_ready);
         }
         if (!ok) break;
      }
   } else if (warp < kMlpActWarps + kMlpLoadWarps) {
      // ---------------- weight staging warps ----------------
      // The stages of this CTA form one sequence (slab by slab, layer by layer, K chunk by K chunk); the loads of
      // stage i + 2 are issued before stage i is stored, into a rotation of three register sets.
      constexpr int NTW = kMlpLoadWarps * 32, WI = 4; // 128 rows x 8 groups = 1024 items of a stage, 4 per thread
      const int t = threadIdx.x - kMlpActWarps * 32;
      int chunks_per_slab = 0;
      for (int l = 0; l < pl.layers; l++) chunks_per_slab += (pl.K[l] + kMlpKC - 1) / kMlpKC;
      const int my_slabs = blockIdx.x < slabs ? (slabs - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
      const int total = my_slabs * chunks_per_slab;
      struct Cursor {
         int l, k0;
      };
      auto geom = [&](const Cursor &c) {
         StageGeom g;
         const int K = pl.K[c.l];
         g.src = pl.W[c.l];
         g.ld = pl.nk[c.l] ? (size_t)K : (size_t)pl.N[c.l];
         g.rows = pl.Np[c.l];
         g.rows_valid = pl.N[c.l];
         g.k0 = c.k0;
         g.groups = (K - c.k0 < kMlpKC ? K - c.k0 : kMlpKC) >> 2;
         g.k_valid = K;
         g.transposed = !pl.nk[c.l];
         g.vec = pl.nk[c.l] && (K & 3) == 0 && (reinterpret_cast<uintptr_t>(pl.W[c.l]) & 15) == 0;
         return g;
      };
      auto advance = [&](Cursor &c) {
         c.k0 += kMlpKC;
         if (c.k0 >= pl.K[c.l]) {
            c.k0 = 0;
            c.l = c.l + 1 == pl.layers ? 0 : c.l + 1;
         }
      };
      float4 w0[WI], w1[WI], w2[WI];
      Cursor cur = {0, 0}, ahead = {0, 0}; // stage being stored, stage being loaded
      int loaded = 0;
      auto load_next = [&](float4 (&v)[WI]) {
         if (loaded < total) {
            stage_load<NTW, WI>(geom(ahead), t, 0, v);
            advance(ahead);
         }
         loaded++;
      };
      int g = 0, s = 0;
      uint32_t ph = 0;
      bool ok = true;
      auto store = [&](const float4 (&v)[WI]) {
         ok = SOFIE_PROF_WAIT(mbar_wait(&w_empty[s], ph ^ 1, &abort_flag, status, kStatusWaitEmpty, g));
         if (!ok) return;
         const StageGeom sg = geom(cur);
         const int Np = pl.Np[cur.l];
         // rows [0, Np) of the stage: hi; rows [Np, 2 Np): lo. Rows n >= N are zero.
         stage_store<NTW, WI>(sg, t, 0, v, ring + (size_t)s * pl.stage_bytes, (uint32_t)(2 * Np * 16) + kMlpPad, (uint32_t)Np * 16);
         mbar_arrive(&w_full[s]);
         advance(cur);
         g++;
         ring_next(s, ph, S);
      };
      load_next(w0);
      load_next(w1);
      for (int i = 0; i < total && ok; i += 3) {
         load_next(w2);
         store(w0);
         if (i + 1 >= total || !ok) break;
         load_next(w0);
         store(w1);
         if (i + 2 >= total || !ok) break;
         load_next(w1);
         store(w2);
      }
   } else {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
         int g = 0, s = 0;
         uint32_t ph = 0, act_ph = 0;
         bool ok = true;
         const uint64_t da_hi = make_smem_desc_noswizzle(smem_u32(a_hi), pl.a_lbo, 128);
         const uint64_t da_lo = make_smem_desc_noswizzle(smem_u32(a_hi + pl.a_bytes), pl.a_lbo, 128);
         for (int slab = blockIdx.x; slab < slabs && ok; slab += gridDim.x) {
            for (int l = 0; l < pl.layers && ok; l++) {
               const int K = pl.K[l], Np = pl.Np[l];
               const uint32_t lbo = (uint32_t)(2 * Np * 16) + kMlpPad;
               const uint32_t idesc_wide = make_idesc<kTF32>(128, 2 * Np), idesc = make_idesc<kTF32>(128, Np);
               ok = SOFIE_PROF_WAIT(mbar_wait(&act_ready, act_ph, &abort_flag, status, kStatusWaitConv, 0x6000 + l));
               act_ph ^= 1;
               if (!ok) break;
               fence_proxy_async();
               tc_fence_after();
               for (int k0 = 0; k0 < K; k0 += kMlpKC, g++, ring_next(s, ph, S)) {
                  ok = SOFIE_PROF_WAIT(mbar_wait(&w_full[s], ph, &abort_flag, status, kStatusWaitFull, g));
                  if (!ok) break;
                  fence_proxy_async();
                  tc_fence_after();
                  const uint64_t db = make_smem_desc_noswizzle(smem_u32(ring + (size_t)s * pl.stage_bytes), lbo, 128);
                  const int ksteps = (K - k0 < kMlpKC ? K - k0 : kMlpKC) >> 3;
                  for (int kk = 0; kk < ksteps; kk++) {
                     // one K step = 8 values = two K groups of each operand
                     const uint64_t a_off = (uint64_t)(((uint32_t)((k0 >> 2) + 2 * kk) * pl.a_lbo) >> 4);
                     const uint64_t b_off = (uint64_t)(((uint32_t)(2 * kk) * lbo) >> 4);
                     tc_mma<kTF32>(tmem_base, da_hi + a_off, db + b_off, idesc_wide, (k0 | kk) ? 1u : 0u); // hi x [hi | lo]
                     tc_mma<kTF32>(tmem_base, da_lo + a_off, db + b_off, idesc, 1u);                        // lo x hi
                  }
                  tc_commit(&w_empty[s]);
               }
               if (ok) tc_commit(&acc_full);
            }
         }
      }
   }
   SOFIE_PROF_REPORT(warp < kMlpActWarps ? "activation" : (warp < kMlpActWarps + kMlpLoadWarps ? "weights" : "mma"));
   tc_fence_before();
   __syncthreads();
   if (warp == kMlpActWarps + kMlpLoadWarps) {
      __syncwarp();
      tc_fence_after();
      tmem_dealloc(tmem_base, pl.tmem_cols);
   }
}

} // namespace umma

// Launches the tensor-core chain when the widths belong to it; returns -1 when the caller should use another kernel.
int launch_mlp_f32_umma(cudaStream_t s, const sofie_mlp_desc *d, const float *X, const float *const *W, const float *const *B, float *Y)
{
   using namespace umma;
   if (!sofie_mlp_tensor_core_shape(d)) return -1;
   MlpTcPlan pl = {};
   pl.M = d->M;
   pl.layers = d->layers;
   int kmax = 0, npmax = 0;
   for (int l = 0; l < d->layers; l++) {
      const int K = d->dims[l], N = d->dims[l + 1];
      pl.K[l] = K;
      pl.N[l] = N;
      pl.Np[l] = (N + 15) & ~15;
      pl.relu[l] = d->relu[l];
      pl.nk[l] = d->w_is_nk[l];
      pl.W[l] = W[l];
      pl.B[l] = B ? B[l] : nullptr;
      if (K > kmax) kmax = K;
      if (pl.Np[l] > npmax) npmax = pl.Np[l];
   }
   pl.a_lbo = 128 * 16 + kMlpPad;
   pl.a_bytes = (uint32_t)(kmax / 4) * pl.a_lbo;
   pl.stage_bytes = (uint32_t)(kMlpKC / 4) * ((uint32_t)(2 * npmax * 16) + kMlpPad);
   pl.stage_bytes = (pl.stage_bytes + 127) & ~127u;
   pl.stages = kMlpMaxStages;
   while (pl.stages > 2 && 2 * pl.a_bytes + pl.stages * pl.stage_bytes + 128 > 226 * 1024) pl.stages--;
   uint32_t cols = 32;
   while (cols < (uint32_t)(2 * npmax)) cols <<= 1;
   pl.tmem_cols = cols;
   const int smem = (int)(2 * pl.a_bytes + pl.stages * pl.stage_bytes) + 128;
   if (smem > 226 * 1024) return -1;
   uint32_t *status = device_status_word(s);
   if (!status) return fail(SOFIE_CUDA_ERR_CUDA, "cannot allocate the device status word");
   const int slabs = (d->M + 127) / 128;
   const int grid = slabs < kNumSMs ? slabs : kNumSMs;
   const int x_vec = d->dims[0] % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0;
   auto kern = umma_mlp_kernel;
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
   SOFIE_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(kMlpTcThreads), smem, s, pl, X, Y, x_vec, status));
   SOFIE_LAUNCH_CHECK("umma_mlp_kernel");
   set_last_engine(SOFIE_ENGINE_TCGEN05);
   return SOFIE_CUDA_OK;
}

} // namespace sofie
