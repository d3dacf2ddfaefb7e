// sm_100a building blocks used by the tensor-core kernels: mbarrier, TMA (cp.async.bulk.tensor,
// never with cluster multicast), tcgen05 (TMEM allocation, MMA, commit, load) and the descriptors
// they take. Every wait is bounded: a wait that runs out records a code in the device status word
// and reports failure to its caller, which then leaves the kernel through the normal exit path
// (TMEM released), so the context stays usable.
#pragma once

#include <cuda.h>
#include "common.cuh"

namespace sofie {
namespace umma {

// ---- status codes written to the device status word ------------------------------------------
constexpr uint32_t kStatusWaitFull = 0x101;   // consumer gave up waiting for a TMA-filled stage
constexpr uint32_t kStatusWaitEmpty = 0x102;  // producer gave up waiting for a free stage
constexpr uint32_t kStatusWaitConv = 0x103;   // MMA issuer gave up waiting for the converted stage
constexpr uint32_t kStatusWaitAccum = 0x104;  // epilogue gave up waiting for the accumulator

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
   asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
   asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
   asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
   asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
   uint32_t done;
   asm volatile("{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(smem_u32(bar)), "r"(parity)
                : "memory");
   return done != 0;
}

// Bounded wait: about one second of SM clock at most. On give-up stores `code` (and where) in the
// status word, raises the CTA's abort flag and returns false.
constexpr long long kWaitLimitCycles = 2000000000LL;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *status, uint32_t code, uint32_t detail,
                                          long long limit_cycles = kWaitLimitCycles)
{
   if (mbar_try_wait(bar, parity)) return true;
   const long long start = clock64();
   while (true) {
      // poll a few times (each try_wait already suspends the thread for a while) before spending
      // issue slots on the clock and the abort flag
#pragma unroll 1
      for (int spin = 0; spin < 16; spin++)
         if (mbar_try_wait(bar, parity)) return true;
      if (*abort_flag) return false;
      if (clock64() - start > limit_cycles) {
         *abort_flag = 1;
         // The word may lie in mapped host memory, where a device atomic is not atomic for the host: plain
         // volatile accesses, detail first, the code last. When several CTAs give up together any one of them
         // may win; every one of them reports a real give-up.
         volatile uint32_t *w = status;
         if (w && w[0] == 0u) {
            w[1] = detail;
            w[2] = blockIdx.x;
            w[3] = blockIdx.y;
            __threadfence_system();
            w[0] = code;
            __threadfence_system();
         }
         return false;
      }
   }
}

// Optional self-profiling (compile with -DSOFIE_UMMA_PROFILE): every bounded wait adds the cycles it
// spent to a per-thread counter that the kernels of CTA 0 print per role when they finish.
#ifdef SOFIE_UMMA_PROFILE
#define SOFIE_PROF_DECL long long prof_wait = 0; const long long prof_begin = clock64();
#define SOFIE_PROF_WAIT(call) ([&] { const long long t0__ = clock64(); const bool r__ = (call); prof_wait += clock64() - t0__; return r__; }())
#define SOFIE_PROF_REPORT(role) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (threadIdx.x & 31) == 0) printf("[umma-prof] %s warp %d: total %lld cycles, waiting %lld\n", role, (int)(threadIdx.x >> 5), clock64() - prof_begin, prof_wait); } while (0)
#else
#define SOFIE_PROF_DECL
#define SOFIE_PROF_WAIT(call) (call)
#define SOFIE_PROF_REPORT(role) do { } while (0)
#endif

// Next slot of a ring of S pipeline stages and the parity of its barriers, without a division: the
// roles that walk the ring do so once per stage, on their critical path.
__device__ __forceinline__ void ring_next(int &slot, uint32_t &phase, int S)
{
   if (++slot == S) {
      slot = 0;
      phase ^= 1u;
   }
}

__device__ __forceinline__ void fence_proxy_async()
{
   asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA: tiled loads global -> shared, completion on an mbarrier. No multicast anywhere. -----
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
   asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, int x, int y, int z, int w,
                                            uint64_t *bar)
{
   asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar))
                : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map)
{
   asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tcgen05 / TMEM ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols)
{
   asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                "r"(ncols)
                : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
   asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
   asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrive on an mbarrier when all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
   asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                : "memory");
}

enum Kind { kTF32 = 0, kI8 = 1, kF8 = 2 };

template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate)
{
   if constexpr (KIND == kTF32) {
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                   "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                   : "memory");
   } else if constexpr (KIND == kI8) {
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                   "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                   : "memory");
   } else {
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                   "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                   : "memory");
   }
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster on one TPC run one MMA of 256 rows ---------
// The leader (cluster rank 0) issues the MMAs; every CTA keeps its 128 rows of A, its half of the
// rows of B and its 128 lanes of the accumulator. None of the loads below is a multicast load.
__device__ __forceinline__ uint32_t cluster_ctarank()
{
   uint32_t r;
   asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
   return r;
}
// Address, in the cluster's shared window, of the same shared-memory location in CTA `rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t cta_addr, uint32_t rank)
{
   uint32_t r;
   asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
   return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
   asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
   asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tensor copy into this CTA's shared memory whose completion bytes are counted on a barrier that may
// lie in the peer CTA (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr)
{
   asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
                : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t ncols)
{
   asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
   asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
   asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `cta_mask` once all MMAs issued
// so far by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t *bar, uint16_t cta_mask)
{
   asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                "h"(cta_mask)
                : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
   static_assert(KIND == kI8 || KIND == kF8, "pair MMAs are built for the 8-bit kinds");
   if constexpr (KIND == kI8) {
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                   "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                   : "memory");
   } else {
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                   "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                   : "memory");
   }
}

// 32 lanes x 32 columns of 32-bit accumulators: thread t of the warp receives lane (base + t),
// columns [col, col + 32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
   asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// The same for 16 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16])
{
   asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
template <int CH>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[CH])
{
   static_assert(CH == 16 || CH == 32, "chunk of 16 or 32 columns");
   if constexpr (CH == 32) tmem_ld_32x32(taddr, r);
   else tmem_ld_32x16(taddr, r);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors -------------------------------------------------------------------------------
// Shared-memory operand descriptor for a K-major tile whose rows are `row_bytes` (32, 64 or 128)
// bytes of K, stored densely and swizzled by TMA with the matching swizzle mode. Rows are grouped
// by 8 (one swizzle atom); groups follow each other at 8*row_bytes.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4 (unused here, 1)
//   bits 32-45 stride byte offset >> 4 bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 swizzle: 2 = 128 B, 4 = 64 B, 6 = 32 B
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, int row_bytes)
{
   const uint64_t layout = row_bytes == 128 ? 2 : (row_bytes == 64 ? 4 : 6);
   uint64_t desc = 0;
   desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
   desc |= (uint64_t)1 << 16;
   desc |= (uint64_t)((8 * row_bytes) >> 4) << 32;
   desc |= (uint64_t)1 << 46;
   desc |= layout << 61;
   return desc;
}

// The same swizzled K-major rows with the 8-row groups `sbo_bytes` apart instead of densely packed. The swizzle is applied
// to the absolute shared-memory address (bits 4-6 xor bits 7-9 for 128-byte rows, fewer bits for shorter rows), both by TMA
// when it writes and by the MMA when it reads, so the start address may be any row of a TMA-written region and the group
// stride any multiple of 16 bytes; the descriptor's base-offset field stays 0 (measured on B200: every row offset and group
// stride tried reads the right bytes with base offset 0, and the wrong ones with the offset the address suggests).
__device__ __forceinline__ uint64_t make_smem_desc_rows(uint32_t smem_addr, int row_bytes, uint32_t sbo_bytes)
{
   const uint64_t layout = row_bytes == 128 ? 2 : (row_bytes == 64 ? 4 : 6);
   uint64_t desc = 0;
   desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
   desc |= (uint64_t)1 << 16;
   desc |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
   desc |= (uint64_t)1 << 46;
   desc |= layout << 61;
   return desc;
}

// K-major operand without swizzle: the tile is made of 8-row x 16-byte core matrices, each 128
// contiguous bytes (8 rows at a 16-byte pitch). sbo_bytes is the distance between consecutive 8-row
// groups, lbo_bytes the distance between the two 16-byte K columns one MMA (32 bytes of K) reads.
__device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
   uint64_t desc = 0;
   desc |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
   desc |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
   desc |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
   desc |= (uint64_t)1 << 46;
   return desc;
}

// Instruction descriptor (dense, K-major A and B, M x N tile):
//   bits 4-5 accumulator format (1 = f32, 2 = s32)   bits 7-9 A format   bits 10-12 B format
//   bits 17-22 N >> 3                                 bits 24-28 M >> 4
template <int KIND>
__host__ __device__ constexpr uint32_t make_idesc(int M, int N)
{
   uint32_t c_fmt = (KIND == kI8) ? 2u : 1u;
   uint32_t a_fmt = (KIND == kTF32) ? 2u : 0u;                       // tf32 | uint8 | e4m3
   uint32_t b_fmt = (KIND == kTF32) ? 2u : ((KIND == kI8) ? 1u : 0u); // tf32 | int8  | e4m3
   return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// ---- host: tensor-map encoding through the driver entry point (no link-time libcuda) ----------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// rank-`rank` tensor map, innermost dimension first; strides in bytes for dims 1..rank-1.
int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, int swizzle_bytes);

} // namespace umma
} // namespace sofie
