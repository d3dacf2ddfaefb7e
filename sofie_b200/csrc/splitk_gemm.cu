// Skinny fp32 GEMM: few output columns (N <= 16), few rows, long K -- the shape of a classifier head
// behind a flattened feature map (256 x 10 x 4096). A 128 x N tile machine would run it on two or
// three SMs; here K is split across the grid instead. Pass 1 writes per-slab partial dot products
// to a scratch buffer [splits][M][N]; pass 2 adds the slabs in a fixed order (deterministic, no
// atomics) and applies alpha, bias and Relu.
#include "contract.cuh"

#include <cstdlib>
#include <map>
#include <mutex>
#include <vector>

namespace sofie {

constexpr int kSplitKMaxN = 16;
constexpr int kSplitKWarps = 8;

// A block = 8 output rows (one per warp) over one K slab, all N columns. The slab of B is staged in
// shared memory once per block, in chunks of kSplitKChunk elements of K, and shared by the 8 rows;
// a lane reads 16 bytes of its A row and of every staged B row per step, so global loads are whole
// 512-byte warp requests and several are in flight per lane.
constexpr int kSplitKChunk = 512; // floats of K per staged chunk: 16 x 512 x 4 B = 32 KB at most

template <bool TB>
__global__ void __launch_bounds__(kSplitKWarps * 32)
gemm_f32_splitk_partial_kernel(int M, int N, int K, int slab, const float *__restrict__ A, const float *__restrict__ B,
                               float *__restrict__ partial)
{
   __shared__ __align__(16) float bs[kSplitKMaxN * kSplitKChunk];
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
   griddep_launch_dependents();
   griddep_wait(); // A (and possibly B) are the previous kernel's output; nothing worth doing before it
   const int m = blockIdx.x * kSplitKWarps + warp;
   const int s = blockIdx.y;
   const int k0 = s * slab, k1 = min(K, k0 + slab);
   float acc[kSplitKMaxN];
#pragma unroll
   for (int n = 0; n < kSplitKMaxN; n++) acc[n] = 0.f;
   const float *a = A + (size_t)(m < M ? m : 0) * K;
   const bool a_vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
   for (int c0 = k0; c0 < k1; c0 += kSplitKChunk) {
      const int len = min(kSplitKChunk, k1 - c0);
      __syncthreads(); // the previous chunk is no longer read
      for (int i = threadIdx.x; i < N * kSplitKChunk; i += kSplitKWarps * 32) {
         const int n = TB ? i / kSplitKChunk : i % N, kk = TB ? i % kSplitKChunk : i / N;
         float v = 0.f;
         if (kk < len) v = TB ? B[(size_t)n * K + c0 + kk] : B[(size_t)(c0 + kk) * N + n];
         bs[n * kSplitKChunk + kk] = v;
      }
      __syncthreads();
      if (m < M) {
#pragma unroll 2
         for (int kk = lane * 4; kk < len; kk += 128) {
            float4 av;
            if (a_vec && kk + 3 < len) {
               av = *reinterpret_cast<const float4 *>(a + c0 + kk);
            } else {
               av.x = a[c0 + kk];
               av.y = kk + 1 < len ? a[c0 + kk + 1] : 0.f;
               av.z = kk + 2 < len ? a[c0 + kk + 2] : 0.f;
               av.w = kk + 3 < len ? a[c0 + kk + 3] : 0.f;
            }
#pragma unroll
            for (int n = 0; n < kSplitKMaxN; n++) {
               if (n < N) {
                  const float4 bv = *reinterpret_cast<const float4 *>(bs + n * kSplitKChunk + kk);
                  acc[n] = fmaf(av.x, bv.x, acc[n]);
                  acc[n] = fmaf(av.y, bv.y, acc[n]);
                  acc[n] = fmaf(av.z, bv.z, acc[n]);
                  acc[n] = fmaf(av.w, bv.w, acc[n]);
               }
            }
         }
      }
   }
   if (m >= M) return;
#pragma unroll
   for (int n = 0; n < kSplitKMaxN; n++) {
      if (n < N) {
         float v = acc[n];
         for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
         if (lane == 0) partial[((size_t)s * M + m) * N + n] = v;
      }
   }
}

__global__ void gemm_f32_splitk_reduce_kernel(sofie_gemm_f32_desc d, int splits, const float *__restrict__ partial,
                                              const float *__restrict__ C, float *__restrict__ Y)
{
   const size_t total = (size_t)d.M * d.N;
   griddep_launch_dependents();
   griddep_wait(); // the partial sums of the kernel before
   for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      float sum = 0.f;
      for (int s = 0; s < splits; s++) sum += partial[(size_t)s * total + i];
      float y = d.alpha * sum;
      if (d.bias_kind == 1) y += d.beta * C[i % d.N];
      else if (d.bias_kind == 2) y += d.beta * C[i];
      Y[i] = d.relu ? relu_ref(y) : y;
   }
}

// ------------------------------------------------------------------------------------------------
// Row-block variant: ONE launch, no scratch. A block owns kRowBlockRows rows of A and the whole of K;
// its 256 threads split K in 16-byte steps, and a thread keeps the N values of B of its step in
// registers for all the block's rows (B is read once per block from L2, A once in all). The per-thread
// sums are added across the warp by shuffles and across the 8 warps in warp order through shared
// memory, so the result does not depend on timing. Taken for classifier heads on small batches, where
// the two launches of the split-K pair and its scratch round trip cost more than the arithmetic.
// four rows per block measured best inside the C2 step (72.3 us against 73.7 with two and 74.8 with eight)
constexpr int kRowBlockRows = 4;
constexpr int kRowBlockMaxRows = 2048; // beyond this B would be re-read from L2 too often: split-K instead

template <int NN>
__global__ void __launch_bounds__(256)
gemm_f32_rowblock_kernel(sofie_gemm_f32_desc d, const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ C,
                         float *__restrict__ Y)
{
   __shared__ float s_part[8][kRowBlockRows][NN];
   const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
   const int m0 = blockIdx.x * kRowBlockRows, K = d.K;
   griddep_launch_dependents();
   griddep_wait(); // A is the previous kernel's output
   float acc[kRowBlockRows][NN];
#pragma unroll
   for (int r = 0; r < kRowBlockRows; r++)
#pragma unroll
      for (int n = 0; n < NN; n++) acc[r][n] = 0.f;
   const float *arow[kRowBlockRows];
#pragma unroll
   for (int r = 0; r < kRowBlockRows; r++) arow[r] = A + (size_t)min(m0 + r, d.M - 1) * K; // rows past M repeat the last one, not stored
   for (int k = threadIdx.x * 4; k < K; k += 1024) {
      float4 b[NN];
#pragma unroll
      for (int n = 0; n < NN; n++) b[n] = __ldg(reinterpret_cast<const float4 *>(B + (size_t)n * K + k));
#pragma unroll
      for (int r = 0; r < kRowBlockRows; r++) {
         const float4 a = *reinterpret_cast<const float4 *>(arow[r] + k);
#pragma unroll
         for (int n = 0; n < NN; n++) {
            acc[r][n] = fmaf(a.x, b[n].x, acc[r][n]);
            acc[r][n] = fmaf(a.y, b[n].y, acc[r][n]);
            acc[r][n] = fmaf(a.z, b[n].z, acc[r][n]);
            acc[r][n] = fmaf(a.w, b[n].w, acc[r][n]);
         }
      }
   }
#pragma unroll
   for (int r = 0; r < kRowBlockRows; r++)
#pragma unroll
      for (int n = 0; n < NN; n++) {
         float v = acc[r][n];
#pragma unroll
         for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
         if (lane == 0) s_part[warp][r][n] = v;
      }
   __syncthreads();
   if (threadIdx.x < kRowBlockRows * NN) {
      const int r = threadIdx.x / NN, n = threadIdx.x - r * NN, m = m0 + r;
      if (m < d.M) {
         float sum = 0.f;
#pragma unroll
         for (int w = 0; w < 8; w++) sum += s_part[w][r][n];
         float y = d.alpha * sum;
         if (d.bias_kind == 1) y += d.beta * C[n];
         else if (d.bias_kind == 2) y += d.beta * C[(size_t)m * NN + n];
         Y[(size_t)m * NN + n] = d.relu ? relu_ref(y) : y;
      }
   }
}

bool rowblock_shape_ok(const sofie_gemm_f32_desc &d, const float *A, const float *B)
{
   static const bool enabled = [] { const char *e = getenv("SOFIE_CUDA_GEMM_ROWBLOCK"); return !e || atoi(e) != 0; }();
   return enabled && !d.transA && d.transB && d.N <= kSplitKMaxN && d.K >= 1024 && d.K % 4 == 0 && d.M <= kRowBlockMaxRows &&
          (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0;
}

int launch_gemm_f32_rowblock(cudaStream_t s, const sofie_gemm_f32_desc &d, const float *A, const float *B, const float *C, float *Y)
{
   if (!rowblock_shape_ok(d, A, B)) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "not a row-block GEMM shape");
   const dim3 grid(ceil_div(d.M, kRowBlockRows)), block(256);
#define SOFIE_ROWBLOCK(NN) \
   case NN: SOFIE_CUDA_TRY(launch_dependent(gemm_f32_rowblock_kernel<NN>, grid, block, 0, s, d, A, B, C, Y)); break
   switch (d.N) {
      SOFIE_ROWBLOCK(1); SOFIE_ROWBLOCK(2); SOFIE_ROWBLOCK(3); SOFIE_ROWBLOCK(4); SOFIE_ROWBLOCK(5); SOFIE_ROWBLOCK(6);
      SOFIE_ROWBLOCK(7); SOFIE_ROWBLOCK(8); SOFIE_ROWBLOCK(9); SOFIE_ROWBLOCK(10); SOFIE_ROWBLOCK(11); SOFIE_ROWBLOCK(12);
      SOFIE_ROWBLOCK(13); SOFIE_ROWBLOCK(14); SOFIE_ROWBLOCK(15);
   default: SOFIE_CUDA_TRY(launch_dependent(gemm_f32_rowblock_kernel<16>, grid, block, 0, s, d, A, B, C, Y)); break;
   }
#undef SOFIE_ROWBLOCK
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

bool splitk_shape_ok(const sofie_gemm_f32_desc &d)
{
   return !d.transA && d.N <= kSplitKMaxN && d.K >= 1024 && (long long)d.M * d.N <= (1 << 16);
}

int splitk_splits(const sofie_gemm_f32_desc &d, size_t scratch_floats)
{
   // enough (row group, slab) blocks to fill the GPU about four times, slabs of at least 128 elements of K
   const int row_groups = ceil_div(d.M, kSplitKWarps);
   int splits = ceil_div(4 * kNumSMs, row_groups);
   if (splits > d.K / 128) splits = d.K / 128;
   if (splits > 64) splits = 64;
   if (splits < 1) splits = 1;
   while (splits > 1 && (size_t)splits * d.M * d.N > scratch_floats) splits--;
   return splits;
}

// Runs both passes with the given scratch buffer of `scratch_floats` floats (device memory).
int launch_gemm_f32_splitk(cudaStream_t s, const sofie_gemm_f32_desc &d, const float *A, const float *B, const float *C,
                           float *Y, float *scratch, size_t scratch_floats)
{
   if (!splitk_shape_ok(d)) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "split-K GEMM takes A[M,K], N <= 16, K >= 1024, M*N <= 65536");
   const int splits = splitk_splits(d, scratch_floats);
   if ((size_t)splits * d.M * d.N > scratch_floats)
      return fail(SOFIE_CUDA_ERR_NOMEM, "split-K scratch of %zu floats is too small for M*N = %lld", scratch_floats,
                  (long long)d.M * d.N);
   int slab = (d.K + splits - 1) / splits;
   slab = (slab + 127) & ~127; // whole 512-byte warp requests per slab
   const int used = (d.K + slab - 1) / slab;
   dim3 grid(ceil_div(d.M, kSplitKWarps), used);
   if (d.transB)
      SOFIE_CUDA_TRY(launch_dependent(gemm_f32_splitk_partial_kernel<true>, grid, dim3(kSplitKWarps * 32), 0, s, d.M, d.N, d.K, slab, A, B, scratch));
   else
      SOFIE_CUDA_TRY(launch_dependent(gemm_f32_splitk_partial_kernel<false>, grid, dim3(kSplitKWarps * 32), 0, s, d.M, d.N, d.K, slab, A, B, scratch));
   const int blocks = (int)ceil_div<size_t>((size_t)d.M * d.N, 256);
   SOFIE_CUDA_TRY(launch_dependent(gemm_f32_splitk_reduce_kernel, dim3(blocks), dim3(256), 0, s, d, used, (const float *)scratch, C, Y));
   set_last_engine(SOFIE_ENGINE_SIMT);
   return SOFIE_CUDA_OK;
}

// Library-owned scratch of the regular entry point. A pool of buffers per device is allocated on the
// first call on that device (which must come before any stream capture); every stream that calls
// gets its own buffer from the pool, so calls on different streams never share one and no
// allocation happens once a capture is running.
constexpr size_t kSplitKScratchFloats = size_t(1) << 19; // 2 MB: 64 slabs x 8192 outputs
constexpr int kSplitKPoolBuffers = 16;

struct SplitKDevicePool {
   float *base = nullptr;
   std::map<cudaStream_t, int> slot_of;
   std::vector<int> free_slots;
   int next_slot = 0;
};
std::mutex g_splitk_pool_mutex;
SplitKDevicePool g_splitk_pools[64];

float *splitk_scratch_for(cudaStream_t s)
{
   int dev = 0;
   if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
   std::lock_guard<std::mutex> lock(g_splitk_pool_mutex);
   SplitKDevicePool &pool = g_splitk_pools[dev];
   if (!pool.base) {
      if (cudaMalloc(&pool.base, kSplitKPoolBuffers * kSplitKScratchFloats * sizeof(float)) != cudaSuccess) {
         cudaGetLastError();
         pool.base = nullptr;
         return nullptr;
      }
   }
   auto it = pool.slot_of.find(s);
   if (it == pool.slot_of.end()) {
      int slot;
      if (!pool.free_slots.empty()) {
         slot = pool.free_slots.back();
         pool.free_slots.pop_back();
      } else if (pool.next_slot < kSplitKPoolBuffers) {
         slot = pool.next_slot++;
      } else {
         return nullptr;
      }
      it = pool.slot_of.emplace(s, slot).first;
   }
   return pool.base + (size_t)it->second * kSplitKScratchFloats;
}

// A stream that is about to be destroyed gives its buffer back (called by the context's destructor after
// the stream has drained), so that the pool bounds the streams alive at one time, not the streams ever made.
void splitk_scratch_release(int device, cudaStream_t s)
{
   if (device < 0 || device >= 64) return;
   std::lock_guard<std::mutex> lock(g_splitk_pool_mutex);
   SplitKDevicePool &pool = g_splitk_pools[device];
   auto it = pool.slot_of.find(s);
   if (it == pool.slot_of.end()) return;
   pool.free_slots.push_back(it->second);
   pool.slot_of.erase(it);
}

int launch_gemm_f32_splitk_auto(cudaStream_t s, const sofie_gemm_f32_desc &d, const float *A, const float *B,
                                const float *C, float *Y)
{
   if (!splitk_shape_ok(d)) return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "not a split-K shape");
   float *scratch = splitk_scratch_for(s);
   if (!scratch) return fail(SOFIE_CUDA_ERR_NOMEM, "no split-K scratch buffer: allocation failed (first call during a stream capture?) or more than 16 streams in use at one time");
   return launch_gemm_f32_splitk(s, d, A, B, C, Y, scratch, kSplitKScratchFloats);
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant. Its scratch is this file-scope device array, so no device allocation
// takes place on any call. In host code the array's name is only a stand-in symbol, not a device
// address: the address each device uses is looked up once per device with cudaGetSymbolAddress
// (with that device current) and that pointer is what the kernels receive.
constexpr size_t kSplitKStaticFloats = SOFIE_CUDA_SPLITK_STATIC_FLOATS;
static __device__ __align__(256) float g_splitk_static_scratch[kSplitKStaticFloats];

static float *splitk_static_scratch(int *status)
{
   static std::mutex mutex;
   static float *per_device[64] = {nullptr};
   int dev = 0;
   cudaError_t err = cudaGetDevice(&dev);
   if (err != cudaSuccess || dev < 0 || dev >= 64) {
      *status = fail(SOFIE_CUDA_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
      return nullptr;
   }
   std::lock_guard<std::mutex> lock(mutex);
   if (!per_device[dev]) {
      float *p = nullptr;
      err = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_splitk_static_scratch);
      if (err != cudaSuccess || !p) {
         cudaGetLastError();
         *status = fail(SOFIE_CUDA_ERR_CUDA, "cudaGetSymbolAddress of the static split-K scratch: %s", cudaGetErrorString(err));
         return nullptr;
      }
      per_device[dev] = p;
   }
   *status = SOFIE_CUDA_OK;
   return per_device[dev];
}

} // namespace sofie

extern "C" int sofie_cuda_gemm_f32_splitk_static(void *stream, const sofie_gemm_f32_desc *d, const float *A, const float *B,
                                                 const float *C, float *Y)
{
   using namespace sofie;
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0, "bad GEMM shape %d x %d x %d", d->M, d->N, d->K);
   SOFIE_REQUIRE(d->bias_kind >= 0 && d->bias_kind <= 2, "bias_kind must be 0, 1 or 2");
   SOFIE_REQUIRE(d->bias_kind == 0 || C != nullptr, "bias_kind set but C is NULL");
   if (d->M == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(A && B && Y, "NULL tensor");
   if (!splitk_shape_ok(*d))
      return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "the allocation-free GEMM takes A[M,K] (no transA), N <= 16 and K >= 1024; got %d x %d x %d",
                  d->M, d->N, d->K);
   if ((long long)d->M * d->N > SOFIE_CUDA_SPLITK_STATIC_MAX_OUTPUTS)
      return fail(SOFIE_CUDA_ERR_INVALID, "M*N = %lld outputs exceed the %d the static scratch is sized for",
                  (long long)d->M * d->N, SOFIE_CUDA_SPLITK_STATIC_MAX_OUTPUTS);
   int rc = SOFIE_CUDA_OK;
   float *scratch = splitk_static_scratch(&rc);
   if (!scratch) return rc;
   return launch_gemm_f32_splitk(as_stream(stream), *d, A, B, C, Y, scratch, kSplitKStaticFloats);
}
