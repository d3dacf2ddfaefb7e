// Fused multi-layer perceptron for small layers: Y = L_{n-1}(... L_0(X)), L_l(x) = act(x W_l^T + b_l),
// all layer widths <= 256 and all weights together small enough for shared memory. One launch
// replaces one GEMM launch per layer: at these sizes (C1: 64 -> 128 -> 128 -> 10, 104 KB of
// weights, 52 kFLOP per sample) a layer is far too small to fill the GPU and its time is launch
// latency plus the round trip of its activations through memory. A block keeps every layer's
// weights in shared memory and walks tiles of ROWS batch rows; activations never leave the SM.
//   weights     [n][ld], ld = K rounded up to 4, plus a pad that makes ld / 4 odd: the rows that the
//               column subgroups of a warp read start 16 bytes apart in the banks
//   activations [row][ld], same padding rule: the rows of a quarter warp hit distinct banks
//   thread      (warp w, lane): batch row lane % ROWS, columns q + CSTEP j with q = w * SUB + lane / ROWS;
//               per four k one 16-byte load of its row and one 16-byte load per column
//   ROWS        32, 16 or 8: the largest that still gives every SM a tile, so that a small batch
//               spreads over the whole GPU (each block stages the weights from L2 either way)
// Staging uses 16-byte asynchronous copies (all of a block's weight bytes in flight at once) when
// the layout allows it: [N][K] weights, K a multiple of 4, 16-byte aligned pointers. The input
// tile of the next batch rows is fetched while the layers after the first run.
// fp32 FMA throughout (K <= 256 per layer, accumulation in order of k).
#include "common.cuh"
#include "contract.cuh"

namespace sofie {
namespace {

constexpr int kMlpThreads = 256;

struct MlpParams {
   sofie_mlp_desc d;
   const float *W[SOFIE_MLP_MAX_LAYERS];
   const float *B[SOFIE_MLP_MAX_LAYERS];
   int w_off[SOFIE_MLP_MAX_LAYERS]; // offset of layer l's [Np][w_ld] weights in shared memory, in floats
   int w_ld[SOFIE_MLP_MAX_LAYERS];
   int b_off[SOFIE_MLP_MAX_LAYERS]; // offset of its Np biases
   int x_off, x_ld;                 // input tile [ROWS][x_ld]
   int act_off[2], act_ld;          // the two activation buffers [ROWS][act_ld]
   int w_vec[SOFIE_MLP_MAX_LAYERS]; // layer's weights can be staged with 16-byte copies
   int x_vec;
};

inline int padded_ld(int k) { return sofie_mlp_padded_ld(k); }

__device__ __forceinline__ void cp_async16(float *dst_smem, const float *src, bool valid)
{
   const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
   const int bytes = valid ? 16 : 0; // 0 source bytes: the 16 destination bytes are zero-filled
   asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(float *dst_smem, const float *src)
{
   const unsigned d = (unsigned)__cvta_generic_to_shared(dst_smem);
   asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }
// wait until at most `n` of the most recently committed groups are still in flight (the count is an immediate)
__device__ __forceinline__ void cp_async_wait_pending(int n)
{
   switch (n) {
   case 0: asm volatile("cp.async.wait_group 0;\n" ::: "memory"); break;
   case 1: asm volatile("cp.async.wait_group 1;\n" ::: "memory"); break;
   case 2: asm volatile("cp.async.wait_group 2;\n" ::: "memory"); break;
   case 3: asm volatile("cp.async.wait_group 3;\n" ::: "memory"); break;
   case 4: asm volatile("cp.async.wait_group 4;\n" ::: "memory"); break;
   case 5: asm volatile("cp.async.wait_group 5;\n" ::: "memory"); break;
   case 6: asm volatile("cp.async.wait_group 6;\n" ::: "memory"); break;
   case 7: asm volatile("cp.async.wait_group 7;\n" ::: "memory"); break;
   default: asm volatile("cp.async.wait_group 8;\n" ::: "memory"); break;
   }
}

// Rows of `kq` 16-byte pieces walked by the whole block without a division per piece: the thread's piece
// index advances by the block size, that is by (step_n rows, step_c pieces) with one carry.
struct PieceWalker {
   int n, c, step_n, step_c, kq;
   __device__ __forceinline__ PieceWalker(int tid, int kq_) : kq(kq_)
   {
      n = tid / kq;
      c = tid - n * kq;
      step_n = kMlpThreads / kq;
      step_c = kMlpThreads - step_n * kq;
   }
   __device__ __forceinline__ void next()
   {
      n += step_n;
      c += step_c;
      if (c >= kq) {
         c -= kq;
         n++;
      }
   }
};

template <int ROWS>
__device__ __forceinline__ void load_x_tile(const MlpParams &p, const float *__restrict__ X, float *sm, int tile, int tid)
{
   const int K0 = p.d.dims[0], M = p.d.M, m0 = tile * ROWS;
   float *xin = sm + p.x_off;
   if (p.x_vec) {
      for (PieceWalker it(tid, K0 >> 2); it.n < ROWS; it.next()) {
         const bool ok = m0 + it.n < M;
         cp_async16(xin + it.n * p.x_ld + 4 * it.c, X + (size_t)(ok ? m0 + it.n : 0) * K0 + 4 * it.c, ok);
      }
   } else {
      const int K0p = (K0 + 3) & ~3;
      for (int i = tid; i < ROWS * K0p; i += kMlpThreads) {
         const int r = i / K0p, k = i - r * K0p;
         xin[r * p.x_ld + k] = (m0 + r < M && k < K0) ? __ldg(X + (size_t)(m0 + r) * K0 + k) : 0.f;
      }
   }
}

// One layer for one thread: batch row `arow`, columns q + CSTEP j for j < J, J = NB * 32 / CSTEP known at compile time
// (NB = the layer's width in units of 32 columns).
template <int ROWS, int NB>
__device__ __forceinline__ void mlp_layer(const float *__restrict__ arow, const float *__restrict__ wrow, const float *__restrict__ bs,
                                          float *__restrict__ nxt, int Kp, int ldw, int N4, int q, bool relu)
{
   constexpr int CSTEP = 8 * (32 / ROWS);
   constexpr int J = NB * 32 / CSTEP;
   float acc[J];
#pragma unroll
   for (int j = 0; j < J; j++) acc[j] = 0.f;
#pragma unroll 2
   for (int k = 0; k < Kp; k += 4) {
      const float4 a = *reinterpret_cast<const float4 *>(arow + k);
#pragma unroll
      for (int j = 0; j < J; j++) {
         const float4 wv = *reinterpret_cast<const float4 *>(wrow + j * CSTEP * ldw + k);
         acc[j] = fmaf(a.x, wv.x, acc[j]);
         acc[j] = fmaf(a.y, wv.y, acc[j]);
         acc[j] = fmaf(a.z, wv.z, acc[j]);
         acc[j] = fmaf(a.w, wv.w, acc[j]);
      }
   }
#pragma unroll
   for (int j = 0; j < J; j++) {
      const int n = q + CSTEP * j;
      if (n < N4) {
         const float v = acc[j] + bs[n];
         nxt[n] = relu ? relu_ref(v) : v;
      }
   }
}

template <int ROWS>
__global__ void __launch_bounds__(kMlpThreads, 1)
mlp_fused_f32_kernel(MlpParams p, const float *__restrict__ X, float *__restrict__ Y)
{
   constexpr int SUB = 32 / ROWS;  // column subgroups of a warp; two columns of one thread are 8 * SUB apart
   extern __shared__ __align__(16) float sm[];
   const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
   const int r = lane % ROWS, q = w * SUB + lane / ROWS;
   const int L = p.d.layers, M = p.d.M;
   const int tiles = (M + ROWS - 1) / ROWS;
   // ---- the first input tile, then weights and biases, once per block
   // Copy groups in order: [input tile + layer 0], [layer 1], ..., [layer L-1]; layer l of the first tile
   // starts as soon as its own group has landed while the later layers' weights are still arriving.
   load_x_tile<ROWS>(p, X, sm, blockIdx.x, tid);
   for (int l = 0; l < L; l++) {
      const int K = p.d.dims[l], N = p.d.dims[l + 1], Np = (N + 31) & ~31, ld = p.w_ld[l];
      float *wt = sm + p.w_off[l];
      const float *Wg = p.W[l];
      if (p.w_vec[l]) {
         for (PieceWalker it(tid, K >> 2); it.n < N; it.next()) cp_async16(wt + it.n * ld + 4 * it.c, Wg + (size_t)it.n * K + 4 * it.c, true);
         for (int i = tid; i < (Np - N) * ld; i += kMlpThreads) wt[N * ld + i] = 0.f; // columns past N contribute nothing
      } else if (p.d.w_is_nk[l]) {
         const int Kp = (K + 3) & ~3;
         for (int i = tid; i < Np * Kp; i += kMlpThreads) {
            const int n = i / Kp, k = i - n * Kp;
            wt[n * ld + k] = (n < N && k < K) ? __ldg(Wg + (size_t)n * K + k) : 0.f;
         }
      } else {
         // global [K][N] -> shared [n][k]: consecutive threads take consecutive n, reads coalesced
         const int Kp = (K + 3) & ~3;
         for (int i = tid; i < Np * Kp; i += kMlpThreads) {
            const int k = i / Np, n = i - k * Np;
            wt[n * ld + k] = (n < N && k < K) ? __ldg(Wg + (size_t)k * N + n) : 0.f;
         }
      }
      float *bs = sm + p.b_off[l];
      for (int n = tid; n < Np; n += kMlpThreads) {
         if (n < N && p.B[l])
            cp_async4(bs + n, p.B[l] + n);
         else
            bs[n] = 0.f;
      }
      cp_async_commit();
   }
   bool first = true;
   for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      const int m0 = tile * ROWS;
      if (!first) {
         cp_async_wait_all();
         __syncthreads(); // this tile's input has landed; the previous tile's buffers are free
      }
      for (int l = 0; l < L; l++) {
         if (first) {
            // groups still allowed in flight: the later layers' and, behind layer 0, the next tile's input
            cp_async_wait_pending(L - 1 - l + (l > 0 ? 1 : 0));
            __syncthreads();
         }
         const int K = p.d.dims[l], N = p.d.dims[l + 1], Kp = (K + 3) & ~3;
         const int ldw = p.w_ld[l], lda = l == 0 ? p.x_ld : p.act_ld;
         const float *arow = sm + (l == 0 ? p.x_off : p.act_off[(l - 1) & 1]) + r * lda;
         const float *wrow = sm + p.w_off[l] + q * ldw;
         const float *bs = sm + p.b_off[l];
         const bool relu = p.d.relu[l] != 0;
         const int N4 = (N + 3) & ~3; // the next layer reads k up to its K rounded to 4: columns N .. N4 are written as zeros
         float *nxt = sm + p.act_off[l & 1] + r * p.act_ld;
         switch (((N + 31) & ~31) >> 5) { // the column count is a compile-time constant inside: no predicated-off work
         case 1: mlp_layer<ROWS, 1>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         case 2: mlp_layer<ROWS, 2>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         case 3: mlp_layer<ROWS, 3>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         case 4: mlp_layer<ROWS, 4>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         case 5: mlp_layer<ROWS, 5>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         case 6: mlp_layer<ROWS, 6>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         case 7: mlp_layer<ROWS, 7>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         default: mlp_layer<ROWS, 8>(arow, wrow, bs, nxt, Kp, ldw, N4, q, relu); break;
         }
         __syncthreads(); // the next layer (or the copy-out) reads what every warp wrote
         if (l == 0) {
            if (tile + (int)gridDim.x < tiles) load_x_tile<ROWS>(p, X, sm, tile + gridDim.x, tid); // the input buffer is free
            cp_async_commit(); // committed even when empty: the group count above does not depend on the tile
         }
      }
      first = false;
      {
         // the tile's rows are one contiguous piece of Y
         const int N = p.d.dims[L];
         const float *out = sm + p.act_off[(L - 1) & 1];
         const int rows = M - m0 < ROWS ? M - m0 : ROWS;
         float *Yt = Y + (size_t)m0 * N;
         for (int i = tid; i < rows * N; i += kMlpThreads) {
            const int rr = i / N, n = i - rr * N;
            Yt[i] = out[rr * p.act_ld + n];
         }
      }
   }
   cp_async_wait_all();
}

template <int ROWS>
int launch_mlp(cudaStream_t stream, MlpParams &p, int floats, int maxact, const float *X, float *Y)
{
   p.x_off = floats;
   p.x_ld = padded_ld(p.d.dims[0]);
   floats += ROWS * p.x_ld;
   p.act_ld = padded_ld(maxact);
   p.act_off[0] = floats;
   p.act_off[1] = floats + ROWS * p.act_ld;
   floats += 2 * ROWS * p.act_ld;
   const size_t smem = (size_t)floats * sizeof(float);
   SOFIE_CUDA_TRY(cudaFuncSetAttribute(mlp_fused_f32_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
   const int tiles = (p.d.M + ROWS - 1) / ROWS;
   mlp_fused_f32_kernel<ROWS><<<tiles < kNumSMs ? tiles : kNumSMs, kMlpThreads, smem, stream>>>(p, X, Y);
   SOFIE_LAUNCH_CHECK("mlp_fused_f32_kernel");
   return SOFIE_CUDA_OK;
}

} // namespace
} // namespace sofie

using namespace sofie;

extern "C" size_t sofie_cuda_mlp_f32_smem(const sofie_mlp_desc *d)
{
   if (!d || d->layers < 1 || d->layers > SOFIE_MLP_MAX_LAYERS) return 0;
   return sofie_mlp_smem_bytes(d);
}

extern "C" int sofie_cuda_mlp_f32(void *stream, const sofie_mlp_desc *d, const float *X, const float *const *W, const float *const *B, float *Y)
{
   SOFIE_REQUIRE(d != nullptr, "NULL descriptor");
   SOFIE_REQUIRE(d->layers >= 1 && d->layers <= SOFIE_MLP_MAX_LAYERS, "1 to %d layers", SOFIE_MLP_MAX_LAYERS);
   SOFIE_REQUIRE(d->M >= 0, "negative batch");
   SOFIE_REQUIRE(W != nullptr, "NULL weight table");
   MlpParams p = {};
   p.d = *d;
   int floats = 0, maxact = 0;
   for (int l = 0; l <= d->layers; l++) {
      SOFIE_REQUIRE(d->dims[l] >= 1, "layer width must be positive");
      if (d->dims[l] > SOFIE_MLP_MAX_WIDTH)
         return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "the fused MLP takes layer widths up to %d, got %d", SOFIE_MLP_MAX_WIDTH, d->dims[l]);
      if (l >= 1 && d->dims[l] > maxact) maxact = d->dims[l];
   }
   for (int l = 0; l < d->layers; l++) {
      SOFIE_REQUIRE(W[l] != nullptr, "NULL weights of layer %d", l);
      const int K = d->dims[l], Np = (d->dims[l + 1] + 31) & ~31;
      p.W[l] = W[l];
      p.B[l] = B ? B[l] : nullptr;
      p.w_vec[l] = d->w_is_nk[l] && K % 4 == 0 && (reinterpret_cast<uintptr_t>(W[l]) & 15) == 0;
      p.w_ld[l] = padded_ld(K);
      p.w_off[l] = floats;
      floats += Np * p.w_ld[l];
      p.b_off[l] = floats;
      floats += Np;
   }
   p.x_vec = d->dims[0] % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0;
   // the size test assumes the largest tile, so that it does not depend on the batch
   const size_t worst = sofie_mlp_smem_bytes(d);
   if (worst > SOFIE_MLP_MAX_SMEM)
      return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "the fused MLP needs %zu bytes of shared memory for these layers (limit %d)", worst, SOFIE_MLP_MAX_SMEM);
   if (d->M == 0) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(X && Y, "NULL tensor");
   cudaStream_t s = as_stream(stream);
   // The tensor-core chain (umma_mlp.cu) runs when the caller forces that engine. It is not the default: measured on
   // B200 for 64 -> 128 -> 128 -> 10 it takes 42 us at 1024 rows (this file's FMA kernel: 17 us, on 128 SMs instead of 8)
   // and 311 us at 2^18 rows (one tensor-core GEMM launch per layer: 193 us) -- every CTA re-reads and re-splits all the
   // weights for each 128-row slab, and those reads from L2 and their shared-memory writes, not the MMAs, set its time.
   if (forced_engine() == SOFIE_ENGINE_TCGEN05) {
      const int rc = launch_mlp_f32_umma(s, d, X, W, B, Y);
      if (rc >= 0) return rc;
      return fail(SOFIE_CUDA_ERR_UNSUPPORTED, "these layer widths are not served by the tensor-core chain");
   }
   int rows = 32;
   while (rows > 8 && (d->M + rows - 1) / rows < kNumSMs) rows >>= 1;
   set_last_engine(SOFIE_ENGINE_SIMT);
   if (rows == 32) return launch_mlp<32>(s, p, floats, maxact, X, Y);
   if (rows == 16) return launch_mlp<16>(s, p, floats, maxact, X, Y);
   return launch_mlp<8>(s, p, floats, maxact, X, Y);
}
