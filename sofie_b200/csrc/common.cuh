// Shared host/device helpers of libSOFIE_cuda: status handling, launch checks, small math.
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "sofie_cuda.h"

namespace sofie {

// Thread-local text of the last failure, returned by sofie_cuda_last_error().
char *last_error_buffer();
int fail(int status, const char *fmt, ...);
void set_last_engine(int engine);
int forced_engine();

// Status word of the kernels that have bounded waits. A kernel that gives up stores a non-zero code
// there and returns normally, so the context stays usable. A stream that belongs to a context reports
// into that context's own word, which lies in mapped pinned host memory: sofie_cuda_ctx_fetch and
// sofie_cuda_ctx_check read it with a plain host load after the stream synchronisation they do anyway,
// and one Session never sees (or clears) another Session's failure. Launches on any other stream share
// one word per device in device memory, read by sofie_cuda_device_check().
uint32_t *device_status_word(cudaStream_t stream); // address the kernel writes to, nullptr on failure
void register_stream_status(cudaStream_t stream, uint32_t *word);
void unregister_stream_status(cudaStream_t stream);

#define SOFIE_CUDA_TRY(expr)                                                                         \
   do {                                                                                              \
      cudaError_t err__ = (expr);                                                                    \
      if (err__ != cudaSuccess)                                                                      \
         return ::sofie::fail(SOFIE_CUDA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                   \
                              cudaGetErrorString(err__), __FILE__, __LINE__);                        \
   } while (0)

#define SOFIE_LAUNCH_CHECK(name)                                                                     \
   do {                                                                                              \
      cudaError_t err__ = cudaGetLastError();                                                        \
      if (err__ != cudaSuccess)                                                                      \
         return ::sofie::fail(SOFIE_CUDA_ERR_CUDA, "launch of %s failed: %s", name,                  \
                              cudaGetErrorString(err__));                                            \
   } while (0)

#define SOFIE_REQUIRE(cond, ...)                                                                     \
   do {                                                                                              \
      if (!(cond)) return ::sofie::fail(SOFIE_CUDA_ERR_INVALID, __VA_ARGS__);                        \
   } while (0)

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

constexpr int kNumSMs = 148; // B200

// ---- programmatic dependent launch ---------------------------------------------------------------
// A kernel launched with launch_dependent() may start while the kernel before it on the stream is
// still running: its blocks become resident as soon as every block of the predecessor has executed
// griddep_launch_dependents() (or exited) and resources are free, run their prologue (barrier setup,
// TMEM allocation, constant weights into shared memory) and then block in griddep_wait() until the
// predecessor has completed and its writes are visible. Rules kept by every kernel launched this way:
// every block executes griddep_wait() before it reads or writes anything another kernel touches and
// before it exits (so that completion of this grid implies completion of all earlier ones); only
// constant data (weights, biases, descriptors) is touched before it. Both instructions are no-ops in
// a kernel that was launched the ordinary way. SOFIE_CUDA_PDL=0 turns the attribute off.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
bool pdl_enabled();

template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args)
{
   cudaLaunchConfig_t cfg = {};
   cfg.gridDim = grid;
   cfg.blockDim = block;
   cfg.dynamicSmemBytes = smem;
   cfg.stream = stream;
   cudaLaunchAttribute attr[1];
   attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
   attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
   cfg.attrs = attr;
   cfg.numAttrs = 1;
   return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T>
__host__ __device__ constexpr T ceil_div(T a, T b)
{
   return (a + b - 1) / b;
}

// ---- requantisation recipe shared by every int8 kernel -------------------------------------------
// q = clamp(rne((float)acc * mult), qmin - zp, qmax - zp) + zp, with no FMA contraction, so a CPU
// evaluating nearbyintf((float)acc * mult) under the default rounding mode gets the same bits.
__device__ __forceinline__ int requant_u8(int acc, float mult, int y_zp, int relu)
{
   // The clamp runs on the float product, the rounding after it: clamp(rne(v), lo, hi) == rne(clamp(v, lo, hi)) for
   // integer bounds because rounding is monotone. A clamped value lies in [-255, 255], where adding 1.5 * 2^23
   // rounds it to the nearest integer, ties to even, in the adder (full rate) and leaves that integer in the low
   // mantissa bits; the float-to-int conversion instruction this replaces runs at a fraction of that rate.
   // Relu on a quantised value, max(q, y_zp), is the lower bound 0 before the zero point is added.
   float v = __fmul_rn(__int2float_rn(acc), mult);
   if (y_zp == 0) {
      // zero point 0: the clamp to [0, 255] (whose lower bound is also the Relu) and the rounding are ONE conversion with
      // round-to-nearest-even and saturation to the uint8 range
      uint32_t q;
      asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(q) : "f"(v));
      return (int)q;
   }
   const float lo = relu ? 0.f : (float)(-y_zp), hi = (float)(255 - y_zp);
   v = fminf(fmaxf(v, lo), hi);
   return __float_as_int(__fadd_rn(v, 12582912.f)) - 0x4B400000 + y_zp;
}

__device__ __forceinline__ float relu_ref(float v)
{
   // The reference's `x > 0 ? x : 0`: NaN and -0 both become +0.
   return v > 0.f ? v : 0.f;
}

__device__ __forceinline__ uint16_t f32_to_bf16_rne(float x)
{
   uint32_t u = __float_as_uint(x);
   if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
   u += 0x7FFFu + ((u >> 16) & 1u);
   return (uint16_t)(u >> 16);
}

__device__ __forceinline__ float bf16_to_f32(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }

} // namespace sofie
