// Context of one emitted Session on one GPU: stream, device arena, persistent allocations (weights),
// pinned staging for host<->device traffic, optional CUDA graph of the infer() kernel sequence.
//
// Replaces what the reference emits as Session data members: one std::vector<float> per weight
// (reference: src/SOFIE_core/src/RModel.cxx:574-595) and the `new char[]` intermediate pool
// (reference: src/SOFIE_core/src/RModel.cxx:597-604).
#include "common.cuh"
#include "contract.cuh"

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <thread>
#include <utility>
#include <vector>

namespace sofie {

static thread_local char g_last_error[512] = "";
static thread_local int g_last_engine = SOFIE_ENGINE_NONE;
static thread_local int g_default_device = -1; // device of contexts created with device < 0 on this thread (-1: environment)
// Initial kernel-family choice from the environment (SOFIE_CUDA_ENGINE = 0, 1 or 2), for A/B runs.
static int initial_engine()
{
   const char *env = std::getenv("SOFIE_CUDA_ENGINE");
   int v = env ? std::atoi(env) : 0;
   return (v >= 0 && v <= 2) ? v : 0;
}
static int g_forced_engine = initial_engine();

char *last_error_buffer() { return g_last_error; }

int fail(int status, const char *fmt, ...)
{
   va_list ap;
   va_start(ap, fmt);
   vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
   va_end(ap);
   return status;
}

void set_last_engine(int engine) { g_last_engine = engine; }
bool pdl_enabled()
{
   static const bool v = [] { const char *e = getenv("SOFIE_CUDA_PDL"); return !e || atoi(e) != 0; }();
   return v;
}
int forced_engine() { return g_forced_engine; }

// Streams of contexts report into their context's word; every other stream into one word per device,
// allocated on first use with that device current.
static std::mutex g_status_mutex;
static uint32_t *g_status_words[64] = {nullptr};
static std::vector<std::pair<cudaStream_t, uint32_t *>> g_stream_status;

void register_stream_status(cudaStream_t stream, uint32_t *word)
{
   std::lock_guard<std::mutex> lock(g_status_mutex);
   g_stream_status.emplace_back(stream, word);
}

void unregister_stream_status(cudaStream_t stream)
{
   std::lock_guard<std::mutex> lock(g_status_mutex);
   for (size_t i = 0; i < g_stream_status.size(); i++)
      if (g_stream_status[i].first == stream) {
         g_stream_status.erase(g_stream_status.begin() + i);
         return;
      }
}

uint32_t *device_status_word(cudaStream_t stream)
{
   int dev = 0;
   std::lock_guard<std::mutex> lock(g_status_mutex);
   for (auto &e : g_stream_status)
      if (e.first == stream) return e.second;
   if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
   if (!g_status_words[dev]) {
      uint32_t *p = nullptr;
      if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
      if (cudaMemset(p, 0, 256) != cudaSuccess) return nullptr;
      g_status_words[dev] = p;
   }
   return g_status_words[dev];
}

// Copies between pageable host memory and the pinned staging slots with several threads: one core copies about 12 GB/s,
// a fifth of what the PCIe link takes. The caller and the helper threads each copy an equal, page-aligned piece of a
// chunk; copy() returns when all pieces are done. SOFIE_CUDA_COPY_THREADS sets the number of threads (default 4, 1 = the
// caller alone). A helper spins for a fraction of a millisecond after a chunk (the next chunk of the same transfer comes
// within that time, and waking a sleeping thread costs as much as its piece of the copy), then sleeps on a condition
// variable; chunks below 4 MB are copied by the caller alone. The helpers end with the context.
class HostCopyPool {
public:
   explicit HostCopyPool(int helpers) : jobs_(helpers > 0 ? helpers : 0)
   {
      for (int i = 0; i < (int)jobs_.size(); i++) threads_.emplace_back([this, i] { work(i); });
   }
   ~HostCopyPool()
   {
      {
         std::lock_guard<std::mutex> lock(mu_);
         stop_.store(true);
      }
      wake_.notify_all();
      for (auto &t : threads_) t.join();
   }
   HostCopyPool(const HostCopyPool &) = delete;
   HostCopyPool &operator=(const HostCopyPool &) = delete;

   void copy(void *dst, const void *src, size_t bytes)
   {
      const size_t parts = jobs_.size() + 1;
      if (parts == 1 || bytes < (size_t(4) << 20)) {
         std::memcpy(dst, src, bytes);
         return;
      }
      const size_t piece = (((bytes + parts - 1) / parts) + 4095) & ~size_t(4095); // parts x piece >= bytes
      const size_t mine = piece < bytes ? piece : bytes; // the caller takes the first piece
      size_t off = mine;
      for (auto &j : jobs_) {
         const size_t n = off >= bytes ? 0 : (bytes - off < piece ? bytes - off : piece);
         j = {static_cast<char *>(dst) + off, static_cast<const char *>(src) + off, n};
         off += n;
      }
      pending_.store((int)jobs_.size(), std::memory_order_relaxed);
      generation_.fetch_add(1, std::memory_order_release); // publishes the jobs to the helpers that are still spinning
      {
         std::lock_guard<std::mutex> lock(mu_);           // ... and to the sleeping ones: no wake-up is lost
      }
      wake_.notify_all();
      std::memcpy(dst, src, mine);
      // the helpers' pieces are as long as the caller's: they finish at about the same time
      while (pending_.load(std::memory_order_acquire) != 0) std::this_thread::yield();
   }

private:
   struct Job {
      char *dst;
      const char *src;
      size_t bytes;
   };
   void work(int index)
   {
      unsigned long long seen = 0;
      for (;;) {
         const auto t0 = std::chrono::steady_clock::now();
         while (generation_.load(std::memory_order_acquire) == seen && !stop_.load(std::memory_order_relaxed)) {
            if (std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(500)) {
               std::unique_lock<std::mutex> lock(mu_);
               wake_.wait(lock, [&] { return stop_.load() || generation_.load(std::memory_order_acquire) != seen; });
               break;
            }
            std::this_thread::yield();
         }
         if (stop_.load()) return;
         seen = generation_.load(std::memory_order_acquire);
         const Job job = jobs_[index];
         if (job.bytes) std::memcpy(job.dst, job.src, job.bytes);
         pending_.fetch_sub(1, std::memory_order_release);
      }
   }
   std::vector<Job> jobs_;
   std::vector<std::thread> threads_;
   std::mutex mu_;
   std::condition_variable wake_;
   std::atomic<unsigned long long> generation_{0};
   std::atomic<int> pending_{0};
   std::atomic<bool> stop_{false};
};

} // namespace sofie

struct sofie_cuda_ctx {
   int device = 0;
   cudaStream_t stream = nullptr;
   char *arena = nullptr;
   size_t arena_bytes = 0;
   std::vector<void *> owned;
   void *staging = nullptr; // pinned: kStagingSlots slots of kStagingSlot bytes, used as a ring
   size_t staging_bytes = 0;
   cudaEvent_t staging_event[4] = {}; // the copy out of (h2d) or into (d2h) a slot has completed
   bool staging_busy[4] = {};         // a copy that read the slot may still be in flight
   std::unique_ptr<sofie::HostCopyPool> copy_pool; // made with the staging ring
   void *result = nullptr;  // pinned, grown on demand: where sofie_cuda_ctx_fetch lands device results
   size_t result_bytes = 0;
   cudaGraph_t graph = nullptr;
   cudaGraphExec_t graph_exec = nullptr;
   bool capturing = false;
   // small results written by the last kernel straight into mapped pinned host memory (no device-to-host copy)
   std::vector<std::pair<char *, size_t>> host_outputs;
   // pipelined input upload: parts of the input are copied on a stream of their own, one event per part
   cudaStream_t copy_stream = nullptr;
   cudaEvent_t part_event[SOFIE_CUDA_MAX_PARTS] = {};
   // status word of this context's kernels (mapped pinned host memory, 256 bytes)
   uint32_t *status = nullptr;
   // per-operator device timers (off unless SOFIE_CUDA_TIMERS is set or sofie_cuda_ctx_timers says so)
   bool timers_on = false;
   std::vector<cudaEvent_t> marks;
   std::vector<char> mark_seen;
};

using namespace sofie;

// The context's status word, read after the stream has been synchronised: a plain host load.
static int report_status(sofie_cuda_ctx *ctx)
{
   volatile uint32_t *w = ctx->status;
   if (w && w[0]) {
      const uint32_t code = w[0], d1 = w[1], d2 = w[2], d3 = w[3];
      w[1] = w[2] = w[3] = 0;
      w[0] = 0;
      return fail(SOFIE_CUDA_ERR_DEVICE, "device status 0x%x (detail 0x%x 0x%x 0x%x)", code, d1, d2, d3);
   }
   return SOFIE_CUDA_OK;
}


namespace {
struct DeviceGuard {
   int prev = -1;
   explicit DeviceGuard(int dev)
   {
      cudaGetDevice(&prev);
      if (prev != dev) cudaSetDevice(dev);
      else prev = -1;
   }
   ~DeviceGuard()
   {
      if (prev >= 0) cudaSetDevice(prev);
   }
};
// Pageable host memory crosses PCIe through pinned staging slots: while the copy engine drains one slot the CPU fills
// the next, so the host memcpy and the DMA overlap instead of alternating.
constexpr int kStagingSlots = 4;
constexpr size_t kStagingSlot = size_t(8) << 20;
constexpr size_t kStagingBytes = kStagingSlots * kStagingSlot;
} // namespace

extern "C" {

const char *sofie_cuda_strerror(int status)
{
   switch (status) {
   case SOFIE_CUDA_OK: return "success";
   case SOFIE_CUDA_ERR_INVALID: return "invalid argument";
   case SOFIE_CUDA_ERR_UNSUPPORTED: return "unsupported configuration";
   case SOFIE_CUDA_ERR_CUDA: return "CUDA error";
   case SOFIE_CUDA_ERR_NOMEM: return "out of device memory or arena range";
   case SOFIE_CUDA_ERR_DEVICE: return "kernel reported a device-side failure";
   default: return "unknown status";
   }
}

const char *sofie_cuda_last_error(void) { return last_error_buffer(); }
int sofie_cuda_abi_version(void) { return SOFIE_CUDA_ABI_VERSION; }
int sofie_cuda_last_engine(void) { return g_last_engine; }

int sofie_cuda_set_engine(int engine)
{
   SOFIE_REQUIRE(engine >= 0 && engine <= 2, "engine must be 0, 1 or 2");
   g_forced_engine = engine;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_set_default_device(int device)
{
   g_default_device = device < 0 ? -1 : device;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_device_count(int *count)
{
   SOFIE_REQUIRE(count != nullptr, "count is NULL");
   *count = 0;
   cudaError_t err = cudaGetDeviceCount(count);
   if (err != cudaSuccess) {
      *count = 0;
      cudaGetLastError();
      return fail(SOFIE_CUDA_ERR_CUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(err));
   }
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_create(sofie_cuda_ctx **out, int device, size_t arena_bytes)
{
   SOFIE_REQUIRE(out != nullptr, "ctx output pointer is NULL");
   *out = nullptr;
   if (device < 0 && g_default_device >= 0) device = g_default_device;
   if (device < 0) {
      const char *env = std::getenv("SOFIE_CUDA_DEVICE");
      device = env ? std::atoi(env) : 0;
   }
   int count = 0;
   int rc = sofie_cuda_device_count(&count);
   if (rc) return rc;
   if (device >= count) return fail(SOFIE_CUDA_ERR_INVALID, "device %d requested, %d visible", device, count);
   DeviceGuard guard(device);
   auto *ctx = new sofie_cuda_ctx();
   ctx->device = device;
   cudaError_t err = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
   if (err == cudaSuccess && arena_bytes) {
      ctx->arena_bytes = (arena_bytes + 255) & ~size_t(255);
      err = cudaMalloc(&ctx->arena, ctx->arena_bytes);
   }
   if (err == cudaSuccess) {
      void *w = nullptr, *d = nullptr;
      err = cudaHostAlloc(&w, 256, cudaHostAllocMapped);
      if (err == cudaSuccess) {
         std::memset(w, 0, 256);
         err = cudaHostGetDevicePointer(&d, w, 0);
         if (err == cudaSuccess && d != w) err = cudaErrorNotSupported; // needs unified addressing
         ctx->status = static_cast<uint32_t *>(w);
      }
   }
   if (err != cudaSuccess) {
      if (ctx->status) cudaFreeHost(ctx->status);
      if (ctx->arena) cudaFree(ctx->arena);
      if (ctx->stream) cudaStreamDestroy(ctx->stream);
      delete ctx;
      cudaGetLastError();
      return fail(err == cudaErrorMemoryAllocation ? SOFIE_CUDA_ERR_NOMEM : SOFIE_CUDA_ERR_CUDA,
                  "context creation on device %d (arena %zu bytes): %s", device, arena_bytes, cudaGetErrorString(err));
   }
   register_stream_status(ctx->stream, ctx->status);
   if (const char *t = std::getenv("SOFIE_CUDA_TIMERS")) ctx->timers_on = std::atoi(t) != 0;
   *out = ctx;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_destroy(sofie_cuda_ctx *ctx)
{
   if (!ctx) return SOFIE_CUDA_OK;
   DeviceGuard guard(ctx->device);
   // nothing of this context may still be running or copying when its memory goes away
   cudaStreamSynchronize(ctx->stream);
   if (ctx->copy_stream) cudaStreamSynchronize(ctx->copy_stream);
   unregister_stream_status(ctx->stream);
   if (ctx->graph_exec) cudaGraphExecDestroy(ctx->graph_exec);
   if (ctx->graph) cudaGraphDestroy(ctx->graph);
   for (void *p : ctx->owned) cudaFree(p);
   if (ctx->arena) cudaFree(ctx->arena);
   for (auto &h : ctx->host_outputs) cudaFreeHost(h.first);
   if (ctx->staging) cudaFreeHost(ctx->staging);
   if (ctx->result) cudaFreeHost(ctx->result);
   splitk_scratch_release(ctx->device, ctx->stream);
   if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
   if (ctx->status) cudaFreeHost(ctx->status);
   for (cudaEvent_t e : ctx->staging_event)
      if (e) cudaEventDestroy(e);
   for (cudaEvent_t e : ctx->marks)
      if (e) cudaEventDestroy(e);
   for (cudaEvent_t e : ctx->part_event)
      if (e) cudaEventDestroy(e);
   cudaStreamDestroy(ctx->stream);
   delete ctx;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_stream(sofie_cuda_ctx *ctx, void **stream)
{
   SOFIE_REQUIRE(ctx && stream, "NULL argument");
   *stream = ctx->stream;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_device(sofie_cuda_ctx *ctx, int *device)
{
   SOFIE_REQUIRE(ctx && device, "NULL argument");
   *device = ctx->device;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_arena(sofie_cuda_ctx *ctx, size_t offset, size_t bytes, void **dptr)
{
   SOFIE_REQUIRE(ctx && dptr, "NULL argument");
   SOFIE_REQUIRE((offset & 255) == 0, "arena offset %zu is not 256-byte aligned", offset);
   if (offset > ctx->arena_bytes || bytes > ctx->arena_bytes - offset)
      return fail(SOFIE_CUDA_ERR_NOMEM, "arena slice [%zu, +%zu) exceeds arena of %zu bytes", offset, bytes,
                  ctx->arena_bytes);
   *dptr = ctx->arena + offset;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_alloc(sofie_cuda_ctx *ctx, size_t bytes, void **dptr)
{
   SOFIE_REQUIRE(ctx && dptr, "NULL argument");
   DeviceGuard guard(ctx->device);
   void *p = nullptr;
   cudaError_t err = cudaMalloc(&p, bytes ? bytes : 256);
   if (err != cudaSuccess) {
      cudaGetLastError();
      return fail(SOFIE_CUDA_ERR_NOMEM, "cudaMalloc of %zu bytes: %s", bytes, cudaGetErrorString(err));
   }
   ctx->owned.push_back(p);
   *dptr = p;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_upload(sofie_cuda_ctx *ctx, const void *host, size_t bytes, void **dptr)
{
   SOFIE_REQUIRE(ctx && dptr && (host || bytes == 0), "NULL argument");
   int rc = sofie_cuda_ctx_alloc(ctx, bytes, dptr);
   if (rc) return rc;
   DeviceGuard guard(ctx->device);
   if (bytes) {
      SOFIE_CUDA_TRY(cudaMemcpyAsync(*dptr, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
      SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
   }
   return SOFIE_CUDA_OK;
}

static int ensure_staging(sofie_cuda_ctx *ctx)
{
   if (ctx->staging) return SOFIE_CUDA_OK;
   SOFIE_CUDA_TRY(cudaMallocHost(&ctx->staging, kStagingBytes));
   ctx->staging_bytes = kStagingBytes;
   for (auto &e : ctx->staging_event) SOFIE_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
   int threads = 4;
   if (const char *e = std::getenv("SOFIE_CUDA_COPY_THREADS")) threads = std::atoi(e);
   const int cores = (int)std::thread::hardware_concurrency();
   if (cores > 0 && threads > cores) threads = cores;
   if (threads < 1) threads = 1;
   if (threads > 16) threads = 16;
   ctx->copy_pool.reset(new HostCopyPool(threads - 1));
   return SOFIE_CUDA_OK;
}

// Pageable host memory is staged through one pinned buffer in chunks; memory the caller already
// pinned (cudaHostRegister / cudaMallocHost) is copied directly and stays asynchronous.
static bool is_pinned(const void *p)
{
   cudaPointerAttributes attr;
   if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
      cudaGetLastError();
      return false;
   }
   return attr.type == cudaMemoryTypeHost;
}

int sofie_cuda_ctx_h2d(sofie_cuda_ctx *ctx, void *dst, const void *src, size_t bytes)
{
   SOFIE_REQUIRE(ctx && dst && src, "NULL argument");
   SOFIE_REQUIRE(!ctx->capturing, "input copies are not part of the captured graph");
   DeviceGuard guard(ctx->device);
   if (is_pinned(src)) {
      SOFIE_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
      return SOFIE_CUDA_OK;
   }
   int rc = ensure_staging(ctx);
   if (rc) return rc;
   size_t done = 0;
   bool used[kStagingSlots] = {};
   for (int slot = 0; done < bytes; slot = (slot + 1) % kStagingSlots) {
      const size_t chunk = bytes - done < kStagingSlot ? bytes - done : kStagingSlot;
      char *stage = static_cast<char *>(ctx->staging) + (size_t)slot * kStagingSlot;
      // a slot is refilled only after the copy that last read it has finished (also a copy of an earlier call)
      if (used[slot] || ctx->staging_busy[slot]) SOFIE_CUDA_TRY(cudaEventSynchronize(ctx->staging_event[slot]));
      ctx->copy_pool->copy(stage, static_cast<const char *>(src) + done, chunk);
      SOFIE_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(dst) + done, stage, chunk, cudaMemcpyHostToDevice, ctx->stream));
      SOFIE_CUDA_TRY(cudaEventRecord(ctx->staging_event[slot], ctx->stream));
      used[slot] = ctx->staging_busy[slot] = true;
      done += chunk;
   }
   return SOFIE_CUDA_OK;
}

int sofie_cuda_selftest_host_copy(void *dst, const void *src, size_t bytes, size_t chunk, int threads, int repeats)
{
   SOFIE_REQUIRE((dst && src) || bytes == 0, "NULL buffer");
   SOFIE_REQUIRE(chunk > 0 && threads >= 1 && threads <= 16 && repeats >= 1, "bad chunk size, thread count or repeat count");
   HostCopyPool pool(threads - 1);
   for (int r = 0; r < repeats; r++)
      for (size_t done = 0; done < bytes; done += chunk)
         pool.copy(static_cast<char *>(dst) + done, static_cast<const char *>(src) + done, bytes - done < chunk ? bytes - done : chunk);
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_h2d_part(sofie_cuda_ctx *ctx, void *dst, const void *src, size_t bytes, int part)
{
   SOFIE_REQUIRE(ctx && dst && src, "NULL argument");
   SOFIE_REQUIRE(part >= 0 && part < SOFIE_CUDA_MAX_PARTS, "part index out of range");
   SOFIE_REQUIRE(!ctx->capturing, "input copies are not part of the captured graph");
   DeviceGuard guard(ctx->device);
   if (!ctx->part_event[part]) SOFIE_CUDA_TRY(cudaEventCreateWithFlags(&ctx->part_event[part], cudaEventDisableTiming));
   if (!is_pinned(src)) {
      // pageable memory goes through the staging ring on the compute stream; the call returns when the part has been
      // staged, so the kernels the caller launches next for this part run while the host stages the following one.
      // The event only keeps sofie_cuda_ctx_wait_part valid
      int rc = sofie_cuda_ctx_h2d(ctx, dst, src, bytes);
      if (rc) return rc;
      SOFIE_CUDA_TRY(cudaEventRecord(ctx->part_event[part], ctx->stream));
      return SOFIE_CUDA_OK;
   }
   if (!ctx->copy_stream) SOFIE_CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
   SOFIE_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
   SOFIE_CUDA_TRY(cudaEventRecord(ctx->part_event[part], ctx->copy_stream));
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_wait_part(sofie_cuda_ctx *ctx, int part)
{
   SOFIE_REQUIRE(ctx != nullptr, "NULL context");
   SOFIE_REQUIRE(part >= 0 && part < SOFIE_CUDA_MAX_PARTS && ctx->part_event[part], "no copy was issued for this part");
   SOFIE_REQUIRE(!ctx->capturing, "input copies are not part of the captured graph");
   DeviceGuard guard(ctx->device);
   SOFIE_CUDA_TRY(cudaStreamWaitEvent(ctx->stream, ctx->part_event[part], 0));
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_d2h(sofie_cuda_ctx *ctx, void *dst, const void *src, size_t bytes)
{
   SOFIE_REQUIRE(ctx && dst && src, "NULL argument");
   SOFIE_REQUIRE(!ctx->capturing, "result copies are not part of the captured graph");
   DeviceGuard guard(ctx->device);
   if (is_pinned(dst)) {
      SOFIE_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
      SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
      return SOFIE_CUDA_OK;
   }
   int rc = ensure_staging(ctx);
   if (rc) return rc;
   // every input copy that used the slots has to be over before results land in them
   SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
   for (auto &b : ctx->staging_busy) b = false;
   // the copies of all slots are queued first, then each is copied out as soon as it has arrived: the host memcpy of
   // one slot overlaps the DMA into the next
   size_t done = 0;
   while (done < bytes) {
      const size_t round = bytes - done < kStagingBytes ? bytes - done : kStagingBytes;
      int slots = 0;
      for (size_t off = 0; off < round; off += kStagingSlot, slots++) {
         const size_t chunk = round - off < kStagingSlot ? round - off : kStagingSlot;
         SOFIE_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(ctx->staging) + off, static_cast<const char *>(src) + done + off, chunk,
                                        cudaMemcpyDeviceToHost, ctx->stream));
         SOFIE_CUDA_TRY(cudaEventRecord(ctx->staging_event[slots], ctx->stream));
      }
      for (int slot = 0; slot < slots; slot++) {
         const size_t off = (size_t)slot * kStagingSlot, chunk = round - off < kStagingSlot ? round - off : kStagingSlot;
         SOFIE_CUDA_TRY(cudaEventSynchronize(ctx->staging_event[slot]));
         ctx->copy_pool->copy(static_cast<char *>(dst) + done + off, static_cast<char *>(ctx->staging) + off, chunk);
      }
      done += round;
   }
   return SOFIE_CUDA_OK;
}

// Device -> pinned host buffer owned by the context, at full link speed; the caller builds its
// result (the vector Session::infer returns) from the returned pointer in one pass, instead of
// zero-filling a vector first and then staging the copy through it. The pointer stays valid until
// the next fetch on this context.
int sofie_cuda_ctx_host_output(sofie_cuda_ctx *ctx, size_t bytes, void **dptr)
{
   SOFIE_REQUIRE(ctx && dptr, "NULL argument");
   SOFIE_REQUIRE(bytes > 0, "empty output");
   DeviceGuard guard(ctx->device);
   void *p = nullptr, *d = nullptr;
   SOFIE_CUDA_TRY(cudaHostAlloc(&p, bytes, cudaHostAllocMapped));
   cudaError_t err = cudaHostGetDevicePointer(&d, p, 0);
   if (err != cudaSuccess || d != p) { // without unified addressing the two views differ: not supported here
      cudaFreeHost(p);
      cudaGetLastError();
      return fail(SOFIE_CUDA_ERR_CUDA, "mapped host memory is not addressable by the device at its host address");
   }
   std::memset(p, 0, bytes);
   ctx->host_outputs.emplace_back(static_cast<char *>(p), bytes);
   *dptr = d;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_fetch(sofie_cuda_ctx *ctx, const void *src, size_t bytes, void **host)
{
   SOFIE_REQUIRE(ctx && src && host, "NULL argument");
   SOFIE_REQUIRE(!ctx->capturing, "result copies are not part of the captured graph");
   DeviceGuard guard(ctx->device);
   for (auto &h : ctx->host_outputs) {
      const char *s8 = static_cast<const char *>(src);
      if (s8 >= h.first && s8 + bytes <= h.first + h.second) {
         // the kernels wrote the result into host memory themselves: wait for them, nothing to copy
         SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
         *host = const_cast<char *>(s8);
         return report_status(ctx);
      }
   }
   if (bytes > ctx->result_bytes) {
      if (ctx->result) cudaFreeHost(ctx->result);
      ctx->result = nullptr;
      ctx->result_bytes = 0;
      SOFIE_CUDA_TRY(cudaMallocHost(&ctx->result, bytes));
      ctx->result_bytes = bytes;
   }
   if (bytes) SOFIE_CUDA_TRY(cudaMemcpyAsync(ctx->result, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
   SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
   *host = ctx->result;
   return report_status(ctx);
}

int sofie_cuda_ctx_sync(sofie_cuda_ctx *ctx)
{
   SOFIE_REQUIRE(ctx, "NULL ctx");
   DeviceGuard guard(ctx->device);
   SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_check(sofie_cuda_ctx *ctx)
{
   SOFIE_REQUIRE(ctx, "NULL ctx");
   SOFIE_REQUIRE(!ctx->capturing, "the stream cannot be synchronised during a graph capture");
   DeviceGuard guard(ctx->device);
   SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
   return report_status(ctx);
}

int sofie_cuda_device_check(int device)
{
   SOFIE_REQUIRE(device >= 0 && device < 64, "device index out of range");
   uint32_t *word = nullptr;
   {
      std::lock_guard<std::mutex> lock(g_status_mutex);
      word = g_status_words[device];
   }
   if (!word) return SOFIE_CUDA_OK; // no kernel with a bounded wait ran outside a context on this device
   DeviceGuard guard(device);
   uint32_t host_word[4] = {0, 0, 0, 0};
   SOFIE_CUDA_TRY(cudaDeviceSynchronize());
   SOFIE_CUDA_TRY(cudaMemcpy(host_word, word, sizeof(host_word), cudaMemcpyDeviceToHost));
   if (host_word[0]) {
      SOFIE_CUDA_TRY(cudaMemset(word, 0, 256));
      return fail(SOFIE_CUDA_ERR_DEVICE, "device status 0x%x (detail 0x%x 0x%x 0x%x)", host_word[0], host_word[1],
                  host_word[2], host_word[3]);
   }
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_timers(sofie_cuda_ctx *ctx, int on)
{
   SOFIE_REQUIRE(ctx, "NULL ctx");
   SOFIE_REQUIRE(!ctx->capturing && !ctx->graph_exec, "switch the timers before the first inference is captured");
   ctx->timers_on = on != 0;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_mark(sofie_cuda_ctx *ctx, int slot)
{
   SOFIE_REQUIRE(ctx, "NULL ctx");
   if (!ctx->timers_on) return SOFIE_CUDA_OK;
   SOFIE_REQUIRE(slot >= 0 && slot < 4096, "timer slot out of range");
   DeviceGuard guard(ctx->device);
   if ((size_t)slot >= ctx->marks.size()) {
      ctx->marks.resize(slot + 1, nullptr);
      ctx->mark_seen.resize(slot + 1, 0);
   }
   if (!ctx->marks[slot]) SOFIE_CUDA_TRY(cudaEventCreate(&ctx->marks[slot]));
   // inside a capture the record becomes a node of the graph that updates this very event on every replay
   SOFIE_CUDA_TRY(cudaEventRecordWithFlags(ctx->marks[slot], ctx->stream, ctx->capturing ? cudaEventRecordExternal : cudaEventRecordDefault));
   ctx->mark_seen[slot] = 1;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_timers_read(sofie_cuda_ctx *ctx, float *ms, int n, int *count)
{
   SOFIE_REQUIRE(ctx && count, "NULL argument");
   SOFIE_REQUIRE(!ctx->capturing, "the stream cannot be synchronised during a graph capture");
   DeviceGuard guard(ctx->device);
   SOFIE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
   // intervals between consecutive recorded marks, in slot order
   int prev = -1, k = 0;
   for (int i = 0; i < (int)ctx->marks.size(); i++) {
      if (!ctx->mark_seen[i]) continue;
      if (prev >= 0) {
         if (ms && k < n) SOFIE_CUDA_TRY(cudaEventElapsedTime(&ms[k], ctx->marks[prev], ctx->marks[i]));
         k++;
      }
      prev = i;
   }
   *count = k;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_graph_begin(sofie_cuda_ctx *ctx)
{
   SOFIE_REQUIRE(ctx, "NULL ctx");
   SOFIE_REQUIRE(!ctx->capturing, "graph capture already in progress");
   DeviceGuard guard(ctx->device);
   if (ctx->graph_exec) {
      cudaGraphExecDestroy(ctx->graph_exec);
      ctx->graph_exec = nullptr;
   }
   if (ctx->graph) {
      cudaGraphDestroy(ctx->graph);
      ctx->graph = nullptr;
   }
   SOFIE_CUDA_TRY(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
   ctx->capturing = true;
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_graph_end(sofie_cuda_ctx *ctx)
{
   SOFIE_REQUIRE(ctx, "NULL ctx");
   SOFIE_REQUIRE(ctx->capturing, "no graph capture in progress");
   DeviceGuard guard(ctx->device);
   ctx->capturing = false;
   SOFIE_CUDA_TRY(cudaStreamEndCapture(ctx->stream, &ctx->graph));
   SOFIE_CUDA_TRY(cudaGraphInstantiate(&ctx->graph_exec, ctx->graph, 0));
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_graph_launch(sofie_cuda_ctx *ctx)
{
   SOFIE_REQUIRE(ctx, "NULL ctx");
   SOFIE_REQUIRE(ctx->graph_exec != nullptr, "no captured graph");
   DeviceGuard guard(ctx->device);
   SOFIE_CUDA_TRY(cudaGraphLaunch(ctx->graph_exec, ctx->stream));
   return SOFIE_CUDA_OK;
}

int sofie_cuda_ctx_graph_ready(sofie_cuda_ctx *ctx, int *ready)
{
   SOFIE_REQUIRE(ctx && ready, "NULL argument");
   *ready = ctx->graph_exec != nullptr;
   return SOFIE_CUDA_OK;
}

} // extern "C"
