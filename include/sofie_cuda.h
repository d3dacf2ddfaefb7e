/*
 * sofie_cuda.h -- C ABI of libSOFIE_cuda, the sm_100a (B200) back end of SOFIE's dense-contraction
 * inference path.
 *
 * This header is what the code emitted by RModel::Generate() includes in place of the block of
 * Fortran BLAS prototypes the reference writes into every generated header
 * (reference: src/SOFIE_core/src/RModel_Base.cxx:40-58). It is plain C: no CUDA types, no C++
 * types, pointers and sizes only. Every function returns an int status (0 = success); nothing
 * throws across this boundary. The emitted Session turns a non-zero status into
 * std::runtime_error, which is the reference's own error convention
 * (reference: src/SOFIE_core/src/RModel.cxx:975-1013).
 *
 * Conventions
 *   - "device pointer" = address in the memory of the GPU the call runs on. Host pointers are
 *     marked "host".
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream). All compute
 *     entry points only enqueue work; they do not synchronise.
 *   - Tensors are dense and row-major. Activations of convolutions are NCHW (the reference's only
 *     layout) or NHWC (the layout the tensor-core path keeps between fused layers); the descriptor
 *     says which.
 *   - There is no CPU fallback: without a usable GPU every compute entry point fails.
 */
#ifndef SOFIE_CUDA_H
#define SOFIE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status ------------------ */
#define SOFIE_CUDA_OK 0
#define SOFIE_CUDA_ERR_INVALID 1     /* bad argument, shape or alignment                          */
#define SOFIE_CUDA_ERR_UNSUPPORTED 2 /* valid request this build has no kernel for                */
#define SOFIE_CUDA_ERR_CUDA 3        /* the CUDA runtime / driver reported an error               */
#define SOFIE_CUDA_ERR_NOMEM 4       /* arena slice out of range or allocation failure            */
#define SOFIE_CUDA_ERR_DEVICE 5      /* a kernel set its status word (a bounded wait ran out)     */

/* Short text for a status code. Never NULL. */
const char *sofie_cuda_strerror(int status);
/* Detail of the last failure on the calling thread ("" if none). Never NULL. */
const char *sofie_cuda_last_error(void);
/* ABI version of the loaded library (SOFIE_CUDA_ABI_VERSION of the build). */
#define SOFIE_CUDA_ABI_VERSION 1
int sofie_cuda_abi_version(void);
/* Number of visible CUDA devices (0 and SOFIE_CUDA_ERR_CUDA when there is no driver). */
int sofie_cuda_device_count(int *count);

/* ------------------------------------------------------------------ context ----------------- */
/*
 * One context per emitted Session and GPU. It replaces the Session members the reference emits:
 * the per-weight std::vector<float> (reference: src/SOFIE_core/src/RModel.cxx:574-595) and the
 * `new char[]` intermediate pool (reference: src/SOFIE_core/src/RModel.cxx:597-604), which the
 * reference never frees. The context owns one stream, one device arena allocated once, the
 * uploaded weights, a pinned staging buffer and, optionally, one captured CUDA graph of infer().
 */
typedef struct sofie_cuda_ctx sofie_cuda_ctx;

/* device < 0: the calling thread's default device when one is set (sofie_cuda_set_default_device), else the
 * environment variable SOFIE_CUDA_DEVICE, else device 0. */
int sofie_cuda_ctx_create(sofie_cuda_ctx **ctx, int device, size_t arena_bytes);
/* Device of the contexts this THREAD creates with device < 0 -- which is how an emitted Session, whose constructor has no
 * device argument (the reference's has none: src/SOFIE_core/src/RModel.cxx:876-884), is placed on a chosen GPU; a
 * negative value returns to the environment variable. One Session per GPU, each constructed after this call, is the
 * reference's one-Session-per-slot idiom (SOFIEHelpers.hxx:23-49) applied to devices. */
int sofie_cuda_set_default_device(int device);
int sofie_cuda_ctx_destroy(sofie_cuda_ctx *ctx);
int sofie_cuda_ctx_stream(sofie_cuda_ctx *ctx, void **stream);
int sofie_cuda_ctx_device(sofie_cuda_ctx *ctx, int *device);
/* Bounds-checked pointer to arena bytes [offset, offset+bytes). Offsets are 256-byte aligned. */
int sofie_cuda_ctx_arena(sofie_cuda_ctx *ctx, size_t offset, size_t bytes, void **dptr);
/* Persistent device allocation owned by the context (weights, packed weights, scale tables). */
int sofie_cuda_ctx_alloc(sofie_cuda_ctx *ctx, size_t bytes, void **dptr);
/* Allocate and fill from host memory; replaces the text-file weight read into fTensor_* vectors
 * (reference: src/SOFIE_core/src/RModel.cxx:970-1018 reads, this uploads what was read). */
int sofie_cuda_ctx_upload(sofie_cuda_ctx *ctx, const void *host, size_t bytes, void **dptr);
/* Host -> device through the context's pinned staging buffer, asynchronous on the context stream
 * (first statement of the emitted infer()). */
int sofie_cuda_ctx_h2d(sofie_cuda_ctx *ctx, void *dst_device, const void *src_host, size_t bytes);
/* Pipelined input upload: the input is copied in up to SOFIE_CUDA_MAX_PARTS parts (slices of the batch) on a
 * copy stream of the context, and the launches that read part p are issued after sofie_cuda_ctx_wait_part(p),
 * which makes the context stream wait for that copy only: the model's leading operators work on part p while
 * part p+1 is still crossing PCIe. Copies from pageable host memory fall back to sofie_cuda_ctx_h2d. The
 * caller must not issue the parts of a new inference before the previous one has been fetched
 * (the emitted infer() ends with sofie_cuda_ctx_fetch, which waits). */
#define SOFIE_CUDA_MAX_PARTS 8
int sofie_cuda_ctx_h2d_part(sofie_cuda_ctx *ctx, void *dst_device, const void *src_host, size_t bytes, int part);
int sofie_cuda_ctx_wait_part(sofie_cuda_ctx *ctx, int part);
/* Device -> host; returns after the data has arrived (last statement of the emitted infer(),
 * replaces `return std::vector<float>(tensor_y, tensor_y + n)`,
 * reference: src/SOFIE_core/src/RModel.cxx:717-740). */
int sofie_cuda_ctx_d2h(sofie_cuda_ctx *ctx, void *dst_host, const void *src_device, size_t bytes);
/* Copies a device result into a pinned host buffer owned by the context (grown on demand) and
 * returns its address; valid until the next fetch. The emitted infer() builds the vector it
 * returns (RModel.cxx:744-801 in the reference) from it in one pass. */
int sofie_cuda_ctx_fetch(sofie_cuda_ctx *ctx, const void *src_device, size_t bytes, void **host);
/* A small result tensor placed in mapped pinned host memory: the kernel that computes it writes across PCIe
 * itself and sofie_cuda_ctx_fetch of that pointer only waits for the stream (no device-to-host copy, which
 * costs more than the few kilobytes of a classifier's output are worth). Meant for tensors that no kernel
 * reads; the memory is zero-initialised and owned by the context. */
int sofie_cuda_ctx_host_output(sofie_cuda_ctx *ctx, size_t bytes, void **dptr);
int sofie_cuda_ctx_sync(sofie_cuda_ctx *ctx);
/* Waits for the context's stream, then reads and clears the context's status word, which a kernel whose
 * bounded wait ran out has set (SOFIE_CUDA_ERR_DEVICE; the kernel itself ended normally and the context
 * stays usable). The word lies in mapped pinned host memory and belongs to this context alone.
 * sofie_cuda_ctx_fetch performs the same check after its own wait, so the emitted infer() never returns
 * the output of a kernel that gave up (the reference has no counterpart: CPU code cannot time out). */
int sofie_cuda_ctx_check(sofie_cuda_ctx *ctx);
/* The same for launches made on streams that belong to no context (direct callers of the compute entry
 * points): one word per device. Synchronises the whole device. */
int sofie_cuda_device_check(int device);
/* Self test of the bounded waits (no counterpart in the reference): launches one CTA that allocates
 * tensor memory and waits on a barrier nothing arrives on, with a limit of `limit_cycles` SM clocks
 * (at most 2e8, about 0.1 s) instead of the library's one second. The kernel gives up, records status
 * 0x1ff with detail 0x7e57 in the status word of the stream's context, releases its tensor memory and,
 * when `reached_exit_device` is not NULL, stores 1 there as its last action. Nothing faults or hangs;
 * the following sofie_cuda_ctx_check / sofie_cuda_ctx_fetch reports SOFIE_CUDA_ERR_DEVICE once. */
int sofie_cuda_selftest_wait_timeout(void *stream, int64_t limit_cycles, uint32_t *reached_exit_device);
/* Self test of the threaded host copy that carries pageable inputs into the pinned staging ring (no
 * counterpart in the reference; needs no GPU): copies `bytes` bytes from src to dst `repeats` times in
 * chunks of `chunk` bytes with `threads` threads (the caller and threads - 1 helpers), exactly as
 * sofie_cuda_ctx_h2d does per staging slot. Returns SOFIE_CUDA_OK, or SOFIE_CUDA_ERR_INVALID for bad arguments. */
int sofie_cuda_selftest_host_copy(void *dst, const void *src, size_t bytes, size_t chunk, int threads, int repeats);
/* Per-operator device timers (no counterpart in the reference, whose only timing is the caller's clock).
 * The emitted Launch() calls sofie_cuda_ctx_mark(ctx, i) before operator i and once more after the last
 * one. With the timers off (the default) a mark does nothing; with them on -- the environment variable
 * SOFIE_CUDA_TIMERS=1 when the context is created, or sofie_cuda_ctx_timers(ctx, 1) before the first
 * inference -- every mark records a CUDA event on the context stream (as a node of the captured graph when
 * a capture is running) and sofie_cuda_ctx_timers_read returns, after waiting for the stream, the
 * milliseconds between consecutive marks of the last inference: one number per operator, in Launch() order.
 * ms may be NULL to ask for the count only; *count is the number of intervals available. The event nodes
 * serialise the kernels around them (no overlap of one kernel's prologue with the previous kernel's tail),
 * so a timed Session is a little slower than an untimed one: use it to see where a step's time goes. */
int sofie_cuda_ctx_timers(sofie_cuda_ctx *ctx, int on);
int sofie_cuda_ctx_mark(sofie_cuda_ctx *ctx, int slot);
int sofie_cuda_ctx_timers_read(sofie_cuda_ctx *ctx, float *ms, int n, int *count);
/* Capture of the kernel sequence of one infer() into a CUDA graph: begin, run the launchers on
 * the context stream, end; then launch replays it. */
int sofie_cuda_ctx_graph_begin(sofie_cuda_ctx *ctx);
int sofie_cuda_ctx_graph_end(sofie_cuda_ctx *ctx);
int sofie_cuda_ctx_graph_launch(sofie_cuda_ctx *ctx);
int sofie_cuda_ctx_graph_ready(sofie_cuda_ctx *ctx, int *ready);

/* ------------------------------------------------------------------ fp32 contractions ------- */
#define SOFIE_LAYOUT_NCHW 0
#define SOFIE_LAYOUT_NHWC 1

/* Which kernel family served the last call of a contraction entry point on this thread:
 * 0 = none yet, 1 = CUDA-core kernel, 2 = tcgen05 tensor-core kernel. For tests and logs. */
#define SOFIE_ENGINE_NONE 0
#define SOFIE_ENGINE_SIMT 1
#define SOFIE_ENGINE_TCGEN05 2
int sofie_cuda_last_engine(void);
/* Force the kernel family for later calls on every thread: 0 = automatic (default),
 * 1 = CUDA cores only, 2 = tcgen05 only (calls with no tcgen05 kernel then fail UNSUPPORTED). */
int sofie_cuda_set_engine(int engine);

/*
 * Y[M,N] = alpha * op(A) * op(B) + beta * broadcast(C), optional Relu. ONNX Gemm / MatMul.
 * Replaces the text emitted by ROperator_Gemm<float>::Generate
 * (reference: src/SOFIE_core/inc/SOFIE/ROperator_Gemm.hxx:292-390): std::copy of the pre-broadcast
 * bias into Y, BLAS::sgemm_, and the separate Relu loop. fp32 in, fp32 out; the tensor-core path
 * evaluates the product as 3 TF32 products of a hi/lo split with fp32 accumulation.
 */
typedef struct sofie_gemm_f32_desc {
   int32_t M, N, K;
   int32_t transA;    /* 0: A is [M,K]; 1: A is [K,M]                                    */
   int32_t transB;    /* 0: B is [K,N]; 1: B is [N,K] (what PyTorch's Linear exports)     */
   float alpha, beta;
   int32_t bias_kind; /* 0: no C (beta ignored); 1: C is [N], broadcast over rows; 2: C is [M,N] */
   int32_t relu;      /* 1: y = y > 0 ? y : 0                                             */
} sofie_gemm_f32_desc;
int sofie_cuda_gemm_f32(void *stream, const sofie_gemm_f32_desc *desc, const float *A, const float *B,
                        const float *C, float *Y);

/*
 * A stack of `batch` independent products with the same descriptor: matrix b of A, B and Y starts b * strideA,
 * b * strideB, b * strideY elements after the first (strideA or strideB = 0: that operand is shared by the whole stack);
 * C, when given, is a per-column bias (bias_kind 1) shared by all. ONNX MatMul of operands with leading "stack"
 * dimensions and Einsum equations of the form "...ik,...kj->...ij". The reference emits one sgemm_ per stack index
 * for both (ROperator_Gemm.hxx:353-387 -- where only the output offset advances, so every index multiplies the first
 * matrices again --, ROperator_Einsum.hxx:275-332); here every index has its own operands, as ONNX defines, and each
 * product takes the same kernels as sofie_cuda_gemm_f32.
 */
int sofie_cuda_gemm_f32_batched(void *stream, const sofie_gemm_f32_desc *desc, const float *A, const float *B, const float *C,
                                float *Y, int32_t batch, int64_t strideA, int64_t strideB, int64_t strideY);

/*
 * Allocation-free skinny GEMM (no counterpart in the reference).
 *
 * Same arithmetic and descriptor as sofie_cuda_gemm_f32, restricted to the split-K shape class
 * (A not transposed, N <= 16, K >= 1024) and to M*N <= SOFIE_CUDA_SPLITK_STATIC_MAX_OUTPUTS. It is
 * meant for callers that must not trigger a device allocation: a serving loop that has handed all
 * free device memory to its own pool, code that runs while another thread captures a CUDA graph
 * in global capture mode (where cudaMalloc is an error), or latency-critical callers for whom the
 * implicit device synchronisation of cudaMalloc / cudaFree is unacceptable. The regular entry point
 * obtains its per-slab partial sums buffer from the CUDA allocator the first time a stream uses
 * it; this one keeps that buffer in a fixed 4 MiB array inside the library image (every GPU that
 * loads libSOFIE_cuda holds those 4 MiB until the process exits) and never calls cudaMalloc,
 * cudaFree or any allocating routine.
 *   - The first call on each device looks up the array's address on that device; make that first
 *     call before starting a stream capture.
 *   - All calls on a device share the one array. Nothing in it has to start at zero (every partial
 *     sum is rewritten before it is read), but two calls that overlap on the GPU -- different
 *     streams, or graphs replayed concurrently -- race on it and corrupt each other's results.
 *   - Shapes outside the class return SOFIE_CUDA_ERR_UNSUPPORTED; more than
 *     SOFIE_CUDA_SPLITK_STATIC_MAX_OUTPUTS outputs return SOFIE_CUDA_ERR_INVALID.
 */
#define SOFIE_CUDA_SPLITK_STATIC_FLOATS (1u << 20)
#define SOFIE_CUDA_SPLITK_STATIC_MAX_OUTPUTS 16384
int sofie_cuda_gemm_f32_splitk_static(void *stream, const sofie_gemm_f32_desc *desc, const float *A, const float *B,
                                      const float *C, float *Y);

/* out[cols,rows] = in[rows,cols]^T, used once per Session to bring a [K,N] weight to [N,K]. */
int sofie_cuda_transpose_f32(void *stream, const float *in, float *out, int32_t rows, int32_t cols);

/*
 * 2-D convolution (cross-correlation) + per-channel bias, optional Relu, optional fused
 * MaxPool 2x2 stride 2. Replaces the text emitted by ROperator_Conv<float>::Generate
 * (reference: src/SOFIE_core/inc/SOFIE/ROperator_Conv.hxx:302-522: weight repack, per-image
 * UTILITY::Im2col (reference: src/SOFIE_core/inc/SOFIE/SOFIE_common.hxx:485-518), sgemm_, saxpy_)
 * and, when relu/pool are set, the following ROperator_Relu and ROperator_Pool sweeps
 * (reference: ROperator_Relu.hxx:54-66, ROperator_Pool.hxx:371-416). No im2col buffer exists.
 * Pads are symmetric as in the reference (ROperator_Conv.hxx:387-410 averages asymmetric pads).
 */
typedef struct sofie_conv2d_desc {
   int32_t N, C, H, W;     /* input  [N,C,H,W]                                            */
   int32_t Cout, kH, kW;   /* weight [Cout, C/group, kH, kW]                              */
   int32_t pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, group;
   int32_t x_layout;       /* SOFIE_LAYOUT_* of X                                          */
   int32_t y_layout;       /* SOFIE_LAYOUT_* of Y                                          */
   int32_t w_packed;       /* 0: W as in ONNX [Cout,C/g,kH,kW]; 1: packed by sofie_cuda_conv2d_pack_* */
   int32_t relu;           /* fused Relu                                                   */
   int32_t pool;           /* 0: none; 2: fused MaxPool kernel 2x2 stride 2 (after Relu)   */
} sofie_conv2d_desc;
int sofie_cuda_conv2d_f32(void *stream, const sofie_conv2d_desc *desc, const float *X, const float *W,
                          const float *bias, float *Y);
/* Repack ONNX weights [Cout,C,kH,kW] to the tensor-core layout [Cout][kH][kW][C] (group 1). */
int sofie_cuda_conv2d_pack_f32(void *stream, const sofie_conv2d_desc *desc, const float *W, float *Wpacked);

/* ConvTranspose 2-D, group 1 (reference: ROperator_ConvTranspose.icc:364-474 with UTILITY::col2im,
 * SOFIE_common.hxx:576-620: per-image filter GEMM, scatter-add, broadcast bias added at the end).
 * X [N,C,H,W], W [C,Cout,kH,kW] (the ONNX layout), bias [Cout] or NULL, Y [N,Cout,oH,oW] with
 * o = stride*(i-1) + dil*(k-1)+1 + out_pad - 2*pad (ShapeInference :83-90), all NCHW.
 * A 1-D ConvTranspose is the same call with H = kH = 1. */
typedef struct sofie_conv_transpose2d_desc {
   int32_t N, C, H, W;
   int32_t Cout;
   int32_t kH, kW, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w;
   int32_t out_pad_h, out_pad_w;
   int32_t relu;            /* fused y = max(y, 0)                                          */
} sofie_conv_transpose2d_desc;
int sofie_cuda_conv_transpose2d_f32(void *stream, const sofie_conv_transpose2d_desc *desc, const float *X, const float *W,
                                    const float *bias, float *Y);
/* The same operator as the reference lowers it (ROperator_ConvTranspose.icc:364-474: filter GEMM, then col2im), with the
 * GEMM on the tensor cores: the images are made channel-last, ONE product [N*H*W, C] x [C, kH*kW*Cout] covers all of
 * them (sofie_cuda_gemm_f32), and every output pixel gathers its taps' products, adds the bias and applies Relu.
 * `scratch` is device memory of sofie_conv_transpose2d_gemm_scratch_bytes(desc) bytes, 256-byte aligned, that the call
 * overwrites (channel-last input, re-ordered filters, the products); 0 bytes = this shape is not served (fewer than 16
 * input channels or a count that is not a multiple of 4: use sofie_cuda_conv_transpose2d_f32). Host arithmetic only, so
 * that a code generator can plan the buffer without a GPU. */
static inline size_t sofie_round_up_floats(size_t n) { return (n + 63) & ~(size_t)63; } /* 256-byte steps */
static inline size_t sofie_conv_transpose2d_gemm_scratch_bytes(const sofie_conv_transpose2d_desc *d)
{
   size_t pixels, taps;
   if (d->C < 16 || d->C % 4 != 0 || d->N < 1 || d->H < 1 || d->W < 1 || d->Cout < 1 || d->kH < 1 || d->kW < 1) return 0;
   pixels = (size_t)d->N * (size_t)d->H * (size_t)d->W;
   taps = (size_t)d->kH * (size_t)d->kW;
   return 4 * (sofie_round_up_floats(pixels * (size_t)d->C) + sofie_round_up_floats(taps * (size_t)d->Cout * (size_t)d->C) +
               sofie_round_up_floats(pixels * taps * (size_t)d->Cout));
}
size_t sofie_cuda_conv_transpose2d_f32_gemm_scratch(const sofie_conv_transpose2d_desc *desc); /* the same value, as an exported symbol */
int sofie_cuda_conv_transpose2d_f32_gemm(void *stream, const sofie_conv_transpose2d_desc *desc, const float *X, const float *W,
                                         const float *bias, float *Y, void *scratch, size_t scratch_bytes);

/* 3-D convolution (reference: ROperator_Conv.hxx with fDim == 3, :95-201 and UTILITY::Im2col_3d, SOFIE_common.hxx:521-573):
 * X [N, C, D, H, W], W [Cout, C/group, kD, kH, kW], Y [N, Cout, oD, oH, oW] with o = (i + 2*pad - (dil*(k-1)+1)) / stride + 1
 * per axis; asymmetric ONNX pads are averaged by the caller as for the 2-D operator. Direct kernel on CUDA cores. */
typedef struct sofie_conv3d_desc {
   int32_t N, C, D, H, W;
   int32_t Cout;
   int32_t kD, kH, kW, pad_d, pad_h, pad_w, stride_d, stride_h, stride_w, dil_d, dil_h, dil_w;
   int32_t group;
   int32_t relu;            /* fused y = max(y, 0)                                          */
} sofie_conv3d_desc;
int sofie_cuda_conv3d_f32(void *stream, const sofie_conv3d_desc *desc, const float *X, const float *W, const float *bias, float *Y);

/* MaxPool / AveragePool 3-D (reference: the fDim == 3 loops of ROperator_Pool.hxx:266-476) on [N, C, D, H, W];
 * pads = (d_begin, h_begin, w_begin, d_end, h_end, w_end) as in ONNX. */
typedef struct sofie_pool3d_desc {
   int32_t mode;            /* 0: max, 1: average                                           */
   int32_t N, C, D, H, W;
   int32_t kD, kH, kW, stride_d, stride_h, stride_w;
   int32_t pads[6];
   int32_t count_include_pad;
} sofie_pool3d_desc;
int sofie_cuda_pool3d_f32(void *stream, const sofie_pool3d_desc *desc, const float *X, float *Y);

/* Einsum of two operands, general form (reference: ROperator_Einsum.hxx:200-332, nested loops or one sgemm_ per
 * stack index): Y[out labels] = sum over all other labels of A[...] * B[...]. The labels are listed by extent, first
 * the n_out output labels in output order, then the n_sum summed ones; a_stride / b_stride give the element stride
 * of each label in A and B (0 when the operand does not carry it). Y is dense row-major over the output labels. */
#define SOFIE_EINSUM_MAX_LABELS 8
typedef struct sofie_einsum_desc {
   int32_t n_out, n_sum;
   int64_t extent[SOFIE_EINSUM_MAX_LABELS];
   int64_t a_stride[SOFIE_EINSUM_MAX_LABELS];
   int64_t b_stride[SOFIE_EINSUM_MAX_LABELS];
} sofie_einsum_desc;
int sofie_cuda_einsum_f32(void *stream, const sofie_einsum_desc *desc, const float *A, const float *B, float *Y);

/* ------------------------------------------------------------------ fp32 memory-bound ops --- */
/* y = x > 0 ? x : 0 (reference: ROperator_Relu.hxx:54-66). In place allowed. */
int sofie_cuda_relu_f32(void *stream, const float *X, float *Y, size_t n);

/* MaxPool / AveragePool 2-D (reference: ROperator_Pool.hxx:266-476). `pads` =
 * (h_begin, w_begin, h_end, w_end) as in ONNX and in the reference's shape inference
 * (ROperator_Pool.hxx:172-189). The reference's loop bounds read the vector in another order
 * (ROperator_Pool.hxx:283-289); both readings agree when the four pads are equal, the only padded
 * case in which the reference stays inside its output tensor. */
typedef struct sofie_pool2d_desc {
   int32_t mode;            /* 0 max, 1 average                                            */
   int32_t N, C, H, W;
   int32_t kH, kW, stride_h, stride_w;
   int32_t pads[4];
   int32_t count_include_pad;
   int32_t layout;          /* SOFIE_LAYOUT_* of both X and Y                               */
} sofie_pool2d_desc;
int sofie_cuda_pool2d_f32(void *stream, const sofie_pool2d_desc *desc, const float *X, float *Y);

/* Softmax along one axis of a tensor viewed as [outer, axis_len, inner]
 * (reference: ROperator_Softmax.hxx:53-184). */
int sofie_cuda_softmax_f32(void *stream, const float *X, float *Y, size_t outer, size_t axis_len, size_t inner);

/* Fused multi-layer perceptron: Y = L_{n-1}(... L_0(X)) with L_l(x) = act(x W_l^T + b_l), one launch
 * for the whole chain of Gemm (+ Relu) operators (reference: one ROperator_Gemm::Generate,
 * ROperator_Gemm.hxx:292-390, per layer). For small layers only: every width <= SOFIE_MLP_MAX_WIDTH
 * and sofie_mlp_smem_bytes(desc) <= SOFIE_MLP_MAX_SMEM (all weights, padded, plus three activation
 * tiles in shared memory); otherwise SOFIE_CUDA_ERR_UNSUPPORTED and the caller issues one
 * sofie_cuda_gemm_f32 per layer. W and B are HOST arrays of `layers` device pointers (B or B[l] may
 * be NULL); w_is_nk[l] = 1 when W_l is stored [dims[l+1]][dims[l]] (ONNX Gemm with transB = 1), 0 for
 * [dims[l]][dims[l+1]]. X is [M, dims[0]], Y is [M, dims[layers]]. 16-byte aligned pointers, [N][K]
 * weights and widths that are multiples of 4 take the fast staging path; everything else is
 * correct but staged element by element. */
#define SOFIE_MLP_MAX_LAYERS 8
#define SOFIE_MLP_MAX_WIDTH 256
#define SOFIE_MLP_MAX_SMEM (200 * 1024)
typedef struct sofie_mlp_desc {
   int32_t M;
   int32_t layers;
   int32_t dims[SOFIE_MLP_MAX_LAYERS + 1];
   int32_t relu[SOFIE_MLP_MAX_LAYERS];
   int32_t w_is_nk[SOFIE_MLP_MAX_LAYERS];
} sofie_mlp_desc;
int sofie_cuda_mlp_f32(void *stream, const sofie_mlp_desc *desc, const float *X, const float *const *W, const float *const *B, float *Y);
/* Shared memory the fused kernel needs for a chain (independent of M): host arithmetic only, so that a
 * code generator can decide between the fused call and one GEMM per layer without a GPU.
 * Rows are padded to a multiple of 4 floats whose quarter is odd (bank spreading). */
static inline int32_t sofie_mlp_padded_ld(int32_t k) { return 4 * ((((k + 3) >> 2) + 1) | 1); }
static inline size_t sofie_mlp_smem_bytes(const sofie_mlp_desc *d)
{
   size_t floats = 0;
   int32_t maxact = 0, l;
   for (l = 0; l < d->layers; l++) {
      const int32_t np = (d->dims[l + 1] + 31) & ~31;
      floats += (size_t)np * sofie_mlp_padded_ld(d->dims[l]) + np;
      if (d->dims[l + 1] > maxact) maxact = d->dims[l + 1];
   }
   floats += 32 * (size_t)sofie_mlp_padded_ld(d->dims[0]) + 2 * 32 * (size_t)sofie_mlp_padded_ld(maxact);
   return floats * sizeof(float);
}
size_t sofie_cuda_mlp_f32_smem(const sofie_mlp_desc *desc); /* the same value, as an exported symbol */
/* Chains that sofie_cuda_mlp_f32 can also run on the tensor cores (tcgen05, 3xTF32, 128 rows per CTA, activations
 * handed from layer to layer through tensor memory and shared memory) when sofie_cuda_set_engine forces that engine:
 * up to four layers, every layer's input width a multiple of 8 and at most 128, outputs at most 128 wide,
 * intermediate widths multiples of 16. Not the default (it is slower than the FMA kernel on small batches and than one
 * tensor-core GEMM per layer on large ones). Host arithmetic only. */
static inline int sofie_mlp_tensor_core_shape(const sofie_mlp_desc *d)
{
   int32_t l;
   if (d->layers < 1 || d->layers > 4) return 0;
   for (l = 0; l < d->layers; l++) {
      const int32_t k = d->dims[l], n = d->dims[l + 1];
      if (k < 8 || k % 8 != 0 || k > 128 || n < 1 || n > 128) return 0;
      if (l + 1 < d->layers && n % 16 != 0) return 0;
   }
   return 1;
}

/* Unary operators, y[i] = f(x[i]). The formulas are the ones the reference emits
 * (ROperator_Sigmoid.hxx:59, ROperator_Tanh.hxx:60, ROperator_LeakyRelu.hxx:73, ROperator_Selu.hxx:59,
 * ROperator_Elu.hxx:71 -- including its `alpha * exp(x) - 1` for x < 0 --, ROperator_BasicUnary.hxx).
 * alpha is read by LEAKY_RELU and ELU only. */
enum {
   SOFIE_UNARY_SIGMOID = 0,
   SOFIE_UNARY_TANH = 1,
   SOFIE_UNARY_LEAKY_RELU = 2,
   SOFIE_UNARY_SELU = 3,
   SOFIE_UNARY_ELU = 4,
   SOFIE_UNARY_NEG = 5,
   SOFIE_UNARY_EXP = 6,
   SOFIE_UNARY_LOG = 7,
   SOFIE_UNARY_SQRT = 8,
   SOFIE_UNARY_RECIPROCAL = 9,
   SOFIE_UNARY_ABS = 10,
   SOFIE_UNARY_ERF = 11,   /* std::erf(x)              (ROperator_Erf.hxx:58)   */
   SOFIE_UNARY_SWISH = 12, /* x / (1 + exp(-x))        (ROperator_Swish.hxx:59) */
   SOFIE_UNARY_COS = 13,   /* ROperator_BasicUnary.hxx */
   SOFIE_UNARY_SIN = 14
};
int sofie_cuda_unary_f32(void *stream, int32_t op, float alpha, const float *X, float *Y, size_t n);

/* Binary operators with multidirectional broadcasting (reference: ROperator_BasicBinary.hxx:18-43,
 * 176-230). The output has `shape` (rank 4, leading 1s for lower ranks); an operand's stride, in
 * elements, is 0 along a dimension it is broadcast over. */
enum { SOFIE_BINARY_ADD = 0, SOFIE_BINARY_SUB = 1, SOFIE_BINARY_MUL = 2, SOFIE_BINARY_DIV = 3 };
typedef struct sofie_binary_desc {
   int32_t op;
   int64_t shape[4];
   int64_t a_stride[4], b_stride[4];
} sofie_binary_desc;
int sofie_cuda_binary_f32(void *stream, const sofie_binary_desc *desc, const float *A, const float *B, float *Y);

/* Inference-mode BatchNormalization on [N, C, HW] (NCHW) or [N, HW, C] (NHWC):
 * y = ((x - mean[c]) * scale[c]) + bias[c], optional Relu; `scale` already holds
 * gamma / sqrt(var + epsilon), which the reference folds at Initialize time
 * (ROperator_BatchNormalization.hxx:163-168, 200-226). */
typedef struct sofie_batchnorm_desc {
   int32_t N, C, HW;
   int32_t layout;          /* SOFIE_LAYOUT_* of X and Y */
   int32_t relu;
} sofie_batchnorm_desc;
int sofie_cuda_batchnorm_f32(void *stream, const sofie_batchnorm_desc *desc, const float *X, const float *scale, const float *bias,
                             const float *mean, float *Y);

/* NCHW <-> NHWC copies for tensors that cross a layout boundary un-fused. */
int sofie_cuda_nchw_to_nhwc_f32(void *stream, const float *X, float *Y, int32_t N, int32_t C, int32_t H, int32_t W);
int sofie_cuda_nhwc_to_nchw_f32(void *stream, const float *X, float *Y, int32_t N, int32_t C, int32_t H, int32_t W);

/* ------------------------------------------------------------------ int8 -------------------- */
/* The reference has no quantised operators (src/SOFIE_parsers/src/RModelParser_ONNX.cxx:154-236
 * registers none); these follow the ONNX operator definitions with int32 accumulation and
 * q = clamp(rne((float)acc * mult[n])) + y_zp, bit-exactly reproducible on a CPU. */

/* QuantizeLinear to uint8: y = saturate(rne(x / scale) + zp). */
int sofie_cuda_quantize_u8(void *stream, const float *X, uint8_t *Y, size_t n, float scale, int32_t zp);
/* DequantizeLinear from uint8: y = (x - zp) * scale. */
int sofie_cuda_dequantize_u8(void *stream, const uint8_t *X, float *Y, size_t n, float scale, int32_t zp);

/*
 * Host-side, once per Session: from HOST int8 weights computes, in a fixed fp32 order,
 *   mult[n] = (a_scale * w_scale[n]) / y_scale     and
 *   corr[n] = bias[n] - a_zp * sum_k W[n][k]       (int32; bias may be NULL)
 * and writes both to the given DEVICE buffers of N elements each. `rows_per_n` is the number of
 * weights per output channel (K for a matmul, C*kH*kW for a convolution).
 */
int sofie_cuda_qlinear_prepare(void *stream, int32_t N, int32_t rows_per_n, const int8_t *W_host, int32_t w_is_nk,
                               float a_scale, int32_t a_zp, const float *w_scale_host, float y_scale,
                               const int32_t *bias_host, float *mult_device, int32_t *corr_device);

/* QLinearMatMul: Y = requant(A[M,K] (uint8) x W (int8), per-output-channel multiplier). */
typedef struct sofie_qgemm_desc {
   int32_t M, N, K;
   int32_t w_is_nk;  /* 1: W is [N,K]; 0: W is [K,N] as ONNX stores it                        */
   int32_t y_zp;
   int32_t relu;     /* q = max(q, y_zp)                                                     */
} sofie_qgemm_desc;
int sofie_cuda_qlinear_matmul(void *stream, const sofie_qgemm_desc *desc, const uint8_t *A, const int8_t *W,
                              const float *mult, const int32_t *corr, uint8_t *Y);
/* QLinearMatMul followed by DequantizeLinear (same scale and zero point as the product's output) in one
 * pass: Y = (q - y_zp) * y_scale with q the uint8 value sofie_cuda_qlinear_matmul writes, bit for bit what
 * sofie_cuda_dequantize_u8 computes from it, without the uint8 tensor's trip through memory. */
int sofie_cuda_qlinear_matmul_f32(void *stream, const sofie_qgemm_desc *desc, const uint8_t *A, const int8_t *W, const float *mult,
                                  const int32_t *corr, float y_scale, float *Yf32);
/* out[N,K] = in[K,N]^T for int8 weights. */
int sofie_cuda_transpose_i8(void *stream, const int8_t *in, int8_t *out, int32_t rows, int32_t cols);

/* QLinearConv 2-D: uint8 activations (zero point x_zp; padding contributes nothing), int8 weights,
 * per-Cout multiplier, optional Relu and fused MaxPool 2x2. `corr` is bias only (int32, may be
 * NULL); the zero-point term is applied per output position because it depends on which taps fall
 * inside the image. */
typedef struct sofie_qconv2d_desc {
   int32_t N, C, H, W, Cout, kH, kW, pad_h, pad_w, stride_h, stride_w;
   int32_t x_layout, y_layout, w_packed;
   int32_t x_zp, y_zp;
   int32_t relu, pool;
} sofie_qconv2d_desc;
int sofie_cuda_qlinear_conv2d(void *stream, const sofie_qconv2d_desc *desc, const uint8_t *X, const int8_t *W,
                              const float *mult, const int32_t *bias, uint8_t *Y);
int sofie_cuda_qconv2d_pack_i8(void *stream, const sofie_qconv2d_desc *desc, const int8_t *W, int8_t *Wpacked);
/* MaxPool 2-D on uint8 (integer max), no padding. */
int sofie_cuda_maxpool2d_u8(void *stream, const uint8_t *X, uint8_t *Y, int32_t N, int32_t C, int32_t H, int32_t W,
                            int32_t kH, int32_t kW, int32_t stride_h, int32_t stride_w, int32_t layout);
/* uint8 NCHW <-> NHWC. */
int sofie_cuda_nchw_to_nhwc_u8(void *stream, const uint8_t *X, uint8_t *Y, int32_t N, int32_t C, int32_t H, int32_t W);
int sofie_cuda_nhwc_to_nchw_u8(void *stream, const uint8_t *X, uint8_t *Y, int32_t N, int32_t C, int32_t H, int32_t W);

/* ------------------------------------------------------------------ FP8 E4M3 ---------------- */
/* Also absent from the reference. E4M3 is the "FN" encoding (max 448, no infinities); bf16 and
 * E4M3 values cross this ABI as raw uint16_t / uint8_t bit patterns. */

/* y = e4m3(x / scale), round to nearest even, saturating. */
int sofie_cuda_quantize_e4m3_f32(void *stream, const float *X, uint8_t *Y, size_t n, float scale);
int sofie_cuda_quantize_e4m3_bf16(void *stream, const uint16_t *X, uint8_t *Y, size_t n, float scale);
int sofie_cuda_cast_bf16_f32(void *stream, const uint16_t *X, float *Y, size_t n);
int sofie_cuda_cast_f32_bf16(void *stream, const float *X, uint16_t *Y, size_t n);
/* max |x| over n values, written to one device float (per-tensor FP8 scale = amax / 448). */
int sofie_cuda_amax_f32(void *stream, const float *X, size_t n, float *amax_device);

/* Y = bf16( relu( (A x W^T) * (a_scale*w_scale) + bias ) ), A [M,K] and W [N,K] E4M3, fp32
 * accumulation. When q_scale > 0 the same pass also writes Yq = e4m3(bf16 result / q_scale), the
 * quantised input of the next FP8 layer, so the activation does not make another trip to HBM. */
typedef struct sofie_fp8_gemm_desc {
   int32_t M, N, K;
   float a_scale, w_scale;
   int32_t relu;
   float q_scale;
} sofie_fp8_gemm_desc;
int sofie_cuda_gemm_e4m3(void *stream, const sofie_fp8_gemm_desc *desc, const uint8_t *A, const uint8_t *W,
                         const float *bias, uint16_t *Ybf16, uint8_t *Yq);
/* The same product with the result written as float: Y = float( bf16( relu(...) ) ), bit for bit what
 * sofie_cuda_gemm_e4m3 followed by sofie_cuda_cast_bf16_f32 writes, without the bf16 tensor's trip through
 * memory (the last layer of a chain whose result goes back to the host as float). q_scale is ignored. */
int sofie_cuda_gemm_e4m3_f32(void *stream, const sofie_fp8_gemm_desc *desc, const uint8_t *A, const uint8_t *W,
                             const float *bias, float *Yf32);

/* Dynamic per-tensor scales ("scales computed from amax" at run time instead of calibrated ones). The first call computes
 * max|x| over the n values, stores scale = amax / 448 (1 for an all-zero tensor) in *scale_device and writes
 * Y = e4m3(x / scale) with the rounding of the static form; the second is sofie_cuda_gemm_e4m3 / _f32 with the
 * activation scale read from device memory (desc->a_scale and desc->q_scale are ignored: the following layer's scale is
 * only known once this product is complete, so its input is quantised by the next dynamic_quantize call). Everything
 * stays on the stream: no value travels to the host. */
int sofie_cuda_dynamic_quantize_e4m3_f32(void *stream, const float *X, uint8_t *Y, size_t n, float *scale_device);
int sofie_cuda_dynamic_quantize_e4m3_bf16(void *stream, const uint16_t *X, uint8_t *Y, size_t n, float *scale_device);
int sofie_cuda_gemm_e4m3_dynamic(void *stream, const sofie_fp8_gemm_desc *desc, const uint8_t *A, const float *a_scale_device,
                                 const uint8_t *W, const float *bias, uint16_t *Ybf16, float *Yf32);

#ifdef __cplusplus
}
#endif
#endif /* SOFIE_CUDA_H */
