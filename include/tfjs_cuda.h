/*
 * C ABI of the B200 `cuda` kernel backend for tfjs-core.
 *
 * This is the boundary a Node N-API shim (or any FFI: ctypes, cffi) binds.  It follows the
 * shape of the reference's only native backend ABI, tfjs-backend-wasm/src/lib.cc:57-132
 * (`register_tensor(id, shape, rank, dtype, ptr)`, `dispose_data(id)`, `add(a_id, b_id,
 * out_id)`, `dispose()`): tensors are integer ids in a table owned by the library, kernels
 * take ids.  Unlike the wasm ABI the table lives in an explicit per-device context, storage
 * is cudaMalloc'd device memory owned by the library, and every call returns a status.
 *
 * Each entry point names the KernelBackend method (tfjs-core/src/backends/backend.ts) or
 * engine call it serves.
 *
 * Conventions
 *  - return 0 on success, a negative tfjs_cuda_status otherwise; never abort, never throw.
 *  - tfjs_cuda_last_error(ctx) gives the message of the last failure on that context.
 *  - kernels only enqueue work on the context's stream and return; tensor_read blocks.
 *  - one context = one device + one stream; calls on one context come from one host
 *    thread at a time.  Different contexts are independent (one per GPU for batch sharding).
 *  - zero-sized tensors are legal everywhere and launch nothing.
 *  - there is no CPU fallback: if no CUDA device is usable, ctx_create fails.
 */
#ifndef TFJS_CUDA_H_
#define TFJS_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tfjs_cuda_ctx tfjs_cuda_ctx;
typedef struct tfjs_cuda_event tfjs_cuda_event;
typedef struct tfjs_cuda_graph tfjs_cuda_graph;
typedef int64_t tfjs_tensor_id; /* 0 is never a valid id; use 0 for "absent" operands */

typedef enum {
  TFJS_CUDA_OK = 0,
  TFJS_CUDA_ERR_INVALID_ARG = -1,
  TFJS_CUDA_ERR_OOM = -2,
  TFJS_CUDA_ERR_CUDA = -3,
  TFJS_CUDA_ERR_TIMEOUT = -4,
  TFJS_CUDA_ERR_UNSUPPORTED = -5,
  TFJS_CUDA_ERR_NOT_FOUND = -6
} tfjs_cuda_status;

/* DataType subset the path stores; numbering of tfjs-backend-wasm/src/lib.cc:26-30.
 * TFJS_F16 is an extension: a float32 tensor whose STORAGE is IEEE half precision (2 bytes per
 * element).  It is the storage of activations in the 16-bit precision class of the reference
 * (KernelBackend.floatPrecision() == 16, backends/backend.ts:120-126; the WebGL backend on
 * devices with half-float textures): tensor_write takes and tensor_read returns float32 values,
 * the convolution, separable-convolution, depthwise and pooling entry points read and write it
 * natively, every other kernel takes it after tfjs_cuda_cast to TFJS_F32. */
typedef enum { TFJS_F32 = 0, TFJS_I32 = 1, TFJS_BOOL = 2, TFJS_F16 = 3 } tfjs_dtype;

/* Activation of fused ops.  linear/relu/prelu are tfjs-core/src/ops/fused_util.ts:20;
 * CLIP is an extension (relu6 = clip(0, 6), i.e. tf.clipByValue fused into the producer). */
typedef enum {
  TFJS_ACT_LINEAR = 0,
  TFJS_ACT_RELU = 1,
  TFJS_ACT_PRELU = 2,
  TFJS_ACT_CLIP = 3
} tfjs_activation;

/* Contraction arithmetic: TF32 = one tcgen05 pass on tf32-rounded operands (max error
 * ~1e-3 relative); TF32X3 = three passes on hi/lo splits (fp32-level, ~1e-6). */
typedef enum { TFJS_MATH_TF32X3 = 0, TFJS_MATH_TF32 = 1 } tfjs_math_mode;

typedef enum { TFJS_BIN_ADD = 0, TFJS_BIN_SUB = 1, TFJS_BIN_MUL = 2, TFJS_BIN_DIV = 3,
               TFJS_BIN_PRELU = 4, TFJS_BIN_NOT_EQUAL = 5 } tfjs_binary_op;
typedef enum { TFJS_UN_RELU = 0, TFJS_UN_CLIP = 1, TFJS_UN_EXP = 2, TFJS_UN_LOG = 3,
               TFJS_UN_INT = 4, TFJS_UN_STEP = 5 /* p0 = alpha */ } tfjs_unary_op;
typedef enum { TFJS_RED_SUM = 0, TFJS_RED_MAX = 1, TFJS_RED_ARGMAX = 2 } tfjs_reduce_op;

/* Conv2DInfo, tfjs-core/src/ops/conv_util.ts:43-64, channelsLast (NHWC) only; padInfo is
 * flattened.  The op layer computes it (computeConv2DInfo :123-182) and passes it down. */
typedef struct {
  int32_t batchSize, inHeight, inWidth, inChannels;
  int32_t outHeight, outWidth, outChannels;
  int32_t strideHeight, strideWidth;
  int32_t dilationHeight, dilationWidth;
  int32_t filterHeight, filterWidth;
  int32_t effectiveFilterHeight, effectiveFilterWidth;
  int32_t padTop, padBottom, padLeft, padRight;
} tfjs_conv2d_info;

/* Fused epilogue: out = act(acc + bias).  bias/prelu are tensor ids or 0.  bias_len and
 * prelu_len are 1 (scalar) or the output channel count (a vector broadcast along the
 * inner-most axis); any other broadcast shape is composed by the caller from the linear
 * op followed by tfjs_cuda_binary, as MathBackendCPU does (backend_cpu.ts:542-555). */
typedef struct {
  tfjs_tensor_id bias;
  int64_t bias_len;
  int32_t activation; /* tfjs_activation */
  tfjs_tensor_id prelu;
  int64_t prelu_len;
  float clip_lo, clip_hi; /* TFJS_ACT_CLIP only */
} tfjs_epilogue;

typedef struct {
  int64_t num_tensors;        /* live entries in the tensor table */
  int64_t bytes_in_use;       /* device bytes held by live tensors */
  int64_t bytes_reserved;     /* device bytes obtained from cudaMalloc (live + cached) */
  int64_t num_buffers_cached; /* free buffers waiting for reuse */
  int64_t num_device_allocs;  /* cudaMalloc calls so far */
} tfjs_cuda_mem_stats;

/* ---- context: the backend factory of tf.registerBackend('cuda', factory)
 *      (tfjs-core/src/engine.ts:220-307) creates one; KernelBackend.dispose() destroys it. */
int tfjs_cuda_ctx_create(int device_ordinal, tfjs_cuda_ctx** out);
/* Number of usable CUDA devices (0 when there is none): one context per device is how a batch is
 * sharded, each registered as its own backend 'cuda:0' ... 'cuda:N-1' (the engine's registry is
 * keyed by name, tfjs-core/src/engine.ts:132-138, 220-232). */
int tfjs_cuda_device_count(int* out);
int tfjs_cuda_ctx_destroy(tfjs_cuda_ctx* ctx);
const char* tfjs_cuda_last_error(const tfjs_cuda_ctx* ctx);
/* Flags mirrored from ENV.registerFlag (environment.ts:32-142).  Keys: "math_mode"
 * (tfjs_math_mode), "use_tensor_cores" (0 forces the CUDA-core kernels), "debug_sync",
 * "dequant_in_gemm" (quantised matMul / 1x1 conv2d weights: 0, the default, expands them once
 * into cached tf32 planes; 1 keeps them uint8 in device memory and dequantises each tile in
 * shared memory inside the GEMM main loop; the results are bit-identical), "fuse_separable"
 * (see tfjs_cuda_separable_conv2d), "gemm_pair" (TF32 matMul / 1x1 conv2d on pairs of CTAs that
 * share each weight tile: 1, the default, where the problem is large enough to pay; 0 never; 2
 * wherever the shape allows; the results are bit-identical either way), "gemm_block_n" (diagnostic:
 * 32, 64, 128 or 256 fixes the tile width of the single-CTA tensor-core matMul, 0 leaves it to the
 * cost model), "pdl" (1 launches the main kernels with programmatic stream
 * serialization, so that a kernel's prologue overlaps its predecessor's tail; default 0),
 * "wait_limit_us" (every device-side wait of the kernels is bounded; a wait that runs out makes
 * the kernel return and the next ctx_sync / tensor_read report TFJS_CUDA_ERR_TIMEOUT, the context
 * stays usable; default 2 s, per device), "debug_canary" (1: every buffer is followed by a guard
 * pattern that is verified when the buffer is released; an overwritten guard is reported as
 * TFJS_CUDA_ERR_CUDA at the next synchronisation), "test_withhold_last_load" (diagnostic: the
 * tensor-core matMul withholds its last load so that the bounded waits run out). */
int tfjs_cuda_ctx_set_option(tfjs_cuda_ctx* ctx, const char* key, double value);
/* Blocks until all enqueued work is done; TFJS_CUDA_ERR_TIMEOUT after timeout_ms (<0: none). */
int tfjs_cuda_ctx_sync(tfjs_cuda_ctx* ctx, int timeout_ms);
/* KernelBackend.memory() (backend.ts:114-116). */
int tfjs_cuda_ctx_memory(tfjs_cuda_ctx* ctx, tfjs_cuda_mem_stats* out);
/* KernelBackend.time(f) (backend.ts:92-94): bracket f() with these; *kernel_ms is device
 * time between them, *num_launches the kernels this library launched in between. */
int tfjs_cuda_ctx_time_begin(tfjs_cuda_ctx* ctx);
int tfjs_cuda_ctx_time_end(tfjs_cuda_ctx* ctx, float* kernel_ms, int64_t* num_launches);
/* Per-kernel device timing, the "extra profile info" of BackendTimingInfo (backend.ts:27-31)
 * and the per-kernel rows of the DEBUG profiler (profiler.ts:30-74): between begin and end an
 * event is recorded after every launch (up to max_launches); profile_get(i) returns the name
 * and the device milliseconds of the i-th launch. */
int tfjs_cuda_profile_begin(tfjs_cuda_ctx* ctx, int max_launches);
int tfjs_cuda_profile_end(tfjs_cuda_ctx* ctx, int* num_launches);
int tfjs_cuda_profile_get(tfjs_cuda_ctx* ctx, int index, const char** name, float* ms);
/* Total kernels launched by this context since creation. */
int64_t tfjs_cuda_ctx_launch_count(const tfjs_cuda_ctx* ctx);
/* The cudaStream_t of the context (as void*), for callers that time with their own events. */
void* tfjs_cuda_ctx_stream(tfjs_cuda_ctx* ctx);

/* ---- tensor storage: KernelBackend.register / write / readSync / read / disposeData
 *      (backend.ts:95-113; CPU backend_cpu.ts:102-129, 199-237). */
int tfjs_cuda_tensor_register(tfjs_cuda_ctx* ctx, tfjs_tensor_id* out_id, int rank,
                              const int64_t* shape, int dtype);
int tfjs_cuda_tensor_write(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, const void* host, size_t nbytes);
int tfjs_cuda_tensor_read(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, void* host, size_t nbytes);
/* Extension of KernelBackend.write for pipelined input: the upload runs on a second stream, after
 * the kernels already enqueued (which may still read the old contents) and concurrently with
 * whatever is enqueued next.  Kernels and reads that take the tensor as an operand wait for it
 * automatically; a captured graph cannot know its inputs, so call tensor_wait(ctx, id) before
 * graph_launch for every tensor written this way.  `host` should be pinned memory
 * (tfjs_cuda_host_alloc) and must stay valid until the upload has finished. */
int tfjs_cuda_tensor_write_async(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, const void* host,
                                 size_t nbytes);
int tfjs_cuda_tensor_wait(tfjs_cuda_ctx* ctx, tfjs_tensor_id id);
/* Non-blocking readback for KernelBackend.read(): the copy into `host` (pinned memory for a
 * truly asynchronous copy) completes when the event does. */
int tfjs_cuda_tensor_read_async(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, void* host, size_t nbytes,
                                tfjs_cuda_event** out_event);
int tfjs_cuda_event_query(tfjs_cuda_event* ev); /* 1 done, 0 pending, <0 error */
int tfjs_cuda_event_wait(tfjs_cuda_event* ev, int timeout_ms);
int tfjs_cuda_event_destroy(tfjs_cuda_event* ev);
/* Idempotent, like backend_cpu.ts:228-237; unknown ids are ignored. */
int tfjs_cuda_tensor_dispose(tfjs_cuda_ctx* ctx, tfjs_tensor_id id);
/* Device pointer and byte size of a tensor's storage (zero-copy interop, benchmarks). */
int tfjs_cuda_tensor_device_ptr(tfjs_cuda_ctx* ctx, tfjs_tensor_id id, void** ptr, size_t* nbytes);
/* Pinned host staging memory for write/read_async callers. */
int tfjs_cuda_host_alloc(void** ptr, size_t nbytes);
int tfjs_cuda_host_free(void* ptr);

/* Extension: keep a weight tensor as uint8 affine-quantised bytes, w = q*scale + min
 * (tfjs-core/src/io/io_utils.ts:122-146, manifest field io/types.ts:103-107).  The id can be
 * passed as the filter / b operand of conv2d and batch_matmul (dequantised in shared memory
 * inside the GEMM main loop) and of depthwise_conv2d.  tensor_read returns the float32
 * values decodeWeights would have produced. */
int tfjs_cuda_tensor_register_quantized(tfjs_cuda_ctx* ctx, tfjs_tensor_id* out_id, int rank,
                                        const int64_t* shape, const uint8_t* q, double scale,
                                        double min);

/* ---- contractions.
 * KernelBackend.batchMatMul / fusedBatchMatMul (backend.ts:128-138; CPU :491-555):
 * a is [batch, a_d1, a_d2], b is [batch, b_d1, b_d2]; out is [batch, M, N] with
 * M = transpose_a ? a_d2 : a_d1, N = transpose_b ? b_d1 : b_d2.  epi may be NULL. */
int tfjs_cuda_batch_matmul(tfjs_cuda_ctx* ctx, tfjs_tensor_id a, tfjs_tensor_id b,
                           tfjs_tensor_id out, int32_t batch, int32_t a_d1, int32_t a_d2,
                           int32_t b_d1, int32_t b_d2, int transpose_a, int transpose_b,
                           const tfjs_epilogue* epi);
/* KernelBackend.conv2d / fusedConv2d (backend.ts:414-422; CPU :1536-1616). */
int tfjs_cuda_conv2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id filter,
                     tfjs_tensor_id out, const tfjs_conv2d_info* info, const tfjs_epilogue* epi);

/* ---- memory-bound kernels.
 * KernelBackend.depthwiseConv2D (backend.ts:431-434; CPU :1979-2035).  epi != NULL is the
 * fused extension depthwise + bias + activation; NULL is the reference method. */
int tfjs_cuda_depthwise_conv2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id filter,
                               tfjs_tensor_id out, const tfjs_conv2d_info* info,
                               const tfjs_epilogue* epi);
/* Extension: the op pair of tf.separableConv2d (ops/conv.ts:574-654) with an epilogue after each
 * half: out = pw_epi(conv2d_1x1(dw_epi(depthwiseConv2D(x, dw_filter)), pw_filter)).  `dw_info` is
 * the depthwise Conv2DInfo; pw_filter is [1, 1, dw_info->outChannels, out_channels]; out is
 * [batch, outHeight, outWidth, out_channels].  3x3 filters with stride 1 or 2, a channel count
 * that is a multiple of 32 up to 256 and up to 256 output channels run, in TF32 mode, as one
 * kernel that keeps the depthwise result in shared memory; other shapes run the two kernels back
 * to back.  Results are bit-identical to the two separate calls.  Option "fuse_separable": 0
 * forces the two-kernel form, 1 (default) fuses where that is the faster form (up to 128
 * channels, and 256 channels at stride 1), 2 fuses every shape the kernel takes. */
int tfjs_cuda_separable_conv2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id dw_filter,
                               tfjs_tensor_id pw_filter, tfjs_tensor_id out,
                               const tfjs_conv2d_info* dw_info, int32_t out_channels,
                               const tfjs_epilogue* dw_epi, const tfjs_epilogue* pw_epi);
/* ---- gradient kernels, so that the engine's tape differentiates through this backend.  One
 *      thread per output element walks the reference's loop nest with a float64 accumulator:
 *      results are bit-identical to MathBackendCPU.  Dilation must be 1 (the op layer asserts
 *      the same, ops/conv.ts:188-192).
 * KernelBackend.conv2dDerInput / conv2dDerFilter (backend.ts:424-429; CPU :1686-1762, 1849-1898):
 * dx [B,inH,inW,Cin] from dy [B,outH,outW,Cout] and filter; dW [fH,fW,Cin,Cout] from x and dy. */
int tfjs_cuda_conv2d_der_input(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy, tfjs_tensor_id filter,
                               tfjs_tensor_id dx, const tfjs_conv2d_info* info);
int tfjs_cuda_conv2d_der_filter(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id dy,
                                tfjs_tensor_id dw, const tfjs_conv2d_info* info);
/* KernelBackend.depthwiseConv2DDerInput / DerFilter (backend.ts:436-442; CPU :2037-2150). */
int tfjs_cuda_depthwise_conv2d_der_input(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy, tfjs_tensor_id filter,
                                         tfjs_tensor_id dx, const tfjs_conv2d_info* info);
int tfjs_cuda_depthwise_conv2d_der_filter(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id dy,
                                          tfjs_tensor_id dw, const tfjs_conv2d_info* info);
/* KernelBackend.maxPoolBackprop / avgPoolBackprop (backend.ts:456-466; CPU :2347-2509): dx of the
 * pooled input x given dy of the pooled output. */
int tfjs_cuda_pool2d_backprop(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy, tfjs_tensor_id x, tfjs_tensor_id dx,
                              const tfjs_conv2d_info* info, int is_avg);
/* Gradient of clipByValue (ops/unary_ops.ts:456-462) as one kernel: out = dy where
 * lo <= x <= hi, else 0 (the reference composes greaterEqual, lessEqual, logicalAnd, where). */
int tfjs_cuda_clip_backprop(tfjs_cuda_ctx* ctx, tfjs_tensor_id dy, tfjs_tensor_id x, tfjs_tensor_id out,
                            float lo, float hi);
/* KernelBackend.transpose (backend.ts:216; the op layer uses it to move reduced axes inner-most,
 * ops/reduction_ops.ts:115-121): out[i0..] = x permuted; `shape` is x's shape. */
int tfjs_cuda_transpose(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id out, int rank,
                        const int64_t* shape, const int32_t* perm);
/* KernelBackend.avgPool / maxPool (backend.ts:453-462; CPU :2273-2343, 2869-2873). */
int tfjs_cuda_pool2d(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id out,
                     const tfjs_conv2d_info* info, int is_avg);
/* KernelBackend.add / subtract / multiply / realDivide / prelu / notEqual (backend.ts:164-178,
 * 329-331; CPU broadcastedBinaryOp :3515-3549).  Shapes follow broadcast_util.ts:58-87; out
 * must be registered with the broadcast shape. */
int tfjs_cuda_binary(tfjs_cuda_ctx* ctx, int op, tfjs_tensor_id a, int a_rank,
                     const int64_t* a_shape, tfjs_tensor_id b, int b_rank, const int64_t* b_shape,
                     tfjs_tensor_id out);
/* KernelBackend.relu / clip / exp / log / int / step (backend.ts:300-346, 401; CPU :1094-1275,
 * 1520-1534). */
int tfjs_cuda_unary(tfjs_cuda_ctx* ctx, int op, tfjs_tensor_id x, tfjs_tensor_id out, float p0,
                    float p1);
/* KernelBackend.sum / max / argMax over the inner-most axes (backend.ts:183, 198, 255;
 * CPU :590-611, 686-712, 906-929): x viewed as [outer, inner]. */
int tfjs_cuda_reduce_last(tfjs_cuda_ctx* ctx, int op, tfjs_tensor_id x, tfjs_tensor_id out,
                          int64_t outer, int64_t inner);
/* Extension: tf.softmax over the last axis as one kernel, with the stage-by-stage float32
 * rounding of the op-layer chain (ops/softmax.ts:57-63, ops/reduction_ops.ts:56-73). */
int tfjs_cuda_softmax_last(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id out, int64_t outer,
                           int64_t inner);
/* KernelBackend.cast (backend.ts:484-486; backend_util.ts:36-71) where a copy is needed:
 * converts x's stored dtype to out's dtype (float->int truncates, ->bool is != 0). */
int tfjs_cuda_cast(tfjs_cuda_ctx* ctx, tfjs_tensor_id x, tfjs_tensor_id out);

/* ---- matMul for callers that must not allocate device memory.
 * No counterpart in the reference: tfjs-core has no notion of a caller that is forbidden to
 * allocate.  out[m, n] = act(a[m, k] . b[k, n] + bias[n]) on the tensor cores, like
 * tfjs_cuda_batch_matmul with batch 1 and no transposes, but every operand is a raw device
 * pointer supplied by the caller (bias may be NULL) and the repacked copy of b that the kernel
 * needs lives in a fixed 8 MiB array inside the library instead of allocator memory, so the
 * call performs no cudaMalloc / cudaFree and touches neither the tensor table nor the buffer
 * cache.  It is meant for hosts that pre-size all device memory (serving loops, plugins that are
 * handed pointers by a framework whose pool they must not disturb).
 * Limits: n * round_up(k, 4) <= 1 048 576 (e.g. 1024 x 1024); k and n multiples of 4, n >= 8;
 * a and out 16-byte aligned; activation linear, relu or clip.  Larger or other shapes are
 * rejected with an error message, never truncated.
 * All calls on one device share the array (each call overwrites all of it that it reads, so
 * nothing needs clearing): calls that overlap on the GPU race and must be serialised by the
 * caller.  The first call on a device resolves the array's address; make it before any stream
 * capture.  Arithmetic follows the context's "math_mode" option; work is enqueued on the
 * context's stream. */
int tfjs_cuda_matmul_static_scratch(tfjs_cuda_ctx* ctx, const float* a, const float* b,
                                    const float* bias, float* out, int64_t m, int64_t k, int64_t n,
                                    int activation, float clip_lo, float clip_hi);

/* ---- extension: CUDA-graph capture of a sequence of calls on the context.
 * Between begin and end, kernel calls are recorded instead of run.  Tensors disposed during
 * the capture keep their buffers inside the graph (replays write to them) until
 * graph_destroy; tensors created during the capture and still alive at graph_end (the
 * outputs) are rewritten by every replay and must not be disposed before the graph is.
 * tensor_read and ctx_sync are rejected while capturing. */
int tfjs_cuda_graph_begin(tfjs_cuda_ctx* ctx);
int tfjs_cuda_graph_end(tfjs_cuda_ctx* ctx, tfjs_cuda_graph** out);
int tfjs_cuda_graph_launch(tfjs_cuda_ctx* ctx, tfjs_cuda_graph* graph);
int tfjs_cuda_graph_destroy(tfjs_cuda_ctx* ctx, tfjs_cuda_graph* graph);

#ifdef __cplusplus
}
#endif
#endif /* TFJS_CUDA_H_ */
