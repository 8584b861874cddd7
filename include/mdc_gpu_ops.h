/*
 * C ABI of libMultiDeviceGPUOps.so: the operator kernels that graphs lowered by
 * Multi-device-model-compiler call on the GPU, written for sm_100a.
 *
 * Part 1 keeps the reference's symbols (name, argument order and meaning; the reference
 * declaration is cited beside each).  Part 2 adds entry points for the ops the encoder
 * configs need and the reference ABI cannot express (fp32 LayerNorm, padding masks, GELU,
 * bf16, pre-packed weights).  All pointers are DEVICE pointers owned by the caller unless
 * a comment says otherwise; all work is asynchronous and ordered on `stream`
 * (a cudaStream_t, spelled void* so this header needs no CUDA include).  Nothing throws
 * across this boundary; failures set the sticky status of mgpuGetLastError()
 * (mdc_gpu_runtime.h) and the call returns without launching.  There is no CPU fallback:
 * without a CUDA device every compute entry point fails with that status set.
 */
#ifndef MDC_GPU_OPS_H_
#define MDC_GPU_OPS_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *mgpu_cuda_stream_t; /* cudaStream_t */

enum { MGPU_DTYPE_F32 = 0, MGPU_DTYPE_F16 = 1, MGPU_DTYPE_BF16 = 2 };
enum { MGPU_ACT_NONE = 0, MGPU_ACT_RELU = 1, MGPU_ACT_GELU_ERF = 2, MGPU_ACT_GELU_TANH = 3 };

/* ======================= Part 1: the reference's symbols ======================= */

/* include/multi-device-model-compiler/Kernels/GPU/Ops.h:23-25, lib/Kernels/GPU/Ops.cu:59-120.
 * output[M,N] = input[M,K] . weight[K,N] + bias[N]; all row-major fp32.  Operands are
 * rounded to fp16 for the tensor cores, accumulation is fp32 (the reference asks cuBLASLt
 * for CUBLAS_COMPUTE_32F_FAST_16F, Ops.cu:74-75); bias and output stay fp32. */
void mgpuMatmul(float *input, float *weight, float *bias, float *output, int64_t M, int64_t N,
                int64_t K, mgpu_cuda_stream_t stream);

/* Ops.h:27-34 / Ops.cu:238-340 and Ops.h:36-42 / Ops.cu:342-374 (CPU twins
 * lib/Kernels/CPU/Ops.cpp:83-210).  fp32 NCHW device tensors, OIHW filter, bias [OC];
 * paddings top / left / bottom / right = PHL / PWL / PHR / PWR (all four honoured), strides
 * SH / SW, ONNX dilations DH / DW; OH / OW are the caller's output extents and must fit the
 * padded input.  output = conv(input, weight) + bias (+ postAdd if hasPostAdd) with ReLU last
 * if hasContainRelu; the filter is applied as a cross-correlation (ONNX Conv and the
 * reference's CPU path; its GPU path requests cuDNN's flipped-filter mode, Ops.cu:258).
 * Operands are rounded to fp16 for the tensor cores, accumulation is fp32.
 * mgpuPool2d: method 0 = max, 1 = average with the padding counted in the divisor.
 * Bad geometry sets the status and launches nothing. */
void mgpuConv2d(float *input, float *weight, float *bias, float *output, float *postAdd, int64_t N,
                int64_t IC, int64_t H, int64_t W, int64_t OC, int64_t KH, int64_t KW, int64_t OH,
                int64_t OW, int64_t PHL, int64_t PWL, int64_t PHR, int64_t PWR, int64_t SH,
                int64_t SW, int64_t DH, int64_t DW, bool hasPostAdd, bool hasContainRelu,
                mgpu_cuda_stream_t stream);
void mgpuPool2d(float *input, float *output, int64_t N, int64_t C, int64_t H, int64_t W, int64_t OH,
                int64_t OW, int64_t KH, int64_t KW, int64_t PHL, int64_t PWL, int64_t PHR,
                int64_t PWR, int64_t SH, int64_t SW, int64_t method, mgpu_cuda_stream_t stream);

/* Ops.h:44-49, lib/Kernels/GPU/LLM.cu:26-158.  One transformer layer, fp32 at the
 * boundary, fp16 inside.  input/output [batch, seq_len, d_model]; qkv [d_model, 3*d_model];
 * gemm_weight [d_model, d_model] + gemm_bias (attention output projection);
 * ffn1_weight [d_model, feed_forward_dim] + ffn1_bias; ffn2_weight [feed_forward_dim,
 * d_model] + ffn2_bias.  LayerNorm has gamma 1 / beta 0 and eps 1e-5 (LLM.cu:39-52), there
 * is no QKV bias and every sequence is full length.  Unlike the reference (which ignores
 * them) the three flags are honoured: norm_first selects pre-LN or post-LN, is_casual adds
 * the causal mask, is_relu selects ReLU (else exact-erf GELU). */
void mgpuLLMDecodingContextLayer(float *input, float *qkv, float *gemm_weight, float *gemm_bias,
                                 float *ffn1_weight, float *ffn1_bias, float *ffn2_weight,
                                 float *ffn2_bias, float *output, int64_t batch, int64_t seq_len,
                                 int64_t d_model, int64_t feed_forward_dim, int64_t head_num,
                                 bool norm_first, bool is_casual, bool is_relu,
                                 mgpu_cuda_stream_t stream);

/* The reference's runner calls the C++ functions gpuOpsInit() / gpuOpsDeinit()
 * (Ops.h:15-16, Ops.cu:43-55); the library exports those with C++ linkage too.  These are
 * the same calls with C linkage for FFI users.  Init is optional (first use initialises). */
int32_t mgpuOpsInit(void);
void mgpuOpsDeinit(void);

/* ======================= Part 2: additions ======================= */

/* Elementwise fp32 ops: what the compiler-generated kernels of a lowered ONNX Add / bias /
 * activation compute (generation: lib/Dialect/Device/IR/GPUOffloadingAttr.cpp:255-313; CPU
 * twin examples/add.ll:26-76).  128-bit vectorised grid-stride kernels; any n, any alignment. */
void mgpuAdd(const float *a, const float *b, float *c, int64_t n, mgpu_cuda_stream_t stream);
void mgpuBiasAdd(const float *x, const float *bias, float *y, int64_t rows, int64_t cols,
                 mgpu_cuda_stream_t stream);
void mgpuActivation(const float *x, float *y, int64_t n, int32_t act, mgpu_cuda_stream_t stream);

/* Element type conversion between MGPU_DTYPE_* buffers (replaces invokeCudaCast,
 * include/multi-device-model-compiler/Kernels/GPU/Utils.h:6-8, lib/Kernels/GPU/Utils.cu:85-103).
 * Round to nearest even. */
void mgpuCast(const void *src, int32_t src_dtype, void *dst, int32_t dst_dtype, int64_t n,
              mgpu_cuda_stream_t stream);

/* Row LayerNorm over the last dimension, fp32 in and out:
 * y = (x - mean) * rsqrt(var + eps) * gamma + beta, biased variance, statistics in fp32.
 * gamma / beta may be NULL (1 / 0).  The reference has only the half-precision template
 * mgpuLayerNorm<half> (Ops.h:57-61, lib/Kernels/GPU/LayerNorm.cu:410-436). */
void mgpuLayerNormF32(const float *x, const float *gamma, const float *beta, float *y, float eps,
                      int64_t m, int64_t n, mgpu_cuda_stream_t stream);

/* General form: x (+ residual) in io_dtype, optional sum_out = x + residual in io_dtype,
 * y in out_dtype; gamma / beta are fp32 (or NULL).  Covers mgpuLayerNorm<half> and
 * mgpuAddResidualPreLayerNorm<half> (Ops.h:63-68, LayerNorm.cu:438-465). */
void mgpuLayerNormEx(const void *x, const void *residual, const float *gamma, const float *beta,
                     void *sum_out, void *y, float eps, int64_t m, int64_t n, int32_t io_dtype,
                     int32_t out_dtype, mgpu_cuda_stream_t stream);

/* weight fp32 [K,N] row-major (the ABI layout) -> 16-bit [N, Kp] with K contiguous, Kp = K
 * rounded up to 8, zero padded: the operand layout the tensor-core Gemm reads. */
void mgpuPackWeight(const float *weight_kn, void *packed_nk, int64_t K, int64_t N, int32_t dtype,
                    mgpu_cuda_stream_t stream);

/* Tensor-core Gemm on 16-bit operands (tcgen05, fp32 accumulation in tensor memory):
 * out[M,N] = act(a[M,Kp] . w[N,Kp]^T + bias[N]) + residual[M,N].
 * a and w are `dtype` (F16 or BF16) with Kp (a multiple of 8) contiguous; bias is fp32 or
 * NULL; residual is `dtype` or NULL; out is `out_dtype`.  Generalises mgpuMatmulEx<half>
 * (Ops.h:51-55, lib/Kernels/GPU/Ops.cu:136-234), which accumulated in fp16. */
void mgpuMatmulEx16(const void *a, const void *w_nk, const float *bias, const void *residual,
                    void *out, int64_t M, int64_t N, int64_t Kp, int32_t dtype, int32_t out_dtype,
                    int32_t act, mgpu_cuda_stream_t stream);

/* Fused multi-head attention on the packed QKV Gemm output (replaces the vendored
 * FusedMHARunnerFP16v2 call at lib/Kernels/GPU/LLM.cu:79-81).
 * qkv [batch*seq_len, 3, heads, head_dim] `dtype`; out [batch*seq_len, heads*head_dim];
 * P = softmax(q.k^T / sqrt(head_dim) + mask), mask = -inf for keys >= seq_lens[b] and, if
 * causal, keys after the query.  seq_lens (int32 [batch], device) may be NULL = all full.
 * head_dim must be 64 or 128 (128 is what the reference's own layer is built for,
 * lib/Kernels/GPU/LLM.cu:18-19).  Rows of padded queries are written (finite; zeros where a whole
 * tile of 128 queries is padding) but carry no meaning; the qkv rows of padded positions are
 * read (their scores are masked) and must hold finite values. */
void mgpuAttention(const void *qkv, const int32_t *seq_lens, void *out, int64_t batch,
                   int64_t seq_len, int64_t heads, int64_t head_dim, bool causal, int32_t dtype,
                   mgpu_cuda_stream_t stream);

/* Encoder stack with weights packed once.  Create returns an opaque handle (NULL on
 * failure).  SetLayer reads fp32 device weights in the layout of
 * mgpuLLMDecodingContextLayer plus optional QKV bias and LayerNorm affine parameters
 * (NULL = absent / identity) and stores 16-bit packed copies inside the handle.  Run
 * executes all layers on x [batch, seq_len, d_model] fp32 -> y fp32; seq_lens as in
 * mgpuAttention.  Scratch comes from the runtime's device pool. */
void *mgpuEncoderStackCreate(int64_t num_layers, int64_t d_model, int64_t feed_forward_dim,
                             int64_t head_num, bool norm_first, bool causal, int32_t act,
                             int32_t dtype, float eps);
void mgpuEncoderStackSetLayer(void *stack, int64_t layer, const float *qkv_weight,
                              const float *qkv_bias, const float *proj_weight,
                              const float *proj_bias, const float *ffn1_weight,
                              const float *ffn1_bias, const float *ffn2_weight,
                              const float *ffn2_bias, const float *ln1_gamma, const float *ln1_beta,
                              const float *ln2_gamma, const float *ln2_beta,
                              mgpu_cuda_stream_t stream);
void mgpuEncoderStackRun(void *stack, const float *x, const int32_t *seq_lens, float *y,
                         int64_t batch, int64_t seq_len, mgpu_cuda_stream_t stream);
void mgpuEncoderStackDestroy(void *stack);

/* Host-buffer form of Run: x and y are HOST pointers (pinned for full speed).  The batch
 * is cut into `chunks` pieces whose upload, compute and download overlap on three
 * streams (with 3 or more chunks the first and last are batch/8 sequences, because only
 * their copies are exposed); returns after y is complete.  seq_lens is a host pointer (or
 * NULL). */
void mgpuEncoderStackRunHost(void *stack, const float *x_host, const int32_t *seq_lens_host,
                             float *y_host, int64_t batch, int64_t seq_len, int32_t chunks);

/* Pipelined form for a stream of batches (no counterpart in the reference).  Submit queues
 * upload, stack and download of one whole batch on three streams and returns a ticket at once;
 * consecutive submissions alternate between two sets of device IO buffers, so batch i+1 uploads
 * while batch i computes and batch i-1 downloads.  x_host / seq_lens_host must stay unchanged
 * and y_host untouched until WaitHost(ticket) returns; at most two submissions may be waiting
 * (a third Submit simply queues behind the first's download).  Returns -1 on failure. */
int64_t mgpuEncoderStackSubmitHost(void *stack, const float *x_host, const int32_t *seq_lens_host,
                                   float *y_host, int64_t batch, int64_t seq_len);
void mgpuEncoderStackWaitHost(void *stack, int64_t ticket);

/* One post-/pre-LN encoder layer in a single call: the argument list of
 * mgpuLLMDecodingContextLayer extended by what the encoder configs need. */
void mgpuTransformerEncoderLayer(const float *input, const float *qkv_weight, const float *qkv_bias,
                                 const float *proj_weight, const float *proj_bias,
                                 const float *ffn1_weight, const float *ffn1_bias,
                                 const float *ffn2_weight, const float *ffn2_bias,
                                 const float *ln1_gamma, const float *ln1_beta,
                                 const float *ln2_gamma, const float *ln2_beta,
                                 const int32_t *seq_lens, float *output, int64_t batch,
                                 int64_t seq_len, int64_t d_model, int64_t feed_forward_dim,
                                 int64_t head_num, bool norm_first, bool causal, int32_t act,
                                 int32_t dtype, float eps, mgpu_cuda_stream_t stream);

/* No counterpart in the reference.  mgpuMatmul for callers that must not allocate device
 * memory (a serving loop that cannot take the device-wide synchronisation of cudaMalloc, or
 * a process whose device memory is already fully reserved by another component): same
 * arguments and result as mgpuMatmul, but the two 16-bit operand copies live in a fixed
 * 16 MiB device array inside the library instead of pool memory, and no allocation call of
 * any kind is made.  Accepts 256 + roundup256(M*Kp*2) + roundup256(N*Kp*2) <= 16 MiB
 * (Kp = K rounded up to 8); anything larger is rejected with the sticky status set.  The
 * first call on a device resolves the array's address: make it before any stream capture.
 * All calls on a device share the array; calls that overlap on the GPU race on it. */
void mgpuMatmulNoAlloc(float *input, float *weight, float *bias, float *output, int64_t M,
                       int64_t N, int64_t K, mgpu_cuda_stream_t stream);

/* Number of kernels this library has launched since load (for launch accounting). */
uint64_t mgpuOpsLaunchCount(void);

/* Per-kernel timing for measurements.  Between Begin and End every kernel launch of this
 * library is bracketed by two CUDA events on its stream; End waits for them and returns,
 * per category (0 Gemm, 1 attention, 2 LayerNorm, 3 elementwise / cast), the summed
 * device time in milliseconds and the number of launches (arrays of 4; either may be NULL).
 * Not to be left on in production: the events add a little work between kernels. */
void mgpuOpsProfileBegin(void);
void mgpuOpsProfileEnd(double *ms_per_category, uint64_t *launches_per_category);
/* Alternative to mgpuOpsProfileEnd: every launch on its own, in launch order (category and
 * milliseconds); returns how many were written (at most capacity). */
int64_t mgpuOpsProfileEndSpans(int32_t *category, float *ms, int64_t capacity);

/* The tensor-core kernels bound every wait on a barrier; a kernel that gives up writes a
 * code into a device status word instead of hanging.  This call synchronises `stream`,
 * returns that word (0 = all kernels completed normally), sets the sticky status if it is
 * non-zero and clears the word. */
uint32_t mgpuOpsCheckDeviceStatus(mgpu_cuda_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MDC_GPU_OPS_H_ */
