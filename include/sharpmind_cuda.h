/*
 * sharpmind_cuda.h -- C ABI of libsharpmind_cuda.so, a CUDA (sm_100a) backend for SharpMind's
 * quantized vec-dot / matmul hot path (GGUF Q8_0, Q4_K, Q6_K) and the fp32 ops the decoder
 * runs around it.
 *
 * Every entry point takes plain pointers and sizes, returns an smc_status (0 = ok) unless
 * stated otherwise, and never falls back to a CPU implementation.  Each declaration cites the
 * SharpMind interface it stands in for (paths relative to the SharpMind repository root).
 *
 * Conventions kept from the reference:
 *   - a weight matrix is [N = outFeatures rows, K = inFeatures], row-major by output row, in
 *     GGUF block layout; `rawWeights` is always the whole tensor;
 *   - Q8_0 rows are padded to whole 32-element blocks per row; K-quants are addressed on the
 *     flat tensor (row r starts at element r*K of the 256-element block stream);
 *   - activations are [M, K] fp32 row-major, outputs [M, N] fp32 row-major;
 *   - dtype uses SharpMind's QuantDType numbering (QuantDType.cs:2-18).
 *
 * Pointers named d_* are device pointers; `stream` is a cudaStream_t passed as void*.
 *
 * Threads and streams.  A context may be used from several host threads.  The host-pointer entry points
 * (smc_*_host), registration and lookup are serialised by the context.  The device entry points (*_dev) only
 * queue work on the caller's stream; those that keep intermediate data in buffers owned by the context
 * (smc_qmatmul_dev with SMC_ACT_Q8 or SMC_ACT_F32 for M > 1 or shapes the one-row kernel does not take, smc_qmatmul_q8_dev
 * over Q4_K at 64 rows and more, smc_qmatmul_tc_dev,
 * smc_sdpa_decode_dev, smc_argmax_dev, smc_decode_step, smc_forward_last_logits) reuse those buffers in stream
 * order: all such calls on one context must go to ONE stream (or be ordered by events).  Work that is to run
 * concurrently on several streams takes one context per stream.
 */
#ifndef SHARPMIND_CUDA_H
#define SHARPMIND_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define SMC_API __declspec(dllexport)
#else
#define SMC_API __attribute__((visibility("default")))
#endif

typedef struct smc_ctx smc_ctx;
typedef struct smc_weight smc_weight;
typedef struct smc_q8act smc_q8act;
typedef struct smc_model smc_model;

typedef enum smc_status {
    SMC_OK = 0,
    SMC_E_INVALID = 1,        /* null pointer, negative size, unknown enum value */
    SMC_E_UNSUPPORTED = 2,    /* dtype / shape / mode combination this build has no kernel for */
    SMC_E_SIZE_MISMATCH = 3,  /* byte count != GetRawTensorByteCount; mirrors the reference's guard */
    SMC_E_CUDA = 4,           /* a CUDA runtime call failed; see smc_last_error */
    SMC_E_NOT_REGISTERED = 5, /* host weight pointer unknown to smc_weight_lookup */
    SMC_E_NO_DEVICE = 6,
    SMC_E_RANGE = 7           /* token id, position or column out of range */
} smc_status;

/* QuantDType values (SharpMind.Core/Quantization/QuantDType.cs:2-18) */
enum { SMC_Q8_0 = 8, SMC_Q4_K = 12, SMC_Q6_K = 14 };

/* How a quantized matmul treats its activations. */
enum {
    SMC_ACT_F32 = 0,  /* fp32 activations x dequantised weights, fp32 accumulate (reference semantics) */
    SMC_ACT_Q8 = 1,   /* activations quantised to Q8_0 blocks on device, exact int32 block dots */
    SMC_REF_ORDER = 2 /* fp32 activations, the scalar tier's own operation order and fp64 running
                         sum: bit-identical to VecDot*_Scalar; any K; needs the raw layout kept */
};

/* smc_weight_register flags */
enum {
    SMC_W_REPACK = 1,   /* build the coalescing-friendly device layout used by the fast kernels */
    SMC_W_KEEP_RAW = 2  /* also keep the GGUF-layout copy (needed by SMC_REF_ORDER and smc_vecdot_*) */
};

/* ---- library / context ------------------------------------------------------------------ */
SMC_API int smc_version(void);
SMC_API int smc_device_count(int *count);
/* Creates a context on `device` (streams, scratch). Replaces the per-call accelerator set-up of
 * SharpMind.GPU/GPUActivationKernels.cs:15-21. */
SMC_API int smc_init(int device, smc_ctx **out);
SMC_API void smc_destroy(smc_ctx *ctx);
/* Text of the last failure on this context (a copy private to the calling thread, valid until that thread's
 * next call of this function). */
SMC_API const char *smc_last_error(smc_ctx *ctx);
/* Per-context switches.  No counterpart in the reference (its tiers are chosen by mapping keys, MappingBuilder.cs).
 *   "pdl"                   1 (default) / 0: launch kernels with programmatic dependent launch, so that a kernel's
 *                           weight prefetch overlaps its predecessor's tail, or fully serialised
 *   "gemv_slots"            ring depth per warp of the one-row matmul kernel, 2..8 (0 = built-in choice)
 *   "gemv_steps_per_stage"  steps per bulk copy of that kernel: 1, 2 or 4 (0 = built-in choice)
 *   "gemv_ctas"             CTAs in its grid (0 = built-in choice: the SMs times the CTAs per SM)
 *   "gemv_warps"            warps per CTA, 24 (one CTA per SM) or 12 (two); 0 = built-in choice by row length
 *   "gemv_prefetch_first"   stages a warp requests before the activation loads are issued, 0..8 (default 1)
 *   "gemv_pair_staging"     1 (default): for fp32 rows of 8192 elements and more the two SMs of a pair (a thread-block
 *                           cluster of two) each quantise half of the row into both shared memories; 0: every CTA
 *                           quantises the whole row; a value above 1 is the row length from which rows are shared
 *   "q8_prefill_tensor_cores"  1 (default): SMC_ACT_Q8 over Q4_K at 64 rows and more runs the tcgen05 kernel on the Q8_0
 *                           activation rows (d * q is exact in its fp16 pairs; same parity bound as the int8 kernels, other
 *                           summation order); 0: the int8 mma.sync kernels at every batch size
 *   "f32_prefill_int8_digits"  1 (default): SMC_ACT_F32 with two rows and more, where no tcgen05 kernel takes the format
 *                           or shape, splits the fp32 rows into three int8 digit planes (fp32 accuracy) and runs the int8
 *                           tensor-core kernels once per plane (the planes live in the context's scratch, like the
 *                           SMC_ACT_Q8 activations of a several-row call); 0: the CUDA-core kernel at every batch size;
 *                           a value above 1: the row count to start from
 *   "f32_one_row_digits_min_mb"  one row in SMC_ACT_F32 takes the same path when the K-quant matrix holds at least this many
 *                           MB (default 32: its three digit rows as one small batch then beat the fp32 one-row kernel);
 *                           0: never
 *   "decode_gate_in_staging_max_ffn"  one sequence per step with quantised activations: the widest FFN whose SiLU-gate is
 *                           formed while the down projection stages its activation row (default 16384); a wider one
 *                           runs the gate as a launch of its own.  Same bits either way
 *   "prompt_attention_mma"  causal attention of a prompt chunk: 1 (default) bf16 tensor-core MMAs on operands split three
 *                           ways (fp32-grade accuracy), 0 the fp32 CUDA-core kernel
 *   "prompt_attention_heads_per_cta"  0 (default): a CTA of that kernel takes two query heads that share a KV head where
 *                           the model has them; 1: always one
 *   "small_batch_ring"      2..32 rows in SMC_ACT_Q8: weights through the bulk-copy ring for 1 Q4_K, 2 every format,
 *                           0 (default) never (then the kernel that fetches its fragments from global memory runs; the
 *                           two add a row's blocks in different orders: results agree within the mode's bound, not
 *                           bit for bit)
 * Results do not depend on any of them.  SMC_E_INVALID for an unknown name. */
SMC_API int smc_set_option(smc_ctx *ctx, const char *name, int value);
/* QuantizationOps.GetRawTensorByteCount for a [N, K] tensor (QuantizationOps.cs:15-72); -1 if dtype unknown. */
SMC_API int64_t smc_raw_tensor_bytes(int dtype, int64_t N, int64_t K);
/* Waits for the device, then reports whether any kernel of this context gave up a bounded wait since
 * the last call (0 = none; the flag is cleared).  No counterpart in the reference: its kernels are
 * synchronous CPU code (QuantizationKernels.cs), so it has no asynchronous failures to surface. */
SMC_API int smc_device_status(smc_ctx *ctx, int *status);
/* Blocks until everything queued on the context's own stream has finished. */
SMC_API int smc_synchronize(smc_ctx *ctx);
/* Device memory for hosts without a CUDA runtime binding of their own (the C# backend assembly; SharpMind.GPU gets its
 * buffers from ILGPU's Accelerator.Allocate1D, GPUActivationKernels.cs:10-20): allocations on the context's device,
 * and copies ordered on `stream` (null = the context's stream) that have completed when the call returns. */
SMC_API int smc_dev_alloc(smc_ctx *ctx, size_t bytes, void **d_out);
SMC_API int smc_dev_free(smc_ctx *ctx, void *d_ptr);
SMC_API int smc_copy_to_device(smc_ctx *ctx, void *d_dst, const void *host_src, size_t bytes, void *stream);
SMC_API int smc_copy_to_host(smc_ctx *ctx, void *host_dst, const void *d_src, size_t bytes, void *stream);

/* ---- weights: uploaded once ---------------------------------------------------------------
 * InferenceLinearLayer.SetRawWeight (SharpMind.Model/Layers/InferenceLinearLayer.cs:200-221)
 * validates the byte count on arrival; registration does the same and returns
 * SMC_E_SIZE_MISMATCH.  The library copies the bytes; the caller keeps ownership of host_raw. */
SMC_API int smc_weight_register(smc_ctx *ctx, const void *host_raw, size_t bytes, int dtype, int N, int K,
                                int flags, smc_weight **out);
/* Same, the GGUF-layout bytes already being in device memory (copied, not adopted). */
SMC_API int smc_weight_register_dev(smc_ctx *ctx, const void *d_raw, size_t bytes, int dtype, int N, int K,
                                    int flags, smc_weight **out);
/* Finds the registration made from this host pointer, so that slots that only receive
 * `byte* rawWeights` (QuantizedMatMulFn, QuantizationOps.cs:9) can reach the device copy. */
SMC_API int smc_weight_lookup(smc_ctx *ctx, const void *host_raw, smc_weight **out);
SMC_API int smc_weight_release(smc_ctx *ctx, smc_weight *w);
SMC_API int smc_weight_shape(const smc_weight *w, int *dtype, int *N, int *K);

/* ---- slot-shaped entry points: host pointers in, host results out, synchronous -------------
 * QuantizedMatMulFn(float* input, byte* rawWeights, float* output, int M, int K, int N)
 * (QuantizationOps.cs:9; the `linear` slot InferenceLinearLayer.cs:146 and the `logit` slot
 * LogitOps.cs:143).  host_raw must have been registered. */
SMC_API int smc_qmatmul_host(smc_ctx *ctx, const float *input, const void *host_raw, float *output, int M,
                             int K, int N, int dtype, int mode);
/* Page-locks `bytes` of host memory at `ptr` (cudaHostRegister) so that the host entry points copy from / to it directly,
 * and releases it again: for hosts that do not link the CUDA runtime themselves (a .NET host pins its float[] with a
 * GCHandle and registers the address once; unregister before the handle is freed).  The memory must stay allocated
 * and must not move while registered. */
SMC_API int smc_host_register(smc_ctx *ctx, void *ptr, size_t bytes);
SMC_API int smc_host_unregister(smc_ctx *ctx, void *ptr);
/* The same slot for a caller that kept the handle registration returned (an InferenceLinearLayer that registers in
 * SetRawWeight, InferenceLinearLayer.cs:200-221, and stores the handle next to RawQuantizedData): no pointer lookup,
 * and weights that never had a host copy (registered from device memory) can be used.  M, K, N as in
 * QuantizedMatMulFn; K and N are checked against the handle (SMC_E_SIZE_MISMATCH).
 * Both host entry points copy from and to page-locked caller memory (cudaHostAlloc / cudaHostRegister; in .NET a
 * pinned, registered array) directly; pageable buffers go through the context's own pinned bounce buffer, which
 * costs a host memcpy each way. */
SMC_API int smc_qmatmul_host_w(smc_ctx *ctx, const float *input, const smc_weight *w, float *output, int M, int K,
                               int N, int mode);
/* VecDotFn(float* input, byte* rawWeights, int col, int inFeatures) (QuantizationOps.cs:8,176-202). */
SMC_API int smc_vecdot_host(smc_ctx *ctx, const float *input, const void *host_raw, int col, int K,
                            int dtype, float *result);
/* ApplyGate(gate, up, dst) = SwiGLU (ActivationOps.cs:52-62, ActivationKernels.cs:194-201). */
SMC_API int smc_swiglu_host(smc_ctx *ctx, const float *gate, const float *up, float *dst, int n);
/* ApplyPointwise(src, dst) = SiLU (ActivationOps.cs:36-46, ActivationKernels.cs:161-168). */
SMC_API int smc_silu_host(smc_ctx *ctx, const float *src, float *dst, int n);
/* ApplySoftmaxRow(src, dst) (ActivationOps.cs:68-72, ActivationKernels.cs:316-348). */
SMC_API int smc_softmax_row_host(smc_ctx *ctx, const float *src, float *dst, int n);
/* ApplyRMSNormRow(src, weight, dst, rmsInv) (ActivationOps.cs:78-86, NormKernels.cs:13-33). */
SMC_API int smc_rmsnorm_row_host(smc_ctx *ctx, const float *src, const float *weight, float *dst, int n,
                                 float rms_inv);
/* ScaledDotProduct(q, k, v, o, seqLen, kvLen, headDim, scale, causal, qStride, oStride, alibiSlope)
 * (AttentionLayer.cs:239-258; flash form AttentionKernels.cs:409-475). k and v are [kvLen, headDim]. */
SMC_API int smc_sdpa_host(smc_ctx *ctx, const float *q, const float *k, const float *v, float *o, int seqLen,
                          int kvLen, int headDim, float scale, int causal, int qStride, int oStride,
                          float alibiSlope);

/* ---- device-resident entry points (asynchronous on `stream`) ------------------------------- */
/* out[M, N] = in[M, K] x W^T.  QuantizedMatMul*_Parallel_* (e.g. QuantizationKernels.Q8.cs:556-574). */
SMC_API int smc_qmatmul_dev(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M, int mode,
                            void *stream);

/* LinearLayer.AddBiasInPlace (SharpMind.Model/Layers/Linearlayer.cs:154-163): d_out[r, j] += d_bias[j] for every row. */
SMC_API int smc_add_bias_dev(smc_ctx *ctx, float *d_out, const float *d_bias, int rows, int n, void *stream);
/* InferenceLinearLayer.Forward (SharpMind.Model/Layers/InferenceLinearLayer.cs:148-190): the matmul of smc_qmatmul_dev
 * followed, when d_bias is not null, by the bias add. */
SMC_API int smc_linear_dev(smc_ctx *ctx, const float *d_in, const smc_weight *w, const float *d_bias, float *d_out, int M,
                           int mode, void *stream);

/* Q8_0 activation buffers: the device form of QuantizedKVCache.QuantizeRowQ8_0
 * (SharpMind.Model/QuantizedKVCache.cs:191-223): d = amax/127 (1 for an all-zero block), stored as
 * fp16 (round to nearest even), q = round-half-even(x/d). */
SMC_API int smc_q8act_create(smc_ctx *ctx, int max_rows, int max_k, smc_q8act **out);
SMC_API int smc_q8act_destroy(smc_ctx *ctx, smc_q8act *a);
SMC_API int smc_quantize_q8_dev(smc_ctx *ctx, const float *d_x, int M, int K, smc_q8act *a, void *stream);
/* Copies the quantised rows back to the host: q [M, K] int8, d_bits [M, K/32] fp16 bit patterns. */
/* FfnKernels.Gated's activation and the row quantiser in one pass: a = Q8_0(SiLU(gate) * up), gate and up being `rows`
 * rows of `ld` floats of which the first F are used (ld = 2 F for a joined gate||up output); the fp32 product is not
 * written.  Same bits as smc_swiglu_dev followed by smc_quantize_q8_dev.  F % 32 == 0. */
SMC_API int smc_swiglu_quantize_q8_dev(smc_ctx *ctx, const float *d_gate, const float *d_up, int rows, int F, int ld, smc_q8act *a,
                                       void *stream);
SMC_API int smc_q8act_read(smc_ctx *ctx, const smc_q8act *a, int8_t *q, uint16_t *d_bits);
/* The same product for prefill-sized M on the tensor cores (tcgen05 MMA, accumulators in tensor memory):
 * Q4_K weights with N % 128 == 0 and K % 256 == 0; the integer part of each weight is exact in fp16 and the
 * activations travel as an fp16 (hi, lo) pair, so the result meets the bound of SMC_ACT_F32.  This is what
 * the M > 1 row loop of QuantizedMatMulQ4K_Parallel_* (QuantizationKernels.Q4.cs:1148-1212) becomes when the
 * whole token batch shares one pass over the weights.  SMC_E_UNSUPPORTED for other formats / shapes.  The
 * first call of a larger M * K allocates scratch in the context (make it outside stream capture). */
SMC_API int smc_qmatmul_tc_dev(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M, void *stream);
/* Matmul on activations already quantised with smc_quantize_q8_dev. */
SMC_API int smc_qmatmul_q8_dev(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *d_out, void *stream);
/* The SMC_ACT_Q8 matmul of smc_qmatmul_dev for hosts that must not allocate device memory while they run
 * (all GPU memory budgeted at start-up, no tolerance for the device-wide synchronisation of cudaMalloc, or
 * an embedding application that forbids allocation after initialisation).  The quantised activations go
 * into a fixed buffer inside the library image instead of the context's growable scratch; no allocation
 * routine is called.  Limit: M * K <= SMC_NOALLOC_MAX_ELEMS activations (SMC_E_RANGE beyond); the buffer
 * (about 0.75 MB) is resident on every GPU that loads the library until the process exits.  All calls on a
 * device share it and it keeps the previous call's contents (nothing needs clearing: every entry read is
 * written first, in stream order); calls that can overlap on one GPU race and must be ordered by the caller.
 * The first call on a device resolves the buffer's address: make it during set-up, before any stream capture.
 * This entry point has no counterpart in the reference, whose kernels run on caller-owned host memory. */
#define SMC_NOALLOC_MAX_ELEMS 524288
SMC_API int smc_qmatmul_q8_noalloc(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M,
                                   void *stream);
/* Per-32-element-block int32 dot sums of weight rows [col0, col1) with row `m` of `a`:
 * d_sums[(c - col0) * K/32 + b].  Verification aid for the integer part of SMC_ACT_Q8. */
SMC_API int smc_block_isums_dev(smc_ctx *ctx, const smc_q8act *a, int m, const smc_weight *w, int col0, int col1,
                                int32_t *d_sums, void *stream);

/* TensorQuantizer.Quantize (TensorQuantizer.cs:80-144 Q8_0; TensorQuantizer.KQuant.cs:173-225 Q4_K,
 * :303-376 Q6_K): fp32 values -> GGUF blocks, n a multiple of the block size. */
SMC_API int smc_quantize_weights_dev(smc_ctx *ctx, int dtype, const float *d_values, int64_t n, void *d_raw,
                                     void *stream);

/* NormLayer.Forward with RmsNormLayer (NormLayer.cs:42-57, RmsNormLayer.cs:8-20, NormKernels.cs:13-60):
 * per row rmsInv = 1/sqrt(mean(x^2)+eps), out = x*rmsInv*w.  d_out may alias d_x. */
SMC_API int smc_rmsnorm_dev(smc_ctx *ctx, const float *d_x, const float *d_w, float *d_out, int rows, int n,
                            float eps, void *stream);
/* FfnKernels.Gated's activation loop (Ffn/FfnKernels.cs:52-56): rows of gate/up with row stride `ld`
 * (ld = 2F and d_up = d_gate + F for the fused gate||up buffer), dst [rows, F] dense. */
SMC_API int smc_swiglu_dev(smc_ctx *ctx, const float *d_gate, const float *d_up, float *d_dst, int rows, int F,
                           int ld, void *stream);
SMC_API int smc_silu_dev(smc_ctx *ctx, const float *d_src, float *d_dst, int64_t n, void *stream);
/* ActivationOps.Softmax row-wise (ActivationOps.cs:118-132). */
SMC_API int smc_softmax_dev(smc_ctx *ctx, const float *d_src, float *d_dst, int rows, int n, void *stream);
/* RoPE table build (SharpMind.Core/Embeddings/RoPE.cs:103-147, no frequency scaling): computed on the
 * host with the same libm calls as the reference's MathF and uploaded; d_cos/d_sin [maxSeq, ropeDim/2]. */
SMC_API int smc_rope_tables(smc_ctx *ctx, float theta, int ropeDim, int maxSeq, float *d_cos, float *d_sin);
/* RoPE.Apply (RoPE.cs:168-259) in place on x [seq, heads, headDim]; neox != 0 pairs (d, d+ropeDim/2). */
SMC_API int smc_rope_dev(smc_ctx *ctx, float *d_x, int seq, int heads, int headDim, int ropeDim, int posOffset,
                         const float *d_cos, const float *d_sin, int neox, void *stream);
/* Tensor<float>.AddInPlace (SharpMind.Core/Tensors/Tensor.cs:328-332): x += y. */
SMC_API int smc_add_dev(smc_ctx *ctx, float *d_x, const float *d_y, int64_t n, void *stream);
/* The residual add and the norm that follows it in a decoder block as one pass (UnhookedTransformerBlock.Forward,
 * UnhookedTransformerBlock.cs:12-47: x.AddInPlace(attnOut); normed = norm2.Forward(x)): x += y, out = RMSNorm(x) * w.
 * Same bits as smc_add_dev followed by smc_rmsnorm_dev. */
SMC_API int smc_add_rmsnorm_dev(smc_ctx *ctx, float *d_x, const float *d_y, const float *d_w, float *d_out, int rows,
                                int n, float eps, void *stream);
/* The same pass with the normalised rows leaving as Q8_0 activations in `a` (QuantizedKVCache.QuantizeRowQ8_0's rules,
 * QuantizedKVCache.cs:191-223), ready for smc_qmatmul_q8_dev: x += y (d_y may be null: no add), a = Q8_0(RMSNorm(x) * w),
 * and d_out = the fp32 rows too when it is not null.  Between two matmuls of a block that runs several rows with
 * quantised activations the fp32 rows are read by nothing else.  Same bits as smc_add_rmsnorm_dev (or smc_rmsnorm_dev)
 * followed by smc_quantize_q8_dev.  n % 32 == 0, n > 256 and 16-byte aligned pointers, else SMC_E_UNSUPPORTED. */
SMC_API int smc_add_rmsnorm_q8_dev(smc_ctx *ctx, float *d_x, const float *d_y, const float *d_w, float *d_out, int rows,
                                   int n, float eps, smc_q8act *a, void *stream);
/* Sampler.Argmax (SharpMind.Inference/Sampler.cs:50-58) per row: first maximum wins. */
SMC_API int smc_argmax_dev(smc_ctx *ctx, const float *d_logits, int rows, int n, int *d_out, void *stream);
/* Sampler.Sample (SharpMind.Inference/Sampler.cs:16-46) per row of d_logits [rows, n]: temperature, guarded softmax,
 * min-p, top-k, top-p, normalise, one categorical draw; temperature <= 0 is the greedy shortcut (Sampler.Argmax).
 * The fields are SamplingConfig's (SamplingConfig.cs: Temperature, TopK 0 = off, TopP 1 = off, MinP 0 = off).
 * d_uniform [rows] holds the number rng.NextSingle() produced for each row (the host keeps its own generator, so a
 * seeded run draws the same stream it would have drawn on the CPU); d_work [rows, n] is scratch for the
 * probabilities.  The logits are not modified.  Probabilities bit-equal to a top-k / top-p cut value are all kept,
 * and sums are formed by a fixed tree instead of the reference's sequential loops: a draw within rounding of a
 * boundary between two tokens may pick the neighbour. */
typedef struct smc_sampling {
    float temperature;
    int top_k;
    float top_p;
    float min_p;
} smc_sampling;
SMC_API int smc_sample_dev(smc_ctx *ctx, const float *d_logits, int rows, int n, const smc_sampling *cfg,
                           const float *d_uniform, float *d_work, int *d_tokens, void *stream);
/* RepetitionPenalty.Apply (SharpMind.Inference/RepetitionPenalty.cs:15-27) in place on d_logits [rows, n]: every
 * DISTINCT id of row r's window d_ids[r, 0 .. window) scales its logit once (positive: divided by the penalty,
 * negative: multiplied); ids outside [0, n) are skipped, so -1 pads a short window. */
SMC_API int smc_repetition_penalty_dev(smc_ctx *ctx, float *d_logits, int rows, int n, const int *d_ids, int window,
                                       float penalty, void *stream);
/* EmbeddingTable.Forward (SharpMind.Core/Embeddings/EmbeddingTable.cs:87-116) gathering rows of a Q8_0
 * table dequantised as ReadQ8_0_Scalar does (QuantizationKernels.Q8.cs:412-433): out[i] = row tokens[i]. */
SMC_API int smc_embed_q8_0_dev(smc_ctx *ctx, const smc_weight *table, const int *d_tokens, int count, float *d_out,
                               void *stream);
/* One query token per sequence against an fp32 KV cache laid out as KVCache does
 * (SharpMind.Model/KVCache.cs:13-14,26-36): [batch, kvHeads, maxSeq, headDim]; q and out are
 * [batch, heads, headDim]; causal with the query at position kvLen-1.  Computes what
 * ScaledDotProductFlash* computes per (batch, head) (AttentionKernels.cs:315-475). */
SMC_API int smc_sdpa_decode_dev(smc_ctx *ctx, const float *d_q, const float *d_k, const float *d_v, float *d_out,
                                int batch, int heads, int kvHeads, int headDim, int kvLen, int maxSeq, float scale,
                                void *stream);
/* KVCache.Update for seqLen == 1 (KVCache.cs:84-150): writes k, v [batch, kvHeads, headDim] at `pos`. */
SMC_API int smc_kv_append_dev(smc_ctx *ctx, const float *d_k, const float *d_v, float *d_kcache, float *d_vcache,
                              int batch, int kvHeads, int headDim, int pos, int maxSeq, void *stream);

/* ---- KV cache objects -----------------------------------------------------------------------
 * IKVCache (SharpMind.Model/IKVCache.cs:7-18) on the device: KVCache (fp32, KVCache.cs) and QuantizedKVCache with Q8_0
 * rows (QuantizedKVCache.cs).  One object holds the keys and values of one attention layer for `batch` lock-step
 * sequences that share one position (CurrentPosition), as the reference's caches do.  Host-side state (the length)
 * changes when the call returns; device work is queued on `stream`, so calls on one object go to one stream. */
typedef struct smc_kv smc_kv;
enum { SMC_KV_F32 = 0, SMC_KV_Q8_0 = 8 };
SMC_API int smc_kv_create(smc_ctx *ctx, int batch, int kvHeads, int maxSeq, int headDim, int kind, smc_kv **out);
SMC_API int smc_kv_destroy(smc_ctx *ctx, smc_kv *kv);
SMC_API int smc_kv_length(const smc_kv *kv);   /* IKVCache.Length */
SMC_API int smc_kv_max_seq(const smc_kv *kv);  /* IKVCache.MaxSeqLen */
SMC_API int smc_kv_reset(smc_ctx *ctx, smc_kv *kv);                 /* Reset(): length = 0 */
SMC_API int smc_kv_truncate(smc_ctx *ctx, smc_kv *kv, int length);  /* Truncate(length): length = min(length, current) */
/* TrimToLast(keep) (KVCache.cs:44-82, QuantizedKVCache.cs:128-160): the last `keep` positions move to the front. */
SMC_API int smc_kv_trim_to_last(smc_ctx *ctx, smc_kv *kv, int keep, void *stream);
/* Update(k, v) (KVCache.cs:84-150, QuantizedKVCache.cs:84-126): d_k, d_v are [batch, seqLen, kvHeads, headDim] fp32 and
 * are appended at the current length (quantised row by row for a Q8_0 cache); SMC_E_RANGE on overflow. */
SMC_API int smc_kv_update_dev(smc_ctx *ctx, smc_kv *kv, const float *d_k, const float *d_v, int batch, int seqLen, void *stream);
/* Snapshot / Restore (KVCache.cs:152-174, QuantizedKVCache.cs:162-189), synchronous, host buffers.  What is saved: the
 * positions [0, length) of EVERY (sequence, head), densely packed [batch][kvHead][length][row], a row being headDim
 * floats or headDim/32 Q8_0 blocks of 34 bytes in the reference's block layout.  (The reference copies the first
 * batch*heads*length rows of its flat array instead, which are the active rows only for a single head; its restore
 * onto the same object still works because nothing else was touched.) */
SMC_API int64_t smc_kv_snapshot_bytes(const smc_kv *kv);  /* bytes per tensor (keys and values have the same size) */
SMC_API int smc_kv_snapshot(smc_ctx *ctx, const smc_kv *kv, void *host_k, void *host_v, int64_t bytes_each, int *position);
SMC_API int smc_kv_restore(smc_ctx *ctx, smc_kv *kv, const void *host_k, const void *host_v, int64_t bytes_each, int position);
/* Causal attention of the LAST seqLen positions against the whole cache (AttentionLayer.Forward's per-(batch, head)
 * loop, AttentionLayer.cs:326-413, with ScaledDotProductFlash* for an fp32 cache, AttentionKernels.cs:315-475, and
 * ScaledDotProductFlashQ8_0* for a Q8_0 one, :489-813): d_q and d_out are [batch, seqLen, heads, headDim]; the keys and
 * values of those positions must have been appended already. */
SMC_API int smc_sdpa_kv_dev(smc_ctx *ctx, const smc_kv *kv, const float *d_q, float *d_out, int batch, int heads, int seqLen,
                            float scale, void *stream);

/* ---- one decode step of a Llama/Qwen-shaped decoder -------------------------------------------
 * What Transformer.ForwardLastLogits computes for [batch, 1] token ids (SharpMind.Model/Transformer.cs:417-463
 * -> DecoderArch.Forward Arch/DecoderArch.cs:115-134 -> UnhookedTransformerBlock.Forward
 * Layers/UnhookedTransformerBlock.cs:12-47 -> AttentionLayer.Forward Layers/Attention/AttentionLayer.cs:260-422,
 * FfnKernels.Gated Layers/Ffn/FfnKernels.cs:35-59).  Weights are handles registered beforehand; norm vectors are
 * device pointers; wgu is the fused gate||up matrix [2*ffn, hidden]; lm_head is the Q8_0 [vocab, hidden] table
 * that also serves as the embedding (tied weights, Transformer.cs:67-73). */
typedef struct smc_model_desc {
    int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq;
    float eps, rope_theta;
    int neox;     /* RoPE pairing: 1 = (d, d + headDim/2) as for qwen/gemma/phi, 0 = adjacent (AttentionLayer.cs:132-144) */
    int qk_norm;  /* per-head RMSNorm of Q and K before RoPE (Qwen3, AttentionLayer.cs:284-285) */
    const smc_weight *const *wq, *const *wk, *const *wv, *const *wo, *const *wgu, *const *wdown; /* [n_layers] */
    const float *const *norm1, *const *norm2, *const *qnorm, *const *knorm;                        /* [n_layers] */
    const float *final_norm;
    const smc_weight *lm_head;
    /* Bias vectors of the linear layers (LinearLayer._bias, added by AddBiasInPlace, Linearlayer.cs:154-163): each
     * member is null (no such biases anywhere) or an array of n_layers device pointers whose entries may be null.
     * bq [heads*headDim], bk / bv [kvHeads*headDim], bo [hidden], bgu [2*ffn], bdown [hidden]. */
    const float *const *bq, *const *bk, *const *bv, *const *bo, *const *bgu, *const *bdown;
    /* Format of the KV cache: SMC_KV_F32 (0, KVCache) or SMC_KV_Q8_0 (8, QuantizedKVCache with Q8_0 rows: a quarter of the
     * bytes a decode step sweeps).  Needs the joined Q/K/V path and headDim 64 or 128. */
    int kv_dtype;
} smc_model_desc;
/* Allocates the fp32 KV cache [layer, max_batch, kvHeads, max_seq, headDim] (KVCache.cs:13-14), RoPE tables
 * and intermediates.  The description's arrays are copied; the weights stay owned by the context. */
SMC_API int smc_model_create(smc_ctx *ctx, const smc_model_desc *desc, int max_batch, smc_model **out);
SMC_API int smc_model_destroy(smc_ctx *ctx, smc_model *m);
/* Device pointers of the K and V caches, e.g. to install a prefilled context. */
SMC_API int smc_model_kv(smc_ctx *ctx, smc_model *m, float **d_k, float **d_v);
/* Installs a context: d_k / d_v are dense [layers, batch, kvHeads, len, headDim] fp32 and become positions
 * [0, len) of the cache (what `len` calls of KVCache.Update would have left, KVCache.cs:84-150). */
SMC_API int smc_model_kv_load(smc_ctx *ctx, smc_model *m, const float *d_k, const float *d_v, int batch, int len,
                              void *stream);
/* Runs the step for `batch` lock-step sequences whose new token sits at position `pos` (the cache already
 * holds positions [0, pos)), writes logits [batch, vocab] and, if d_argmax is not null, the greedy token per
 * sequence (Sampler.Argmax, Sampler.cs:50-58).  `mode` is one of SMC_ACT_F32 / SMC_ACT_Q8 / SMC_REF_ORDER. */
SMC_API int smc_decode_step(smc_ctx *ctx, smc_model *m, const int *d_tokens, int batch, int pos, int mode,
                            float *d_logits, int *d_argmax, void *stream);

/* Transformer.ForwardLastLogits with seqLen > 1 (prompt processing; SharpMind.Model/Transformer.cs, block order
 * UnhookedTransformerBlock.cs:12-47, causal attention AttentionKernels.cs:315-475 with queryBase = kvLen - seqLen):
 * `seqLen` consecutive tokens of ONE sequence (cache slot `seq`) at positions pos .. pos + seqLen - 1.  Their K and
 * V are appended to the cache, every token attends causally to positions 0 .. its own, and d_logits [vocab] /
 * d_argmax [1] receive the LAST token's logits and greedy pick.  Prompts longer than a caller wants to hold in
 * scratch are fed in chunks (pos advancing); the first call of a longer chunk grows the activation scratch
 * (after a device-wide synchronisation), so make it outside stream capture, and re-capture any CUDA graph of
 * smc_decode_step recorded on this model before that call: it still points at the old buffers.  Needs the joined Q/K/V path (one weight format per layer, headDim 64 or 128);
 * SMC_E_UNSUPPORTED otherwise, SMC_E_RANGE past the cache (KVCache.cs:89-91). */
SMC_API int smc_forward_last_logits(smc_ctx *ctx, smc_model *model, const int *d_tokens, int seqLen, int seq, int pos,
                                    int mode, float *d_logits, int *d_argmax, void *stream);

/* Transformer.Forward over `seqLen` tokens of one sequence (the K + 1 draft tokens of a verification round,
 * MedusaGenerator.cs:247-260): as smc_forward_last_logits, but d_logits is [seqLen, vocab] (row i predicts the token
 * after token i), d_argmax [seqLen] the greedy pick per row, and d_hidden (may be null) [seqLen, hidden] receives the
 * final-normed hidden states.  The model's cache keeps no length of its own: IKVCache.Truncate(n) after a rejected draft
 * (MedusaGenerator.cs:394-398, SpeculativeGenerator's Restore) is the caller passing pos = n on its next call; rows past
 * it are never read and are overwritten by the next append. */
SMC_API int smc_forward_logits(smc_ctx *ctx, smc_model *model, const int *d_tokens, int seqLen, int seq, int pos, int mode,
                               float *d_logits, int *d_argmax, float *d_hidden, void *stream);
/* The acceptance rule of a verification round (MedusaGenerator.cs:262-283): d_draft [heads + 1] holds the model's own
 * greedy token followed by the heads' guesses, d_argmax [heads + 1] the greedy pick after each of them;
 * *d_accepted = 1 + the longest prefix i < heads with d_argmax[i] == d_draft[i + 1]. */
SMC_API int smc_verify_greedy_dev(smc_ctx *ctx, const int *d_argmax, const int *d_draft, int heads, int *d_accepted, void *stream);
/* MedusaHeads.Predict on a Q8_0 head (MedusaHeads.cs:64-130): head h maps the normed hidden state through
 * h' = SiLU(hidden W_h + b_h) (d_head_w [k][hidden][hidden] fp32 with W[j * hidden + i], d_head_b [k][hidden]) and the
 * shared LM head picks its token: d_tokens [k].  d_work holds k * (hidden + vocab) floats.  The head transform is summed
 * in the reference's order; the LM head runs in SMC_REF_ORDER when the weight kept its GGUF copy, else SMC_ACT_F32. */
SMC_API int smc_medusa_predict_dev(smc_ctx *ctx, const float *d_hidden, const float *d_head_w, const float *d_head_b, int k,
                                   int hidden, const smc_weight *lm_head, float *d_work, int *d_tokens, void *stream);

/* One activation row whose elementwise producer rides in the matmul's staging (SMC_ACT_Q8 arithmetic, weights that
 * the one-row bulk-copy kernel takes: registered with SMC_W_REPACK, K % 1024 == 0 for Q8_0 / K % 2048 == 0 for the
 * K-quants, K <= 8192; SMC_E_UNSUPPORTED otherwise):
 *   smc_qmatmul_swiglu_dev   out = (SiLU(gate) * up) W^T      FfnKernels.Gated (FfnKernels.cs:35-59): activation, then down
 *   smc_qmatmul_addnorm_dev  out = (RMSNorm(x + add) * w) W^T  UnhookedTransformerBlock.Forward (UnhookedTransformerBlock.cs:12-47):
 *                            residual add, norm, projection; x + add is written to d_sum when that is not null, d_add may
 *                            be null (plain norm).  The sum of squares is taken in another order than smc_rmsnorm_dev's, so
 *                            the two agree to rounding, not bit for bit. */
SMC_API int smc_qmatmul_swiglu_dev(smc_ctx *ctx, const float *d_gate, const float *d_up, const smc_weight *w, float *d_out,
                                   void *stream);
SMC_API int smc_qmatmul_addnorm_dev(smc_ctx *ctx, const float *d_x, const float *d_add, const float *d_norm_w, float eps,
                                    float *d_sum, const smc_weight *w, float *d_out, void *stream);

/* A new weight whose rows are the rows of parts[0], parts[1], ... in order (same dtype and K, all registered
 * with SMC_W_REPACK): how the decoder turns Wq / Wk / Wv into one matmul.  The parts stay valid. */
SMC_API int smc_weight_concat_rows(smc_ctx *ctx, const smc_weight *const *parts, int count, smc_weight **out);
/* The gate and up projections of a gated feed-forward block (FfnKernels.Gated, Layers/Ffn/FfnKernels.cs:35-59) woven
 * into one matrix [2 * ffn, hidden] with row 2i = gate row i and row 2i + 1 = up row i, for smc_qmatmul_swiglu_pairs_dev.
 * Both weights registered with SMC_W_REPACK, same format and shape; Q6_K rows must be whole 2048-element units. */
SMC_API int smc_weight_interleave_rows(smc_ctx *ctx, const smc_weight *gate, const smc_weight *up, smc_weight **out);
/* One activation row through an interleaved gate / up matrix with the activation in the matmul's epilogue:
 * d_act[i] = SiLU(w[2i] . x) * (w[2i + 1] . x), i < N / 2, in the arithmetic of smc_qmatmul_dev(SMC_ACT_Q8) followed by
 * smc_swiglu_dev (same bits).  The block's second matmul then stages a plain row: with the SiLU-gate in ITS staging
 * (smc_qmatmul_swiglu_dev) every SM recomputes SiLU over the whole row, which costs more than the memory it saves once
 * the row is long (6.4 us for 14 336 elements, measured).  Shapes the one-row bulk-copy kernel takes; else
 * SMC_E_UNSUPPORTED. */
SMC_API int smc_qmatmul_swiglu_pairs_dev(smc_ctx *ctx, const float *d_x, const smc_weight *w_interleaved, float *d_act, void *stream);

/* ---- GGUF files to device weights -------------------------------------------------------------
 * GgufLoader (SharpMind.Model/Format/GgufLoader.cs): LoadMeta's header parse (:124-176) and LoadSingleTensor's copy of
 * a tensor's raw bytes (:512-672), with the device as the destination: the file is memory-mapped and a tensor goes
 * from the mapping to the GPU in one registration.  dtype uses GGUF's numbering, which is QuantDType's (F32 = 0,
 * F16 = 1, Q8_0 = 8, Q4_K = 12, Q6_K = 14); dims[0] is the innermost dimension (inFeatures). */
typedef struct smc_gguf smc_gguf;
SMC_API int smc_gguf_open(smc_ctx *ctx, const char *path, smc_gguf **out);
SMC_API int smc_gguf_close(smc_ctx *ctx, smc_gguf *g);
SMC_API int smc_gguf_tensor_count(const smc_gguf *g);
/* Index of the tensor called `name`, or -1. */
SMC_API int smc_gguf_find(const smc_gguf *g, const char *name);
/* bytes = GetRawTensorByteCount(shape, dtype) (QuantizationOps.cs:15-72), -1 for a format this library does not size. */
SMC_API int smc_gguf_tensor_info(const smc_gguf *g, int index, const char **name, int *dtype, int *n_dims, int64_t *dims4,
                                 int64_t *bytes);
/* Scalar metadata (ModelMetaData.GetLong / GetFloat / GetString); SMC_E_NOT_REGISTERED / null when the key is absent. */
SMC_API int smc_gguf_meta_int(const smc_gguf *g, const char *key, int64_t *value);
SMC_API int smc_gguf_meta_float(const smc_gguf *g, const char *key, double *value);
SMC_API const char *smc_gguf_meta_string(const smc_gguf *g, const char *key);
/* Registers a Q8_0 / Q4_K / Q6_K matrix (N = dims[1], K = dims[0]) straight from the mapping; flags as for
 * smc_weight_register.  SMC_E_UNSUPPORTED for other formats. */
SMC_API int smc_gguf_register(smc_ctx *ctx, const smc_gguf *g, int index, int flags, smc_weight **out);
/* An F32 or F16 tensor (norm vectors, biases) as fp32 into device memory; `count` must be its element count. */
SMC_API int smc_gguf_read_f32(smc_ctx *ctx, const smc_gguf *g, int index, float *d_dst, int64_t count);

/* ---- row-split matmul across GPUs -----------------------------------------------------------
 * No reference counterpart: SharpMind runs one device per process (Accelerator selection in
 * SharpMind.GPU/GPUDevice.cs); these entry points exist for the sharded large-matrix configurations.
 * One process per GPU holds the rows [rank * N / world, (rank + 1) * N / world) of a matrix as an
 * ordinary registered weight.  A gather object owns this rank's receive buffer: `world` chunks of
 * `count` floats, chunk r being rank r's output slice ([M, N_local] row-major).  Peers map each other's
 * buffers through CUDA IPC: every rank exports a 64-byte handle, the host exchanges them by any means
 * (one all-gather of bytes at start-up) and calls connect with all of them in rank order.  The exchange
 * itself moves no data through the host or a collective library: the producing kernel stores its slice
 * into every peer's buffer over NVLink and returns when every peer's slice has arrived here.
 * All ranks must issue the same sequence of exchanges on an object; calls on one object must not overlap
 * (one stream).  A peer that does not show up within the wait limit (2 s unless smc_gather_set_wait_ns changed it)
 * raises smc_device_status (value 2): the kernel still ends, the context stays usable, the data of that exchange is
 * invalid.  Teardown: every rank finishes its device work and all ranks meet (a barrier of the host's choosing) BEFORE
 * any of them calls smc_gather_destroy, and likewise after a status 2 before the objects are reused or destroyed: a
 * peer's kernel may still be storing into this rank's buffer. 
 * Every rank of a world must create its object with the SAME capacity: a peer's buffer is addressed through this
 * rank's own layout. */
typedef struct smc_gather smc_gather;
#define SMC_IPC_HANDLE_BYTES 64
SMC_API int smc_gather_create(smc_ctx *ctx, int rank, int world, size_t capacity_floats, smc_gather **out);
SMC_API int smc_gather_export(smc_ctx *ctx, smc_gather *g, unsigned char *handle /* [64] */);
SMC_API int smc_gather_connect(smc_ctx *ctx, smc_gather *g, const unsigned char *handles /* [world][64] */);
/* The same for ranks that live in ONE process (one host thread per GPU, or several objects on one GPU): `all` holds the
 * `world` objects in rank order, all[rank] == g; the peers' buffers are addressed directly, no IPC handle is involved.
 * Objects on different GPUs need peer access between them enabled by the caller. */
SMC_API int smc_gather_connect_local(smc_ctx *ctx, smc_gather *g, smc_gather *const *all /* [world] */);
/* Limit of every wait of an exchange on this object, in nanoseconds (default 2 000 000 000). */
SMC_API int smc_gather_set_wait_ns(smc_ctx *ctx, smc_gather *g, unsigned long long ns);
/* Device address of the receive buffer (chunk r at d_buf + r * count for an exchange of `count` floats). */
SMC_API int smc_gather_buffer(smc_ctx *ctx, smc_gather *g, float **d_buf);
/* y_local = x W_local^T written as this rank's chunk, then exchanged; on return of the launch's completion
 * the buffer holds [world][M][N_local].  Same modes and errors as smc_qmatmul_dev. */
SMC_API int smc_qmatmul_gather_dev(smc_ctx *ctx, smc_gather *g, const float *d_in, const smc_weight *w_local, int M,
                                   int mode, void *stream);
/* A matmul split along K (tensor-parallel "down" projection: rank g holds columns [k0_g, k1_g) of every row, as a
 * registered weight [N, k1_g - k0_g], and the matching slice of the activation row): every rank computes partial sums
 * of all N outputs, the partials are exchanged, and every rank ends with dense[0 .. M*N) = sum over ranks IN RANK ORDER
 * (fp32, the same additions on every rank: all ranks hold bit-identical results; they differ from the unsplit matmul by
 * summation order only, within the mode's parity bound).  One row in SMC_ACT_Q8 runs as ONE kernel: partial sums leave
 * as packets from the lanes that finish them and the kernel's tail adds them.  d_up != null: the activation is
 * SiLU(d_in) * d_up, formed while the row is staged (the SwiGLU of a row-split gate||up stays local, so a whole FFN
 * costs one exchange).  Other shapes: matmul, gather of the partials, a small adding kernel.  The buffer needs
 * world * M * N floats.  The result is read from smc_gather_buffer. */
SMC_API int smc_qmatmul_reduce_dev(smc_ctx *ctx, smc_gather *g, const float *d_in, const float *d_up, const smc_weight *w_local,
                                   int M, int mode, void *stream);
/* Exchange alone: this rank's chunk (count floats at d_buf + rank * count) was written by earlier work on
 * `stream`. */
SMC_API int smc_gather_exchange_dev(smc_ctx *ctx, smc_gather *g, size_t count, void *stream);
SMC_API int smc_gather_destroy(smc_ctx *ctx, smc_gather *g);

#ifdef __cplusplus
}
#endif
#endif /* SHARPMIND_CUDA_H */
