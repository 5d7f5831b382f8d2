// C ABI: context, weight registry, dispatch of the quantized matmul, and the host-pointer
// ("slot-shaped") entry points that mirror the reference's kernel signatures.
//
// The host-pointer calls exist for API fidelity with SharpMind's JigSaw slots, which hand a kernel
// native host pointers and expect results in host memory on return
// (QuantizedMatMulFn / VecDotFn, SharpMind.Core/Quantization/QuantizationOps.cs:8-9; ApplyGate etc.,
// SharpMind.Core/Activations/ActivationOps.cs:36-86).  They stage through pinned memory, run the same
// device kernels as the *_dev entry points and synchronise.  There is no CPU compute path anywhere.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <type_traits>

#include "smc_common.cuh"

int smc_fail(smc_ctx *ctx, int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx) {
        std::lock_guard<std::mutex> lock(ctx->mu_error);
        ctx->last_error = buf;
    }
    return code;
}

namespace {

int ensure_dev(smc_ctx *ctx, float **p, size_t *cap, size_t bytes)
{
    if (bytes <= *cap) return SMC_OK;
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    size_t want = bytes + bytes / 4 + 4096;
    SMC_CUDA(ctx, cudaMalloc(p, want));
    *cap = want;
    return SMC_OK;
}

int ensure_pinned(smc_ctx *ctx, size_t bytes)
{
    if (bytes <= ctx->h_pin_cap) return SMC_OK;
    if (ctx->h_pin) cudaFreeHost(ctx->h_pin);
    ctx->h_pin = nullptr;
    ctx->h_pin_cap = 0;
    size_t want = bytes + bytes / 4 + 4096;
    SMC_CUDA(ctx, cudaMallocHost(&ctx->h_pin, want));
    ctx->h_pin_cap = want;
    return SMC_OK;
}

// Host -> device through the pinned bounce buffer (pageable source memory would otherwise make the
// copy synchronous and slow); device -> host likewise.
int h2d(smc_ctx *ctx, void *dst, const void *src, size_t bytes)
{
    int rc = ensure_pinned(ctx, bytes);
    if (rc) return rc;
    memcpy(ctx->h_pin, src, bytes);
    SMC_CUDA(ctx, cudaMemcpyAsync(dst, ctx->h_pin, bytes, cudaMemcpyHostToDevice, ctx->stream));
    // the bounce buffer is reused by the next copy: wait for this one
    SMC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return SMC_OK;
}

// Host -> device without the wait, for a call whose next use of the bounce buffer is the result copy queued behind
// its own kernel on the same stream: `pinned_bytes` (>= bytes) is reserved up front so that the buffer is not
// reallocated while this copy is in flight.
int h2d_queued(smc_ctx *ctx, void *dst, const void *src, size_t bytes, size_t pinned_bytes)
{
    int rc = ensure_pinned(ctx, pinned_bytes > bytes ? pinned_bytes : bytes);
    if (rc) return rc;
    memcpy(ctx->h_pin, src, bytes);
    SMC_CUDA(ctx, cudaMemcpyAsync(dst, ctx->h_pin, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return SMC_OK;
}

int d2h(smc_ctx *ctx, void *dst, const void *src, size_t bytes)
{
    int rc = ensure_pinned(ctx, bytes);
    if (rc) return rc;
    SMC_CUDA(ctx, cudaMemcpyAsync(ctx->h_pin, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    SMC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    memcpy(dst, ctx->h_pin, bytes);
    return SMC_OK;
}

// Page-locked host memory (cudaHostAlloc / cudaHostRegister by the caller) is copied from and to directly: no bounce
// buffer, no host memcpy.  Anything else (ordinary pageable memory, or a pointer the runtime cannot classify) is not.
// The answer for the caller's last few buffers is remembered (a layer calls with the same rows again and again, and the
// query costs about a microsecond): a stale answer only chooses the other, equally correct, way of copying.
bool host_is_pinned(smc_ctx *ctx, const void *p)
{
    for (int i = 0; i < 4; ++i)
        if (ctx->pin_seen[i] == p) return ctx->pin_is[i];
    cudaPointerAttributes at{};
    bool pinned = false;
    if (cudaPointerGetAttributes(&at, p) == cudaSuccess) pinned = at.type == cudaMemoryTypeHost;
    else cudaGetLastError();  // an unknown pointer is not an error of this call
    const int slot = ctx->pin_next++ & 3;
    ctx->pin_seen[slot] = p, ctx->pin_is[slot] = pinned;
    return pinned;
}

bool known_dtype(int dtype) { return dtype == SMC_Q8_0 || dtype == SMC_Q4_K || dtype == SMC_Q6_K; }

void free_weight(smc_weight *w)
{
    if (!w) return;
    cudaFree(w->d_raw);
    cudaFree(w->q8_qs);
    cudaFree(w->q8_d);
    cudaFree(w->q6u);
    delete w;
}

// Shared tail of the two registration entry points: w->d_raw already holds the GGUF bytes.
int finish_register(smc_ctx *ctx, smc_weight *w)
{
    const int K = w->K;
    const bool shape_ok = (w->dtype == SMC_Q8_0) ? (K % 32 == 0) : (K % 256 == 0);
    if ((w->flags & SMC_W_REPACK) && shape_ok) {
        int rc = smc_launch_repack(ctx, w, ctx->stream);
        if (rc) return rc;
        SMC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        w->fast = true;
        // Q4_K computes straight from the GGUF layout; the other formats can drop it
        if (w->dtype != SMC_Q4_K && !(w->flags & SMC_W_KEEP_RAW)) {
            cudaFree(w->d_raw);
            w->d_raw = nullptr;
        }
    }
    return SMC_OK;
}

int check_register_args(smc_ctx *ctx, const void *src, size_t bytes, int dtype, int N, int K, smc_weight **out)
{
    if (!ctx || !src || !out || N <= 0 || K <= 0) return smc_fail(ctx, SMC_E_INVALID, "weight_register: bad arguments");
    if (!known_dtype(dtype)) return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight_register: dtype %d not supported", dtype);
    int64_t expect = smc_raw_tensor_bytes(dtype, N, K);
    if ((int64_t)bytes != expect)
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH,
                        "RawQuantizedData size mismatch: dtype=%d, K=%d, N=%d, expected=%lld, actual=%zu", dtype, K, N,
                        (long long)expect, bytes);
    return SMC_OK;
}

}  // namespace

extern "C" {

int smc_version(void) { return 100; }

int smc_device_count(int *count)
{
    if (!count) return SMC_E_INVALID;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    *count = (e == cudaSuccess) ? n : 0;
    return e == cudaSuccess ? SMC_OK : SMC_E_NO_DEVICE;
}

int64_t smc_raw_tensor_bytes(int dtype, int64_t N, int64_t K)
{
    switch (dtype) {
    case SMC_Q8_0: return N * ((K + 31) / 32) * 34;
    case SMC_Q4_K: return ((N * K + 255) / 256) * 144;
    case SMC_Q6_K: return ((N * K + 255) / 256) * 210;
    default: return -1;
    }
}

int smc_init(int device, smc_ctx **out)
{
    if (!out) return SMC_E_INVALID;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return SMC_E_NO_DEVICE;
    if (device < 0 || device >= n) return SMC_E_INVALID;
    if (cudaSetDevice(device) != cudaSuccess) return SMC_E_CUDA;
    smc_ctx *ctx = new smc_ctx();
    ctx->device = device;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) ctx->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return SMC_E_CUDA;
    }
    if (cudaMalloc(&ctx->d_status, sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_status, 0, sizeof(int)) != cudaSuccess) {
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return SMC_E_CUDA;
    }
    *out = ctx;
    return SMC_OK;
}

int smc_set_option(smc_ctx *ctx, const char *name, int value)
{
    if (!ctx || !name) return smc_fail(ctx, SMC_E_INVALID, "set_option: bad arguments");
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (!strcmp(name, "pdl")) ctx->use_pdl = value != 0;
    else if (!strcmp(name, "gemv_slots")) ctx->tma_slots = value >= 2 && value <= 8 ? value : 0;
    else if (!strcmp(name, "gemv_steps_per_stage")) ctx->tma_ss = (value == 1 || value == 2 || value == 4) ? value : 0;
    else if (!strcmp(name, "gemv_ctas")) ctx->tma_ctas = value >= 1 && value <= 4096 ? value : 0;
    else if (!strcmp(name, "gemv_warps")) ctx->tma_warps = (value == 12 || value == 24) ? value : 0;
    else if (!strcmp(name, "gemv_prefetch_first")) ctx->tma_pre = value >= 0 && value <= 8 ? value : 1;
    else if (!strcmp(name, "prompt_attention_mma")) ctx->attn_mma = value ? 1 : 0;
    else if (!strcmp(name, "gemv_pair_staging")) ctx->tma_cluster = value < 0 ? 0 : value;
    else if (!strcmp(name, "q8_prefill_tensor_cores")) ctx->q8_prefill_tc = value ? 1 : 0;
    else if (!strcmp(name, "f32_prefill_int8_digits")) ctx->f32_digits = value < 0 ? 0 : value;
    else if (!strcmp(name, "f32_one_row_digits_min_mb")) ctx->f32_digits_row_mb = value < 0 ? 0 : value;
    else if (!strcmp(name, "decode_gate_in_staging_max_ffn")) ctx->ffn_fuse_max = value < 0 ? 0 : value;
    else if (!strcmp(name, "prompt_attention_heads_per_cta")) ctx->attn_hpc = value == 1 ? 1 : 0;
    else if (!strcmp(name, "small_batch_ring")) ctx->mt_ring = value >= 0 && value <= 2 ? value : 0;
    else return smc_fail(ctx, SMC_E_INVALID, "set_option: unknown option '%s'", name);
    return SMC_OK;
}

void smc_destroy(smc_ctx *ctx)
{
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto &kv : ctx->by_host) free_weight(kv.second);
    ctx->by_host.clear();
    cudaFree(ctx->d_stage_in);
    cudaFree(ctx->d_stage_out);
    cudaFree(ctx->d_stage_aux);
    cudaFree(ctx->d_attn_part);
    cudaFree(ctx->d_prefill);
    cudaFree(ctx->d_argmax);
    cudaFree(ctx->d_status);
    if (ctx->h_pin) cudaFreeHost(ctx->h_pin);
    smc_q8act_free(ctx->act);
    smc_q8act_free(ctx->digits);
    cudaFree(ctx->d_digit_out);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *smc_last_error(smc_ctx *ctx)
{
    if (!ctx) return "null context";
    // the text is copied into a per-thread buffer so that a failure on another thread cannot change it under the reader
    static thread_local std::string copy;
    std::lock_guard<std::mutex> lock(ctx->mu_error);
    copy = ctx->last_error;
    return copy.c_str();
}

int smc_device_status(smc_ctx *ctx, int *status)
{
    if (!ctx || !status) return smc_fail(ctx, SMC_E_INVALID, "device_status: bad arguments");
    SMC_CUDA(ctx, cudaDeviceSynchronize());
    SMC_CUDA(ctx, cudaMemcpy(status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status) {
        SMC_CUDA(ctx, cudaMemset(ctx->d_status, 0, sizeof(int)));
        return smc_fail(ctx, SMC_E_CUDA, "a kernel gave up a bounded wait (status %d): its outputs are invalid", *status);
    }
    return SMC_OK;
}

int smc_synchronize(smc_ctx *ctx)
{
    if (!ctx) return SMC_E_INVALID;
    SMC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return SMC_OK;
}

// Device memory for hosts that bring no CUDA runtime binding of their own (the C# assembly): plain allocations on the
// context's device; copies are ordered on `stream` (null: the context's own stream) and have completed on return.
int smc_dev_alloc(smc_ctx *ctx, size_t bytes, void **out)
{
    if (!ctx || !out || bytes == 0) return smc_fail(ctx, SMC_E_INVALID, "dev_alloc: bad arguments");
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    SMC_CUDA(ctx, cudaMalloc(out, bytes));
    return SMC_OK;
}

int smc_dev_free(smc_ctx *ctx, void *d_ptr)
{
    if (!ctx) return SMC_E_INVALID;
    if (!d_ptr) return SMC_OK;
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    SMC_CUDA(ctx, cudaFree(d_ptr));
    return SMC_OK;
}

int smc_copy_to_device(smc_ctx *ctx, void *d_dst, const void *host_src, size_t bytes, void *stream)
{
    if (!ctx || (bytes && (!d_dst || !host_src))) return smc_fail(ctx, SMC_E_INVALID, "copy_to_device: bad arguments");
    cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    SMC_CUDA(ctx, cudaMemcpyAsync(d_dst, host_src, bytes, cudaMemcpyHostToDevice, s));
    SMC_CUDA(ctx, cudaStreamSynchronize(s));
    return SMC_OK;
}

int smc_copy_to_host(smc_ctx *ctx, void *host_dst, const void *d_src, size_t bytes, void *stream)
{
    if (!ctx || (bytes && (!host_dst || !d_src))) return smc_fail(ctx, SMC_E_INVALID, "copy_to_host: bad arguments");
    cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    SMC_CUDA(ctx, cudaMemcpyAsync(host_dst, d_src, bytes, cudaMemcpyDeviceToHost, s));
    SMC_CUDA(ctx, cudaStreamSynchronize(s));
    return SMC_OK;
}

// ------------------------------------------------------------------------------------------ weights
int smc_weight_register(smc_ctx *ctx, const void *host_raw, size_t bytes, int dtype, int N, int K, int flags,
                        smc_weight **out)
{
    int rc = check_register_args(ctx, host_raw, bytes, dtype, N, K, out);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    smc_weight *w = new smc_weight();
    w->dtype = dtype, w->N = N, w->K = K, w->flags = flags, w->raw_bytes = bytes, w->host_key = host_raw;
    cudaError_t e = cudaMalloc(&w->d_raw, bytes);
    // The copy is ordered on the context's stream, where the repack kernels run: a plain cudaMemcpy from pageable
    // memory returns once the bytes are staged, with the transfer itself still in flight on the legacy stream, and
    // the context's stream does not synchronise with that one.
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->d_raw, host_raw, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        free_weight(w);
        return smc_fail(ctx, SMC_E_CUDA, "weight upload failed: %s", cudaGetErrorString(e));
    }
    rc = finish_register(ctx, w);
    if (rc) {
        free_weight(w);
        return rc;
    }
    auto it = ctx->by_host.find(host_raw);
    if (it != ctx->by_host.end()) {  // the same host buffer registered again replaces the old copy
        free_weight(it->second);
        ctx->by_host.erase(it);
    }
    ctx->by_host[host_raw] = w;
    *out = w;
    return SMC_OK;
}

int smc_weight_register_dev(smc_ctx *ctx, const void *d_raw, size_t bytes, int dtype, int N, int K, int flags,
                            smc_weight **out)
{
    int rc = check_register_args(ctx, d_raw, bytes, dtype, N, K, out);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    smc_weight *w = new smc_weight();
    w->dtype = dtype, w->N = N, w->K = K, w->flags = flags, w->raw_bytes = bytes, w->host_key = nullptr;
    cudaError_t e = cudaMalloc(&w->d_raw, bytes);
    // whatever produced the bytes (on any stream) has to be finished, and the copy has to be ordered before the
    // repack kernels on the context's stream
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->d_raw, d_raw, bytes, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        free_weight(w);
        return smc_fail(ctx, SMC_E_CUDA, "weight copy failed: %s", cudaGetErrorString(e));
    }
    rc = finish_register(ctx, w);
    if (rc) {
        free_weight(w);
        return rc;
    }
    ctx->by_host[w] = w;  // keyed by itself so that the context owns and frees it
    *out = w;
    return SMC_OK;
}

int smc_weight_lookup(smc_ctx *ctx, const void *host_raw, smc_weight **out)
{
    if (!ctx || !host_raw || !out) return smc_fail(ctx, SMC_E_INVALID, "weight_lookup: bad arguments");
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->by_host.find(host_raw);
    if (it == ctx->by_host.end())
        return smc_fail(ctx, SMC_E_NOT_REGISTERED, "no weight was registered from host pointer %p", host_raw);
    *out = it->second;
    return SMC_OK;
}

int smc_weight_release(smc_ctx *ctx, smc_weight *w)
{
    if (!ctx || !w) return smc_fail(ctx, SMC_E_INVALID, "weight_release: bad arguments");
    std::lock_guard<std::mutex> lock(ctx->mu);
    const void *key = w->host_key ? w->host_key : static_cast<const void *>(w);
    auto it = ctx->by_host.find(key);
    if (it == ctx->by_host.end() || it->second != w)
        return smc_fail(ctx, SMC_E_NOT_REGISTERED, "weight %p does not belong to this context", (void *)w);
    ctx->by_host.erase(it);
    cudaStreamSynchronize(ctx->stream);
    free_weight(w);
    return SMC_OK;
}

int smc_weight_shape(const smc_weight *w, int *dtype, int *N, int *K)
{
    if (!w) return SMC_E_INVALID;
    if (dtype) *dtype = w->dtype;
    if (N) *N = w->N;
    if (K) *K = w->K;
    return SMC_OK;
}

// ------------------------------------------------------------------------------------------ matmul
int smc_q8act_create(smc_ctx *ctx, int max_rows, int max_k, smc_q8act **out)
{
    if (!ctx || !out) return smc_fail(ctx, SMC_E_INVALID, "q8act_create: bad arguments");
    cudaSetDevice(ctx->device);
    return smc_q8act_alloc(ctx, max_rows, max_k, out);
}

int smc_q8act_destroy(smc_ctx *ctx, smc_q8act *a)
{
    if (!ctx || !a) return smc_fail(ctx, SMC_E_INVALID, "q8act_destroy: bad arguments");
    smc_q8act_free(a);
    return SMC_OK;
}

int smc_quantize_q8_dev(smc_ctx *ctx, const float *d_x, int M, int K, smc_q8act *a, void *stream)
{
    if (!ctx || !d_x || !a || M <= 0 || K <= 0) return smc_fail(ctx, SMC_E_INVALID, "quantize_q8: bad arguments");
    return smc_launch_quantize_q8(ctx, d_x, M, K, a, static_cast<cudaStream_t>(stream));
}

int smc_swiglu_quantize_q8_dev(smc_ctx *ctx, const float *d_gate, const float *d_up, int rows, int F, int ld, smc_q8act *a, void *stream)
{
    if (!ctx || !d_gate || !d_up || !a || rows <= 0 || F <= 0 || ld < F) return smc_fail(ctx, SMC_E_INVALID, "swiglu_quantize_q8: bad arguments");
    return smc_launch_swiglu_quantize_q8(ctx, d_gate, d_up, rows, F, ld, a, static_cast<cudaStream_t>(stream));
}

int smc_q8act_read(smc_ctx *ctx, const smc_q8act *a, int8_t *q, uint16_t *d_bits)
{
    if (!ctx || !a || a->M <= 0) return smc_fail(ctx, SMC_E_INVALID, "q8act_read: buffer holds no rows");
    SMC_CUDA(ctx, cudaDeviceSynchronize());
    size_t n = (size_t)a->M * a->K;
    if (q) SMC_CUDA(ctx, cudaMemcpy(q, a->q, n, cudaMemcpyDeviceToHost));
    if (d_bits) SMC_CUDA(ctx, cudaMemcpy(d_bits, a->dbits, n / 32 * sizeof(uint16_t), cudaMemcpyDeviceToHost));
    return SMC_OK;
}

int smc_qmatmul_q8_dev(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *d_out, void *stream)
{
    if (!ctx || !a || !w || !d_out) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_q8: bad arguments");
    if (a->K != w->K) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_q8: activations have K=%d, weight has K=%d", a->K, w->K);
    if (!w->fast)
        return smc_fail(ctx, SMC_E_UNSUPPORTED,
                        "quantised-activation matmul needs a weight registered with SMC_W_REPACK and K %% %d == 0",
                        w->dtype == SMC_Q8_0 ? 32 : 256);
    // prefill-sized batches over Q4_K: the quantised rows go through the tcgen05 kernel (their values d * q are exact in
    // its fp16 pairs), three times the rate of the int8 mma.sync kernels; same parity bound, not the same bits as a
    // small batch (the products are the same, their fp32 summation is not)
    if (ctx->q8_prefill_tc && a->M >= 64 && smc_prefill_supported(w, a->M))
        return smc_launch_prefill_q4k_q8(ctx, a, w, d_out, static_cast<cudaStream_t>(stream));
    return smc_launch_gemv_q8(ctx, a, w, d_out, static_cast<cudaStream_t>(stream));
}

// SMC_ACT_F32 at prefill sizes over a format without a tcgen05 kernel: the fp32 rows become three int8 digit planes
// (x = d1 q1 + d2 q2 + d3 q3 to 6e-8 of a block's largest value), each plane goes through the integer tensor-core
// kernels and the three products are added, smallest last.  Three passes of the int8 kernels instead of M / 8 passes
// of the CUDA-core kernel over the weights; same parity bound as that kernel (tested), other bits.
static int qmatmul_f32_digits(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M, cudaStream_t s)
{
    std::lock_guard<std::mutex> lock(ctx->mu_scratch);  // held until everything is queued, like the Q8 scratch
    int rc;
    smc_q8act *&a = ctx->digits;
    const size_t need = (size_t)3 * M * w->K;
    if (!a || ctx->digits_cap < need) {
        if (a) {  // growing allocates: make the first call of a new size outside stream capture
            cudaDeviceSynchronize();
            smc_q8act_free(a);
            a = nullptr;
            ctx->digits_cap = 0;
        }
        if ((rc = smc_q8act_alloc(ctx, 3 * M, w->K, &a))) return rc;
        ctx->digits_cap = need;
    }
    a->max_rows = (int)(ctx->digits_cap / w->K), a->max_k = w->K;  // the same allocation (digits_cap values), seen with this K
    const size_t out_bytes = (size_t)3 * M * w->N * sizeof(float);
    if (ctx->digit_out_cap < out_bytes) {
        if (ctx->d_digit_out) {
            cudaDeviceSynchronize();
            cudaFree(ctx->d_digit_out);
            ctx->d_digit_out = nullptr, ctx->digit_out_cap = 0;
        }
        SMC_CUDA(ctx, cudaMalloc(&ctx->d_digit_out, out_bytes));
        ctx->digit_out_cap = out_bytes;
    }
    // the planes are 3 M rows of one batch: the weights are read once for all three
    if ((rc = smc_launch_quantize_q8_digits(ctx, d_in, M, w->K, a, s))) return rc;
    if ((rc = smc_launch_gemv_q8(ctx, a, w, ctx->d_digit_out, s))) return rc;
    return smc_launch_sum3(ctx, ctx->d_digit_out, d_out, (long long)M * w->N, s);
}

// `gd` (row-split across GPUs): when the one-row TMA kernel runs, it also exchanges the output slice with the
// peers and *fused is set; otherwise the caller launches the exchange after this returns.
static int qmatmul_impl(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M, int mode,
                        cudaStream_t s, const smc_gather_dev *gd = nullptr, bool *fused = nullptr)
{
    switch (mode) {
    case SMC_REF_ORDER: return smc_launch_gemv_ref(ctx, d_in, w, d_out, M, 0, w->N, s);
    case SMC_ACT_F32:
        // prefill-sized batches of Q4_K run on the tcgen05 tensor cores (same parity bound, see smc_prefill.cu)
        if (M >= 64 && smc_prefill_supported(w, M) && (reinterpret_cast<uintptr_t>(d_in) & 15) == 0)
            return smc_launch_prefill_q4k(ctx, d_in, w, d_out, M, s);
        if (ctx->f32_digits && M >= (ctx->f32_digits > 1 ? ctx->f32_digits : 2) && w->fast && (reinterpret_cast<uintptr_t>(d_in) & 15) == 0)
            return qmatmul_f32_digits(ctx, d_in, w, d_out, M, s);
        // one row over a large matrix: its three digit rows through the several-row integer kernel beat the fp32 one-row kernel
        // (from about 32 MB on for the K-quants: 28672 x 4096 Q4_K 66 -> 32 us, 57344 x 8192 249 -> 98 us; small matrices are
        // launch-bound)
        if (M == 1 && ctx->f32_digits && ctx->f32_digits_row_mb > 0 && w->dtype != SMC_Q8_0 && w->fast && smc_tma_supported(w, 1) &&
            smc_raw_tensor_bytes(w->dtype, w->N, w->K) >= (int64_t)ctx->f32_digits_row_mb << 20 && (reinterpret_cast<uintptr_t>(d_in) & 15) == 0)
            return qmatmul_f32_digits(ctx, d_in, w, d_out, M, s);
        if (w->fast && (reinterpret_cast<uintptr_t>(d_in) & 15) == 0) return smc_launch_gemv_f32(ctx, d_in, w, d_out, M, s);
        // shapes the vector kernels do not take (ragged K, rows that start inside a block) run in the
        // reference's own order instead
        return smc_launch_gemv_ref(ctx, d_in, w, d_out, M, 0, w->N, s);
    case SMC_ACT_Q8: {
        if (!w->fast)
            return smc_fail(ctx, SMC_E_UNSUPPORTED,
                            "SMC_ACT_Q8 needs a weight registered with SMC_W_REPACK and K %% %d == 0",
                            w->dtype == SMC_Q8_0 ? 32 : 256);
        // a single row is quantised inside the GEMV kernel while it is staged: one launch, no scratch
        if (M == 1 && smc_tma_supported(w, 1) && (reinterpret_cast<uintptr_t>(d_in) & 15) == 0) {
            if (!gd) return smc_launch_gemv_tma_f32in(ctx, d_in, w, d_out, s);
            *fused = true;
            return smc_launch_gemv_tma_gather(ctx, d_in, w, d_out, gd, s);
        }
        // Everything else goes through the context's one scratch buffer of quantised activations.  The lock is held
        // until both kernels are queued, so host threads cannot interleave their launches or free the buffer under
        // one another; on the device the buffer is reused in stream order, which is why calls that use it have to
        // share one stream per context (see the header).
        std::unique_lock<std::mutex> lock(ctx->mu_scratch);
        if (!ctx->act || ctx->act->max_rows < M || ctx->act->max_k < w->K) {
            // growing the scratch allocates: make the first call of a new size outside stream capture
            int rows = ctx->act ? (ctx->act->max_rows > M ? ctx->act->max_rows : M) : (M > 32 ? M : 32);
            int k = ctx->act ? (ctx->act->max_k > w->K ? ctx->act->max_k : w->K) : w->K;
            if (ctx->act) {
                cudaDeviceSynchronize();
                smc_q8act_free(ctx->act);
                ctx->act = nullptr;
            }
            int rc = smc_q8act_alloc(ctx, rows, k, &ctx->act);
            if (rc) return rc;
        }
        int rc = smc_launch_quantize_q8(ctx, d_in, M, w->K, ctx->act, s);
        if (rc) return rc;
        if (gd && M == 1 && smc_tma_supported(w, 1)) {
            *fused = true;
            return smc_launch_gemv_tma_xg(ctx, ctx->act, nullptr, w, d_out, gd, s);
        }
        if (ctx->q8_prefill_tc && M >= 64 && smc_prefill_supported(w, M)) return smc_launch_prefill_q4k_q8(ctx, ctx->act, w, d_out, s, true);
        return smc_launch_gemv_q8(ctx, ctx->act, w, d_out, s);
    }
    default: return smc_fail(ctx, SMC_E_INVALID, "qmatmul: unknown mode %d", mode);
    }
}

int smc_qmatmul_dev(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M, int mode, void *stream)
{
    if (!ctx || !d_in || !w || !d_out || M < 0) return smc_fail(ctx, SMC_E_INVALID, "qmatmul: bad arguments");
    if (M == 0) return SMC_OK;
    return qmatmul_impl(ctx, d_in, w, d_out, M, mode, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

int smc_qmatmul_dev_gather(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M, int mode,
                           cudaStream_t s, const smc_gather_dev *gd, bool *fused)
{
    *fused = false;
    return qmatmul_impl(ctx, d_in, w, d_out, M, mode, s, gd, fused);
}

extern "C" {

static int one_row_fusable(smc_ctx *ctx, const smc_weight *w, const char *what, int max_k)
{
    if (!w->fast || w->K > max_k || !smc_tma_supported(w, 1))
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "%s: the weight is not one the one-row bulk-copy kernel takes (K = %d)", what, w->K);
    return SMC_OK;
}

int smc_qmatmul_swiglu_dev(smc_ctx *ctx, const float *d_gate, const float *d_up, const smc_weight *w, float *d_out, void *stream)
{
    if (!ctx || !d_gate || !d_up || !w || !d_out) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_swiglu: bad arguments");
    if ((reinterpret_cast<uintptr_t>(d_gate) | reinterpret_cast<uintptr_t>(d_up)) & 15)
        return smc_fail(ctx, SMC_E_INVALID, "qmatmul_swiglu: gate and up must be 16-byte aligned");
    int rc = one_row_fusable(ctx, w, "qmatmul_swiglu", 65536);
    if (rc) return rc;
    return smc_launch_gemv_tma_swiglu(ctx, d_gate, d_up, w, d_out, static_cast<cudaStream_t>(stream));
}

int smc_qmatmul_addnorm_dev(smc_ctx *ctx, const float *d_x, const float *d_add, const float *d_norm_w, float eps, float *d_sum,
                            const smc_weight *w, float *d_out, void *stream)
{
    if (!ctx || !d_x || !d_norm_w || !w || !d_out) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_addnorm: bad arguments");
    if ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_add) | reinterpret_cast<uintptr_t>(d_norm_w) |
         reinterpret_cast<uintptr_t>(d_sum)) & 15)
        return smc_fail(ctx, SMC_E_INVALID, "qmatmul_addnorm: operands must be 16-byte aligned");
    int rc = one_row_fusable(ctx, w, "qmatmul_addnorm", 9216);  // a thread keeps its chunks in registers across the norm
    if (rc) return rc;
    smc_norm_prologue pro{d_add, d_norm_w, d_sum, eps};
    return smc_launch_gemv_tma_addnorm(ctx, d_x, &pro, w, d_out, static_cast<cudaStream_t>(stream));
}

int smc_weight_concat_rows(smc_ctx *ctx, const smc_weight *const *parts, int count, smc_weight **out)
{
    if (!ctx || !parts || !out || count <= 0 || !parts[0]) return smc_fail(ctx, SMC_E_INVALID, "weight_concat: bad arguments");
    const int dtype = parts[0]->dtype, K = parts[0]->K;
    long long N = 0;
    bool raw = true;
    for (int i = 0; i < count; ++i) {
        const smc_weight *p = parts[i];
        if (!p || p->dtype != dtype || p->K != K) return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "weight_concat: parts differ in dtype or K");
        if (!p->fast) return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight_concat: parts must be registered with SMC_W_REPACK");
        if (dtype == SMC_Q6_K && ((long long)p->N * K / 256) % 8 != 0)
            return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight_concat: a Q6_K part must hold a multiple of 2048 elements");
        raw = raw && p->d_raw != nullptr;
        N += p->N;
    }
    if (N > INT32_MAX) return smc_fail(ctx, SMC_E_RANGE, "weight_concat: too many rows");
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    smc_weight *w = new smc_weight();
    w->dtype = dtype, w->N = (int)N, w->K = K, w->flags = SMC_W_REPACK | (raw ? SMC_W_KEEP_RAW : 0), w->fast = true;
    w->raw_bytes = (size_t)smc_raw_tensor_bytes(dtype, (int)N, K);
    cudaError_t e = cudaSuccess;
    // bytes per row of every array of the compute layout (rows are whole blocks when `fast`)
    const size_t blk = (size_t)K / 256;
    auto cat = [&](auto smc_weight::*field, size_t per_row) {
        using T = std::remove_reference_t<decltype(w->*field)>;
        if (e != cudaSuccess || per_row == 0) return;
        uint8_t *dst = nullptr;
        e = cudaMalloc(&dst, per_row * (size_t)N);
        if (e != cudaSuccess) return;
        w->*field = reinterpret_cast<T>(dst);
        size_t off = 0;
        for (int i = 0; i < count && e == cudaSuccess; ++i) {
            const size_t bytes = per_row * (size_t)parts[i]->N;
            e = cudaMemcpyAsync(dst + off, reinterpret_cast<const uint8_t *>(parts[i]->*field), bytes, cudaMemcpyDeviceToDevice,
                                ctx->stream);
            off += bytes;
        }
    };
    if (raw) cat(&smc_weight::d_raw, (size_t)smc_raw_tensor_bytes(dtype, 1, K));
    if (dtype == SMC_Q8_0) {
        cat(&smc_weight::q8_qs, (size_t)K);
        cat(&smc_weight::q8_d, (size_t)K / 32 * 2);
    } else if (dtype == SMC_Q6_K) {
        cat(&smc_weight::q6u, blk * (SMC_Q6U_BYTES / 8));  // parts were checked to be whole units
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        free_weight(w);
        return smc_fail(ctx, SMC_E_CUDA, "weight_concat: %s", cudaGetErrorString(e));
    }
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->by_host[static_cast<const void *>(w)] = w;  // no host bytes: the handle is its own key
    }
    *out = w;
    return SMC_OK;
}

int smc_weight_interleave_rows(smc_ctx *ctx, const smc_weight *a, const smc_weight *b, smc_weight **out)
{
    if (!ctx || !a || !b || !out) return smc_fail(ctx, SMC_E_INVALID, "weight_interleave: bad arguments");
    if (a->dtype != b->dtype || a->K != b->K || a->N != b->N)
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "weight_interleave: the two weights differ in dtype or shape");
    if (!a->fast || !b->fast) return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight_interleave: weights must be registered with SMC_W_REPACK");
    const int dtype = a->dtype, K = a->K, N = a->N;
    if (dtype == SMC_Q6_K && K % 2048) return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight_interleave: Q6_K rows must be whole 2048-element units");
    if (dtype != SMC_Q8_0 && K % 256) return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight_interleave: rows must be whole blocks");
    if (2LL * N > INT32_MAX) return smc_fail(ctx, SMC_E_RANGE, "weight_interleave: too many rows");
    const bool raw = a->d_raw && b->d_raw;
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    smc_weight *w = new smc_weight();
    w->dtype = dtype, w->N = 2 * N, w->K = K, w->flags = SMC_W_REPACK | (raw ? SMC_W_KEEP_RAW : 0), w->fast = true;
    w->raw_bytes = (size_t)smc_raw_tensor_bytes(dtype, 2 * N, K);
    cudaError_t e = cudaSuccess;
    // row 2i of the result = row i of a, row 2i + 1 = row i of b, for every array of the compute layout
    auto weave = [&](auto smc_weight::*field, size_t per_row) {
        using T = std::remove_reference_t<decltype(w->*field)>;
        if (e != cudaSuccess || per_row == 0) return;
        uint8_t *dst = nullptr;
        e = cudaMalloc(&dst, per_row * 2 * (size_t)N);
        if (e != cudaSuccess) return;
        w->*field = reinterpret_cast<T>(dst);
        e = cudaMemcpy2DAsync(dst, 2 * per_row, reinterpret_cast<const uint8_t *>(a->*field), per_row, per_row, (size_t)N,
                              cudaMemcpyDeviceToDevice, ctx->stream);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(dst + per_row, 2 * per_row, reinterpret_cast<const uint8_t *>(b->*field), per_row, per_row, (size_t)N,
                                  cudaMemcpyDeviceToDevice, ctx->stream);
    };
    if (raw) weave(&smc_weight::d_raw, (size_t)smc_raw_tensor_bytes(dtype, 1, K));
    if (dtype == SMC_Q8_0) {
        weave(&smc_weight::q8_qs, (size_t)K);
        weave(&smc_weight::q8_d, (size_t)K / 32 * 2);
    } else if (dtype == SMC_Q6_K) {
        weave(&smc_weight::q6u, (size_t)K / 2048 * SMC_Q6U_BYTES);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        free_weight(w);
        return smc_fail(ctx, SMC_E_CUDA, "weight_interleave: %s", cudaGetErrorString(e));
    }
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->by_host[static_cast<const void *>(w)] = w;  // no host bytes: the handle is its own key
    }
    *out = w;
    return SMC_OK;
}

int smc_qmatmul_swiglu_pairs_dev(smc_ctx *ctx, const float *d_x, const smc_weight *w, float *d_act, void *stream)
{
    if (!ctx || !d_x || !w || !d_act) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_swiglu_pairs: bad arguments");
    if (reinterpret_cast<uintptr_t>(d_x) & 15) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_swiglu_pairs: the activation row must be 16-byte aligned");
    if (w->N & 1) return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "qmatmul_swiglu_pairs: the interleaved matrix has an odd row count");
    int rc = one_row_fusable(ctx, w, "qmatmul_swiglu_pairs", 65536);
    if (rc) return rc;
    return smc_launch_gemv_tma_any(ctx, nullptr, d_x, nullptr, nullptr, w, d_act, nullptr, false, true, static_cast<cudaStream_t>(stream));
}

int smc_qmatmul_tc_dev(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M, void *stream)
{
    if (!ctx || !d_in || !w || !d_out || M < 0) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_tc: bad arguments");
    if (M == 0) return SMC_OK;
    return smc_launch_prefill_q4k(ctx, d_in, w, d_out, M, static_cast<cudaStream_t>(stream));
}

int smc_block_isums_dev(smc_ctx *ctx, const smc_q8act *a, int m, const smc_weight *w, int col0, int col1,
                        int32_t *d_sums, void *stream)
{
    if (!ctx || !a || !w || !d_sums || m < 0 || m >= a->M || col0 < 0 || col1 > w->N || col0 > col1 || a->K != w->K)
        return smc_fail(ctx, SMC_E_INVALID, "block_isums: bad arguments");
    if ((w->dtype == SMC_Q8_0 && w->K % 32) || (w->dtype != SMC_Q8_0 && w->K % 256))
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "block_isums: K must be a whole number of blocks");
    return smc_launch_block_isums(ctx, a, m, w, col0, col1, d_sums, static_cast<cudaStream_t>(stream));
}

int smc_quantize_weights_dev(smc_ctx *ctx, int dtype, const float *d_values, int64_t n, void *d_raw, void *stream)
{
    if (!ctx || !d_values || !d_raw) return smc_fail(ctx, SMC_E_INVALID, "quantize_weights: bad arguments");
    return smc_launch_quantize_weights(ctx, dtype, d_values, n, d_raw, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------ host slots
// Host activations in, host results out, on a weight the caller already holds a handle of.
static int qmatmul_host_impl(smc_ctx *ctx, const float *input, const smc_weight *w, float *output, int M, int mode)
{
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    int rc;
    size_t in_bytes = (size_t)M * w->K * sizeof(float), out_bytes = (size_t)M * w->N * sizeof(float);
    if ((rc = ensure_dev(ctx, &ctx->d_stage_in, &ctx->stage_in_cap, in_bytes))) return rc;
    if ((rc = ensure_dev(ctx, &ctx->d_stage_out, &ctx->stage_out_cap, out_bytes))) return rc;
    // one wait per call: input copy, kernels and result copy are ordered by the stream.  Page-locked caller buffers
    // are the source and the target of the copies themselves; pageable ones go through the context's bounce buffer.
    const bool pin_in = host_is_pinned(ctx, input), pin_out = host_is_pinned(ctx, output);  // under ctx->mu
    if (pin_in) SMC_CUDA(ctx, cudaMemcpyAsync(ctx->d_stage_in, input, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
    else if ((rc = h2d_queued(ctx, ctx->d_stage_in, input, in_bytes, pin_out ? in_bytes : out_bytes))) return rc;
    if ((rc = qmatmul_impl(ctx, ctx->d_stage_in, w, ctx->d_stage_out, M, mode, ctx->stream))) {
        cudaStreamSynchronize(ctx->stream);
        return rc;
    }
    if (!pin_out) return d2h(ctx, output, ctx->d_stage_out, out_bytes);
    SMC_CUDA(ctx, cudaMemcpyAsync(output, ctx->d_stage_out, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    SMC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return SMC_OK;
}

int smc_qmatmul_host(smc_ctx *ctx, const float *input, const void *host_raw, float *output, int M, int K, int N,
                     int dtype, int mode)
{
    if (!ctx || !input || !host_raw || !output || M < 0 || K <= 0 || N <= 0)
        return smc_fail(ctx, SMC_E_INVALID, "qmatmul_host: bad arguments");
    smc_weight *w = nullptr;
    int rc = smc_weight_lookup(ctx, host_raw, &w);
    if (rc) return rc;
    if (w->dtype != dtype || w->K != K || w->N != N)
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "qmatmul_host: weight was registered as dtype=%d N=%d K=%d, call says dtype=%d N=%d K=%d",
                        w->dtype, w->N, w->K, dtype, N, K);
    if (M == 0) return SMC_OK;
    return qmatmul_host_impl(ctx, input, w, output, M, mode);
}

int smc_host_register(smc_ctx *ctx, void *ptr, size_t bytes)
{
    if (!ctx || !ptr || bytes == 0) return smc_fail(ctx, SMC_E_INVALID, "host_register: bad arguments");
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    SMC_CUDA(ctx, cudaHostRegister(ptr, bytes, cudaHostRegisterPortable));
    for (int i = 0; i < 4; ++i)
        if (ctx->pin_seen[i] == ptr) ctx->pin_seen[i] = nullptr;  // a remembered "pageable" answer for this address is stale
    return SMC_OK;
}

int smc_host_unregister(smc_ctx *ctx, void *ptr)
{
    if (!ctx || !ptr) return smc_fail(ctx, SMC_E_INVALID, "host_unregister: bad arguments");
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    SMC_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // no copy of this context may still be reading it
    SMC_CUDA(ctx, cudaHostUnregister(ptr));
    for (int i = 0; i < 4; ++i)
        if (ctx->pin_seen[i] == ptr) ctx->pin_seen[i] = nullptr;
    return SMC_OK;
}

int smc_qmatmul_host_w(smc_ctx *ctx, const float *input, const smc_weight *w, float *output, int M, int K, int N, int mode)
{
    if (!ctx || !input || !w || !output || M < 0) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_host_w: bad arguments");
    if (w->K != K || w->N != N)
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "qmatmul_host_w: weight is N=%d K=%d, call says N=%d K=%d", w->N, w->K, N, K);
    if (M == 0) return SMC_OK;
    return qmatmul_host_impl(ctx, input, w, output, M, mode);
}

int smc_vecdot_host(smc_ctx *ctx, const float *input, const void *host_raw, int col, int K, int dtype, float *result)
{
    if (!ctx || !input || !host_raw || !result || K <= 0) return smc_fail(ctx, SMC_E_INVALID, "vecdot_host: bad arguments");
    smc_weight *w = nullptr;
    int rc = smc_weight_lookup(ctx, host_raw, &w);
    if (rc) return rc;
    if (w->dtype != dtype || w->K != K)
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "vecdot_host: weight was registered as dtype=%d K=%d", w->dtype, w->K);
    if (col < 0 || col >= w->N) return smc_fail(ctx, SMC_E_RANGE, "vecdot_host: col %d outside [0, %d)", col, w->N);
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    if ((rc = ensure_dev(ctx, &ctx->d_stage_in, &ctx->stage_in_cap, (size_t)K * sizeof(float)))) return rc;
    if ((rc = ensure_dev(ctx, &ctx->d_stage_out, &ctx->stage_out_cap, (size_t)w->N * sizeof(float)))) return rc;
    if ((rc = h2d(ctx, ctx->d_stage_in, input, (size_t)K * sizeof(float)))) return rc;
    // a single dot runs in the scalar tier's order: it is what the reference's vec-dot tests pin
    if ((rc = smc_launch_gemv_ref(ctx, ctx->d_stage_in, w, ctx->d_stage_out, 1, col, col + 1, ctx->stream))) return rc;
    return d2h(ctx, result, ctx->d_stage_out + col, sizeof(float));
}

static int unary_host(smc_ctx *ctx, const float *a, const float *b, float *dst, int n, int op, float scalar)
{
    if (!ctx || !a || !dst || n < 0) return smc_fail(ctx, SMC_E_INVALID, "bad arguments");
    if (n == 0) return SMC_OK;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    size_t bytes = (size_t)n * sizeof(float);
    int rc;
    if ((rc = ensure_dev(ctx, &ctx->d_stage_in, &ctx->stage_in_cap, bytes))) return rc;
    if ((rc = ensure_dev(ctx, &ctx->d_stage_out, &ctx->stage_out_cap, bytes))) return rc;
    if ((rc = h2d(ctx, ctx->d_stage_in, a, bytes))) return rc;
    if (b) {
        if ((rc = ensure_dev(ctx, &ctx->d_stage_aux, &ctx->stage_aux_cap, bytes))) return rc;
        if ((rc = h2d(ctx, ctx->d_stage_aux, b, bytes))) return rc;
    }
    switch (op) {
    case 0: rc = smc_swiglu_dev(ctx, ctx->d_stage_in, ctx->d_stage_aux, ctx->d_stage_out, 1, n, n, ctx->stream); break;
    case 1: rc = smc_silu_dev(ctx, ctx->d_stage_in, ctx->d_stage_out, n, ctx->stream); break;
    case 2: rc = smc_softmax_dev(ctx, ctx->d_stage_in, ctx->d_stage_out, 1, n, ctx->stream); break;
    default: rc = smc_launch_rmsnorm_row(ctx, ctx->d_stage_in, ctx->d_stage_aux, ctx->d_stage_out, n, scalar, ctx->stream); break;
    }
    if (rc) return rc;
    return d2h(ctx, dst, ctx->d_stage_out, bytes);
}

int smc_swiglu_host(smc_ctx *ctx, const float *gate, const float *up, float *dst, int n)
{
    if (!up) return smc_fail(ctx, SMC_E_INVALID, "swiglu_host: bad arguments");
    return unary_host(ctx, gate, up, dst, n, 0, 0.f);
}
int smc_silu_host(smc_ctx *ctx, const float *src, float *dst, int n) { return unary_host(ctx, src, nullptr, dst, n, 1, 0.f); }
int smc_softmax_row_host(smc_ctx *ctx, const float *src, float *dst, int n)
{
    if (n == 0) return smc_fail(ctx, SMC_E_INVALID, "softmax_row_host: empty row");
    return unary_host(ctx, src, nullptr, dst, n, 2, 0.f);
}
int smc_rmsnorm_row_host(smc_ctx *ctx, const float *src, const float *weight, float *dst, int n, float rms_inv)
{
    if (!weight) return smc_fail(ctx, SMC_E_INVALID, "rmsnorm_row_host: bad arguments");
    return unary_host(ctx, src, weight, dst, n, 3, rms_inv);
}

int smc_sdpa_host(smc_ctx *ctx, const float *q, const float *k, const float *v, float *o, int seqLen, int kvLen,
                  int headDim, float scale, int causal, int qStride, int oStride, float alibiSlope)
{
    if (!ctx || !q || !k || !v || !o || seqLen < 0 || kvLen < 0 || headDim <= 0 || qStride < headDim || oStride < headDim)
        return smc_fail(ctx, SMC_E_INVALID, "sdpa_host: bad arguments");
    if (headDim > 256)  // AttentionKernels.cs:225-227 throws ArgumentOutOfRangeException
        return smc_fail(ctx, SMC_E_RANGE, "headDim %d exceeds FlashMaxHeadDim 256", headDim);
    if (seqLen == 0) return SMC_OK;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    size_t qn = (size_t)(seqLen - 1) * qStride + headDim, on = (size_t)(seqLen - 1) * oStride + headDim;
    size_t kvn = (size_t)kvLen * headDim;
    int rc;
    if ((rc = ensure_dev(ctx, &ctx->d_stage_in, &ctx->stage_in_cap, qn * sizeof(float)))) return rc;
    if ((rc = ensure_dev(ctx, &ctx->d_stage_out, &ctx->stage_out_cap, on * sizeof(float)))) return rc;
    if ((rc = ensure_dev(ctx, &ctx->d_stage_aux, &ctx->stage_aux_cap, (2 * kvn + 4) * sizeof(float)))) return rc;
    if ((rc = h2d(ctx, ctx->d_stage_in, q, qn * sizeof(float)))) return rc;
    if (kvn) {
        if ((rc = h2d(ctx, ctx->d_stage_aux, k, kvn * sizeof(float)))) return rc;
        if ((rc = h2d(ctx, ctx->d_stage_aux + kvn, v, kvn * sizeof(float)))) return rc;
    }
    // rows of o between the headDim-wide outputs belong to the caller: fetch, overwrite, return
    if (oStride != headDim)
        if ((rc = h2d(ctx, ctx->d_stage_out, o, on * sizeof(float)))) return rc;
    if ((rc = smc_launch_sdpa_tile(ctx, ctx->d_stage_in, ctx->d_stage_aux, ctx->d_stage_aux + kvn, ctx->d_stage_out,
                                   seqLen, kvLen, headDim, scale, causal, qStride, oStride, alibiSlope, ctx->stream)))
        return rc;
    return d2h(ctx, o, ctx->d_stage_out, on * sizeof(float));
}

}  // extern "C"
