// Device-resident KV cache objects behind the reference's IKVCache surface (SharpMind.Model/IKVCache.cs): Update,
// Reset, Truncate, TrimToLast, Length / MaxSeqLen, Snapshot / Restore, for the fp32 cache (KVCache.cs) and the Q8_0
// cache (QuantizedKVCache.cs), and attention over such a cache.
//
// Layout in HBM.  fp32: [batch][kvHead][maxSeq][headDim] floats, KVCache's own layout.  Q8_0: the reference keeps
// 34-byte blocks (fp16 scale + 32 int8) per row, which are only 2-byte aligned; here a tensor is two planes, quants
// [batch][kvHead][maxSeq][headDim] int8 (rows of 64 / 128 bytes, 16-byte loads) and scales
// [batch][kvHead][maxSeq][headDim/32] fp16.  Same byte count (34 per 32 elements).  Snapshot / Restore speak the
// reference's block layout, so bytes saved by either side can be loaded by the other.
//
// Quantisation on Update is QuantizedKVCache.QuantizeRowQ8_0 (QuantizedKVCache.cs:191-223): d = amax / 127 (1 for a
// zero block), stored as fp16 (round to nearest even), q = round-half-even(x / d) with the unrounded d.
#include <vector>

#include "smc_common.cuh"

struct smc_kv {
    int kind = SMC_KV_F32;
    int batch = 0, kv_heads = 0, max_seq = 0, head_dim = 0;
    int length = 0;            // CurrentPosition
    float *k = nullptr, *v = nullptr;        // fp32 planes
    int8_t *kq = nullptr, *vq = nullptr;     // Q8_0 quants
    __half *kd = nullptr, *vd = nullptr;     // Q8_0 block scales
};

namespace {

// src [batch][seqLen][kvHeads][hd] -> cache rows at positions pos0 .. pos0 + seqLen - 1 (KVCache.Update, KVCache.cs:84-150)
__global__ void __launch_bounds__(256) kv_update_f32_kernel(const float *__restrict__ sk, const float *__restrict__ sv,
                                                            float *__restrict__ dk, float *__restrict__ dv, long long total,
                                                            int seqLen, int kvh, int hd, int pos0, int maxSeq)
{
    smc_grid_dep_sync();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int d = (int)(t % hd);
        long long r = t / hd;
        const int h = (int)(r % kvh);
        r /= kvh;
        const int s = (int)(r % seqLen);
        const long long b = r / seqLen;
        const size_t dst = (((size_t)b * kvh + h) * maxSeq + pos0 + s) * hd + d;
        dk[dst] = sk[t];
        dv[dst] = sv[t];
    }
}

// One warp per 32-element block of a K or V row (QuantizedKVCache.Update + QuantizeRowQ8_0).
__global__ void __launch_bounds__(256) kv_update_q8_kernel(const float *__restrict__ sk, const float *__restrict__ sv,
                                                           int8_t *__restrict__ kq, __half *__restrict__ kd,
                                                           int8_t *__restrict__ vq, __half *__restrict__ vd, long long nblocks,
                                                           int seqLen, int kvh, int hd, int pos0, int maxSeq)
{
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31, bpr = hd / 32;
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); blk < 2 * nblocks; blk += stride) {
        const bool isv = blk >= nblocks;
        long long r = isv ? blk - nblocks : blk;
        const int bi = (int)(r % bpr);
        r /= bpr;
        const int h = (int)(r % kvh);
        r /= kvh;
        const int s = (int)(r % seqLen);
        const long long b = r / seqLen;
        const float x = (isv ? sv : sk)[(((size_t)b * seqLen + s) * kvh + h) * hd + 32 * bi + lane];
        float amax = fabsf(x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float d = __fdiv_rn(amax, 127.0f);
        if (amax == 0.0f) d = 1.0f;
        const int q = max(-128, min(127, __float2int_rn(__fdiv_rn(x, d))));
        const size_t row = ((size_t)b * kvh + h) * maxSeq + pos0 + s;
        (isv ? vq : kq)[row * hd + 32 * bi + lane] = (int8_t)q;
        if (lane == 0) (isv ? vd : kd)[row * bpr + bi] = __float2half_rn(d);
    }
}

// TrimToLast: rows [offset, offset + keep) of every (sequence, head) move to [0, keep).  The ranges may overlap, so the
// rows of one (sequence, head) are moved by ONE CTA in ascending order, a batch of rows at a time with a barrier
// between reading and writing.
__global__ void __launch_bounds__(256) kv_trim_kernel(uint8_t *__restrict__ base, size_t head_stride, size_t row_bytes, int offset,
                                                      int keep)
{
    extern __shared__ __align__(16) uint8_t buf[];
    uint8_t *p = base + (size_t)blockIdx.x * head_stride;
    const size_t chunk = 16384;  // bytes staged per round (dynamic shared memory)
    const size_t total = (size_t)keep * row_bytes, shift = (size_t)offset * row_bytes;
    for (size_t at = 0; at < total; at += chunk) {
        const size_t n = total - at < chunk ? total - at : chunk;
        for (size_t i = threadIdx.x; i < n; i += blockDim.x) buf[i] = p[shift + at + i];
        __syncthreads();
        for (size_t i = threadIdx.x; i < n; i += blockDim.x) p[at + i] = buf[i];
        __syncthreads();
    }
}

// planes <-> the reference's 34-byte blocks, positions [0, len) of every (sequence, head), densely packed
__global__ void __launch_bounds__(256) kv_q8_to_blocks_kernel(const int8_t *__restrict__ q, const __half *__restrict__ d,
                                                              uint8_t *__restrict__ out, long long nblocks, int len, int maxSeq, int hd)
{
    const int bpr = hd / 32;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < nblocks * 32; t += stride) {
        const long long blk = t >> 5;
        const int i = (int)(t & 31), bi = (int)(blk % bpr);
        long long r = blk / bpr;
        const int pos = (int)(r % len);
        const long long head = r / len;
        const size_t row = (size_t)head * maxSeq + pos;
        uint8_t *o = out + blk * 34;
        o[2 + i] = (uint8_t)q[row * hd + 32 * bi + i];
        if (i == 0) *reinterpret_cast<uint16_t *>(o) = __half_as_ushort(d[row * bpr + bi]);
    }
}
__global__ void __launch_bounds__(256) kv_blocks_to_q8_kernel(const uint8_t *__restrict__ in, int8_t *__restrict__ q,
                                                              __half *__restrict__ d, long long nblocks, int len, int maxSeq, int hd)
{
    const int bpr = hd / 32;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < nblocks * 32; t += stride) {
        const long long blk = t >> 5;
        const int i = (int)(t & 31), bi = (int)(blk % bpr);
        long long r = blk / bpr;
        const int pos = (int)(r % len);
        const long long head = r / len;
        const size_t row = (size_t)head * maxSeq + pos;
        const uint8_t *o = in + blk * 34;
        q[row * hd + 32 * bi + i] = (int8_t)o[2 + i];
        if (i == 0) d[row * bpr + bi] = __ushort_as_half(*reinterpret_cast<const uint16_t *>(o));
    }
}
__global__ void __launch_bounds__(256) kv_f32_pack_kernel(const float *__restrict__ src, float *__restrict__ dst, long long total,
                                                          int len, int maxSeq, int hd, int to_cache)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int e = (int)(t % hd);
        long long r = t / hd;
        const int pos = (int)(r % len);
        const long long head = r / len;
        const size_t c = ((size_t)head * maxSeq + pos) * hd + e;
        if (to_cache) dst[c] = src[t];
        else dst[t] = src[c];
    }
}

// Attention of ONE query row against a Q8_0 cache, any number of keys: one CTA of 128 threads per (sequence, head,
// query row); keys in tiles of 256, each thread scores two of them, the running max / sum are the flash recurrence of
// ScaledDotProductFlashQ8_0Scalar (AttentionKernels.cs:724-813), thread d accumulates output dim d.  Used where several
// query rows meet a Q8_0 cache (prompt chunks, speculative verification); the one-row decode step has its own kernel.
template <int HD>
__global__ void __launch_bounds__(128) sdpa_q8_rows_kernel(const float *__restrict__ q, const int8_t *__restrict__ kq,
                                                           const __half *__restrict__ kd, const int8_t *__restrict__ vq,
                                                           const __half *__restrict__ vd, float *__restrict__ out, int seqLen,
                                                           int heads, int kvHeads, int kvLen, int maxSeq, float scale)
{
    constexpr int TK = 256, BPR = HD / 32;
    __shared__ float sq[HD];
    __shared__ float sp[TK];
    __shared__ float red[4];
    smc_grid_dep_sync();
    const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z, t = threadIdx.x;
    const int kvh = h / (heads / kvHeads);
    const size_t head = (size_t)b * kvHeads + kvh;
    const int8_t *kqb = kq + head * (size_t)maxSeq * HD, *vqb = vq + head * (size_t)maxSeq * HD;
    const __half *kdb = kd + head * (size_t)maxSeq * BPR, *vdb = vd + head * (size_t)maxSeq * BPR;
    const float *qi = q + (((size_t)b * seqLen + i) * heads + h) * HD;
    const int eff = min(kvLen - seqLen + i + 1, kvLen);  // causal: the queries are the last seqLen positions
    for (int d = t; d < HD; d += 128) sq[d] = qi[d];
    float o = 0.f, m = -INFINITY, l = 0.f;
    __syncthreads();
    for (int start = 0; start < eff; start += TK) {
        const int len = min(TK, eff - start);
        float s2[2];
        float tmax = -INFINITY;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int j = t + 128 * u;
            s2[u] = -INFINITY;
            if (j < len) {
                const int8_t *kr = kqb + (size_t)(start + j) * HD;
                float dot = 0.f;
#pragma unroll
                for (int bi = 0; bi < BPR; ++bi) {
                    const float d = __half2float(kdb[(size_t)(start + j) * BPR + bi]);
                    float part = 0.f;
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        const uint4 kw = *reinterpret_cast<const uint4 *>(kr + 32 * bi + 16 * w);
                        const uint32_t ws[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            part = fmaf(sq[32 * bi + 16 * w + e], (float)(int)(int8_t)((ws[e >> 2] >> (8 * (e & 3))) & 0xFF), part);
                    }
                    dot = fmaf(part, d, dot);
                }
                s2[u] = dot * scale;
                tmax = fmaxf(tmax, s2[u]);
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
        if ((t & 31) == 0) red[t >> 5] = tmax;
        __syncthreads();
        tmax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        const float mn = fmaxf(m, tmax), alpha = expf(m - mn);
        float psum = 0.f;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int j = t + 128 * u;
            if (j < len) {
                const float p = expf(s2[u] - mn);
                sp[j] = p;
                psum += p;
            }
        }
        __syncthreads();  // red is read by everyone, sp is written
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
        if ((t & 31) == 0) red[t >> 5] = psum;
        __syncthreads();
        l = fmaf(l, alpha, (red[0] + red[1]) + (red[2] + red[3]));
        m = mn;
        if (t < HD) {
            o *= alpha;
            const int bi = t >> 5;
            for (int j = 0; j < len; ++j)
                o = fmaf(sp[j] * __half2float(vdb[(size_t)(start + j) * BPR + bi]), (float)vqb[(size_t)(start + j) * HD + t], o);
        }
        __syncthreads();
    }
    if (t < HD) out[(((size_t)b * seqLen + i) * heads + h) * HD + t] = l > 0.f ? __fdiv_rn(o, l) : 0.f;
}

int grid_cap(long long items, int per, int cap)
{
    long long g = (items + per - 1) / per;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

size_t row_bytes_ref(const smc_kv *kv) { return kv->kind == SMC_KV_Q8_0 ? (size_t)(kv->head_dim / 32) * 34 : (size_t)kv->head_dim * 4; }

}  // namespace

// internal accessors for the decoder
void smc_kv_planes(const smc_kv *kv, void **k, void **v, __half **kd, __half **vd)
{
    *k = kv->kind == SMC_KV_Q8_0 ? (void *)kv->kq : (void *)kv->k;
    *v = kv->kind == SMC_KV_Q8_0 ? (void *)kv->vq : (void *)kv->v;
    *kd = kv->kd, *vd = kv->vd;
}

// q, out [batch, seqLen, heads, hd]; the planes belong to `batch` sequences of kvHeads heads with maxSeq rows each
int smc_launch_sdpa_q8_rows(smc_ctx *ctx, const float *q, const int8_t *kq, const __half *kd, const int8_t *vq, const __half *vd, float *out,
                            int batch, int seqLen, int heads, int kvHeads, int hd, int kvLen, int maxSeq, float scale, cudaStream_t s)
{
    if (hd != 64 && hd != 128) return smc_fail(ctx, SMC_E_UNSUPPORTED, "a Q8_0 cache with headDim %d (64 and 128 are built)", hd);
    // a chunk of a prompt (16 rows and more): the tensor-core kernel, one sequence at a time, its K / V tiles staged as d * q
    if (ctx->attn_mma && seqLen >= 16 && smc_sdpa_prefill_mma_supported(heads, kvHeads, hd)) {
        const size_t per_seq = (size_t)kvHeads * maxSeq * hd;
        for (int b = 0; b < batch; ++b) {
            const int rc = smc_launch_sdpa_prefill_mma_q8(ctx, q + (size_t)b * seqLen * heads * hd, kq + b * per_seq, kd + b * (per_seq / 32),
                                                          vq + b * per_seq, vd + b * (per_seq / 32), out + (size_t)b * seqLen * heads * hd,
                                                          seqLen, heads, kvHeads, hd, kvLen - seqLen, maxSeq, scale, s);
            if (rc) return rc;
        }
        return SMC_OK;
    }
    const dim3 grid(seqLen, heads, batch);
    if (hd == 128)
        smc_launch_dep(ctx->use_pdl, sdpa_q8_rows_kernel<128>, grid, dim3(128), 0, s, q, kq, kd, vq, vd, out, seqLen, heads, kvHeads, kvLen, maxSeq, scale);
    else
        smc_launch_dep(ctx->use_pdl, sdpa_q8_rows_kernel<64>, grid, dim3(128), 0, s, q, kq, kd, vq, vd, out, seqLen, heads, kvHeads, kvLen, maxSeq, scale);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

extern "C" {

int smc_kv_create(smc_ctx *ctx, int batch, int kvHeads, int maxSeq, int headDim, int kind, smc_kv **out)
{
    if (!ctx || !out || batch <= 0 || kvHeads <= 0 || maxSeq <= 0 || headDim <= 0) return smc_fail(ctx, SMC_E_INVALID, "kv_create: bad arguments");
    if (kind != SMC_KV_F32 && kind != SMC_KV_Q8_0) return smc_fail(ctx, SMC_E_UNSUPPORTED, "kv_create: kind %d (fp32 = 0 and Q8_0 = 8 are built)", kind);
    if (kind == SMC_KV_Q8_0 && headDim % 32) return smc_fail(ctx, SMC_E_UNSUPPORTED, "kv_create: a Q8_0 cache needs headDim %% 32 == 0");
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    smc_kv *kv = new smc_kv();
    kv->kind = kind, kv->batch = batch, kv->kv_heads = kvHeads, kv->max_seq = maxSeq, kv->head_dim = headDim;
    const size_t n = (size_t)batch * kvHeads * maxSeq * headDim;
    cudaError_t e;
    if (kind == SMC_KV_F32) {
        e = cudaMalloc(&kv->k, n * 4);
        if (e == cudaSuccess) e = cudaMalloc(&kv->v, n * 4);
        if (e == cudaSuccess) e = cudaMemset(kv->k, 0, n * 4);
        if (e == cudaSuccess) e = cudaMemset(kv->v, 0, n * 4);
    } else {
        e = cudaMalloc(&kv->kq, n);
        if (e == cudaSuccess) e = cudaMalloc(&kv->vq, n);
        if (e == cudaSuccess) e = cudaMalloc(&kv->kd, n / 32 * 2);
        if (e == cudaSuccess) e = cudaMalloc(&kv->vd, n / 32 * 2);
        if (e == cudaSuccess) e = cudaMemset(kv->kq, 0, n);
        if (e == cudaSuccess) e = cudaMemset(kv->vq, 0, n);
        if (e == cudaSuccess) e = cudaMemset(kv->kd, 0, n / 32 * 2);
        if (e == cudaSuccess) e = cudaMemset(kv->vd, 0, n / 32 * 2);
    }
    if (e != cudaSuccess) {
        smc_kv_destroy(ctx, kv);
        return smc_fail(ctx, SMC_E_CUDA, "kv_create: %s", cudaGetErrorString(e));
    }
    *out = kv;
    return SMC_OK;
}

int smc_kv_destroy(smc_ctx *ctx, smc_kv *kv)
{
    if (!kv) return smc_fail(ctx, SMC_E_INVALID, "kv_destroy: bad arguments");
    if (ctx) cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    cudaFree(kv->k), cudaFree(kv->v), cudaFree(kv->kq), cudaFree(kv->vq), cudaFree(kv->kd), cudaFree(kv->vd);
    delete kv;
    return SMC_OK;
}

int smc_kv_length(const smc_kv *kv) { return kv ? kv->length : 0; }
int smc_kv_max_seq(const smc_kv *kv) { return kv ? kv->max_seq : 0; }

int smc_kv_reset(smc_ctx *ctx, smc_kv *kv)
{
    if (!kv) return smc_fail(ctx, SMC_E_INVALID, "kv_reset: bad arguments");
    kv->length = 0;
    return SMC_OK;
}

int smc_kv_truncate(smc_ctx *ctx, smc_kv *kv, int length)
{
    if (!kv || length < 0) return smc_fail(ctx, SMC_E_INVALID, "kv_truncate: bad arguments");
    if (length < kv->length) kv->length = length;  // Math.Min(length, CurrentPosition)
    return SMC_OK;
}

int smc_kv_update_dev(smc_ctx *ctx, smc_kv *kv, const float *d_k, const float *d_v, int batch, int seqLen, void *stream)
{
    if (!ctx || !kv || !d_k || !d_v || batch < 0 || batch > kv->batch || seqLen < 0) return smc_fail(ctx, SMC_E_INVALID, "kv_update: bad arguments");
    if (kv->length + seqLen > kv->max_seq)
        return smc_fail(ctx, SMC_E_RANGE, "KVCache overflow: position %d + seqLen %d exceeds capacity %d", kv->length, seqLen, kv->max_seq);
    if (batch == 0 || seqLen == 0) return SMC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long total = (long long)batch * seqLen * kv->kv_heads * kv->head_dim;
    if (kv->kind == SMC_KV_F32)
        smc_launch_dep(ctx->use_pdl, kv_update_f32_kernel, dim3(grid_cap(total, 256, ctx->sm_count * 8)), dim3(256), 0, s, d_k, d_v, kv->k,
                       kv->v, total, seqLen, kv->kv_heads, kv->head_dim, kv->length, kv->max_seq);
    else
        smc_launch_dep(ctx->use_pdl, kv_update_q8_kernel, dim3(grid_cap(total / 16, 8, ctx->sm_count * 8)), dim3(256), 0, s, d_k, d_v,
                       kv->kq, kv->kd, kv->vq, kv->vd, total / 32, seqLen, kv->kv_heads, kv->head_dim, kv->length, kv->max_seq);
    SMC_LAUNCH_CHECK(ctx);
    kv->length += seqLen;
    return SMC_OK;
}

int smc_kv_trim_to_last(smc_ctx *ctx, smc_kv *kv, int keep, void *stream)
{
    if (!ctx || !kv || keep < 0) return smc_fail(ctx, SMC_E_RANGE, "kv_trim_to_last: keep must not be negative");
    if (keep == 0) {
        kv->length = 0;
        return SMC_OK;
    }
    if (keep >= kv->length) return SMC_OK;
    const int offset = kv->length - keep, heads = kv->batch * kv->kv_heads;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto run = [&](void *base, size_t row_bytes) {
        kv_trim_kernel<<<heads, 256, 16384, s>>>(static_cast<uint8_t *>(base), (size_t)kv->max_seq * row_bytes, row_bytes, offset, keep);
    };
    if (kv->kind == SMC_KV_F32) {
        run(kv->k, (size_t)kv->head_dim * 4), run(kv->v, (size_t)kv->head_dim * 4);
    } else {
        run(kv->kq, (size_t)kv->head_dim), run(kv->vq, (size_t)kv->head_dim);
        run(kv->kd, (size_t)kv->head_dim / 32 * 2), run(kv->vd, (size_t)kv->head_dim / 32 * 2);
    }
    SMC_LAUNCH_CHECK(ctx);
    kv->length = keep;
    return SMC_OK;
}

int64_t smc_kv_snapshot_bytes(const smc_kv *kv)
{
    return kv ? (int64_t)kv->batch * kv->kv_heads * kv->length * (int64_t)row_bytes_ref(kv) : 0;
}

int smc_kv_snapshot(smc_ctx *ctx, const smc_kv *kv, void *host_k, void *host_v, int64_t bytes_each, int *position)
{
    if (!ctx || !kv || !position) return smc_fail(ctx, SMC_E_INVALID, "kv_snapshot: bad arguments");
    *position = kv->length;
    const int64_t need = smc_kv_snapshot_bytes(kv);
    if (need == 0) return SMC_OK;
    if (!host_k || !host_v || bytes_each != need)
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "kv_snapshot: the cache holds %lld bytes per tensor, caller offers %lld", (long long)need, (long long)bytes_each);
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    SMC_CUDA(ctx, cudaDeviceSynchronize());
    uint8_t *tmp = nullptr;
    SMC_CUDA(ctx, cudaMalloc(&tmp, (size_t)need));
    const long long heads = (long long)kv->batch * kv->kv_heads;
    cudaError_t e = cudaSuccess;
    for (int which = 0; which < 2 && e == cudaSuccess; ++which) {
        if (kv->kind == SMC_KV_F32) {
            const long long total = heads * kv->length * kv->head_dim;
            kv_f32_pack_kernel<<<grid_cap(total, 256, ctx->sm_count * 8), 256>>>(which ? kv->v : kv->k, reinterpret_cast<float *>(tmp), total,
                                                                              kv->length, kv->max_seq, kv->head_dim, 0);
        } else {
            const long long nblocks = heads * kv->length * (kv->head_dim / 32);
            kv_q8_to_blocks_kernel<<<grid_cap(nblocks * 32, 256, ctx->sm_count * 8), 256>>>(which ? kv->vq : kv->kq, which ? kv->vd : kv->kd, tmp,
                                                                                         nblocks, kv->length, kv->max_seq, kv->head_dim);
        }
        e = cudaMemcpy(which ? host_v : host_k, tmp, (size_t)need, cudaMemcpyDeviceToHost);
    }
    cudaFree(tmp);
    if (e != cudaSuccess) return smc_fail(ctx, SMC_E_CUDA, "kv_snapshot: %s", cudaGetErrorString(e));
    return SMC_OK;
}

int smc_kv_restore(smc_ctx *ctx, smc_kv *kv, const void *host_k, const void *host_v, int64_t bytes_each, int position)
{
    if (!ctx || !kv || position < 0 || position > kv->max_seq) return smc_fail(ctx, SMC_E_INVALID, "kv_restore: bad arguments");
    const int64_t need = (int64_t)kv->batch * kv->kv_heads * position * (int64_t)row_bytes_ref(kv);
    if (need && (!host_k || !host_v || bytes_each != need))
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "kv_restore: %d positions are %lld bytes per tensor, caller offers %lld", position, (long long)need, (long long)bytes_each);
    if (need) {
        SMC_CUDA(ctx, cudaSetDevice(ctx->device));
        SMC_CUDA(ctx, cudaDeviceSynchronize());
        uint8_t *tmp = nullptr;
        SMC_CUDA(ctx, cudaMalloc(&tmp, (size_t)need));
        const long long heads = (long long)kv->batch * kv->kv_heads;
        cudaError_t e = cudaSuccess;
        for (int which = 0; which < 2 && e == cudaSuccess; ++which) {
            e = cudaMemcpy(tmp, which ? host_v : host_k, (size_t)need, cudaMemcpyHostToDevice);
            if (e != cudaSuccess) break;
            if (kv->kind == SMC_KV_F32) {
                const long long total = heads * position * kv->head_dim;
                kv_f32_pack_kernel<<<grid_cap(total, 256, ctx->sm_count * 8), 256>>>(reinterpret_cast<const float *>(tmp), which ? kv->v : kv->k, total,
                                                                                  position, kv->max_seq, kv->head_dim, 1);
            } else {
                const long long nblocks = heads * position * (kv->head_dim / 32);
                kv_blocks_to_q8_kernel<<<grid_cap(nblocks * 32, 256, ctx->sm_count * 8), 256>>>(tmp, which ? kv->vq : kv->kq, which ? kv->vd : kv->kd,
                                                                                             nblocks, position, kv->max_seq, kv->head_dim);
            }
            e = cudaDeviceSynchronize();
        }
        cudaFree(tmp);
        if (e != cudaSuccess) return smc_fail(ctx, SMC_E_CUDA, "kv_restore: %s", cudaGetErrorString(e));
    }
    kv->length = position;
    return SMC_OK;
}

int smc_sdpa_kv_dev(smc_ctx *ctx, const smc_kv *kv, const float *d_q, float *d_out, int batch, int heads, int seqLen, float scale,
                    void *stream)
{
    if (!ctx || !kv || !d_q || !d_out || batch < 0 || batch > kv->batch || heads <= 0 || heads % kv->kv_heads || seqLen <= 0 ||
        seqLen > kv->length)
        return smc_fail(ctx, SMC_E_INVALID, "sdpa_kv: bad arguments (the cache holds %d positions)", kv ? kv->length : 0);
    if (kv->head_dim > 256) return smc_fail(ctx, SMC_E_RANGE, "headDim %d exceeds FlashMaxHeadDim 256", kv->head_dim);
    if (batch == 0) return SMC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int hd = kv->head_dim;
    if (seqLen == 1) {
        if (kv->kind == SMC_KV_Q8_0)
            return smc_sdpa_decode_any(ctx, d_q, kv->kq, kv->vq, kv->kd, kv->vd, d_out, batch, heads, kv->kv_heads, hd, kv->length, kv->max_seq, scale, s);
        return smc_sdpa_decode_any(ctx, d_q, kv->k, kv->v, nullptr, nullptr, d_out, batch, heads, kv->kv_heads, hd, kv->length, kv->max_seq, scale, s);
    }
    if (kv->kind == SMC_KV_Q8_0)
        return smc_launch_sdpa_q8_rows(ctx, d_q, kv->kq, kv->kd, kv->vq, kv->vd, d_out, batch, seqLen, heads, kv->kv_heads, hd, kv->length,
                                       kv->max_seq, scale, s);
    // fp32 cache, several query rows: the prompt kernel, one sequence at a time
    if (hd != 64 && hd != 128) return smc_fail(ctx, SMC_E_UNSUPPORTED, "sdpa_kv: several query rows need headDim 64 or 128");
    const size_t per_seq = (size_t)kv->kv_heads * kv->max_seq * hd;
    for (int b = 0; b < batch; ++b) {
        int rc = smc_launch_sdpa_prefill(ctx, d_q + (size_t)b * seqLen * heads * hd, kv->k + b * per_seq, kv->v + b * per_seq,
                                         d_out + (size_t)b * seqLen * heads * hd, seqLen, heads, kv->kv_heads, hd, kv->length - seqLen,
                                         kv->max_seq, scale, s);
        if (rc) return rc;
    }
    return SMC_OK;
}

}  // extern "C"
