// One decode step of a Llama/Qwen-shaped decoder, device resident: the order of operations of
// Transformer.ForwardLastLogits (SharpMind.Model/Transformer.cs:417-463), DecoderArch.Forward
// (SharpMind.Model/Arch/DecoderArch.cs:115-134), UnhookedTransformerBlock.Forward
// (SharpMind.Model/Layers/UnhookedTransformerBlock.cs:12-47), AttentionLayer.Forward
// (SharpMind.Model/Layers/Attention/AttentionLayer.cs:260-422) and FfnKernels.Gated
// (SharpMind.Model/Layers/Ffn/FfnKernels.cs:35-59), for seqLen = 1 and `batch` lock-step sequences sharing
// one position (the only batched semantics the reference's KVCache defines, KVCache.cs:21,149).
// The step is a sequence of launches of the kernels in this library on the caller's stream, with the
// elementwise work between two matmuls folded into one launch each (joined Q/K/V matmul, then per-head
// norm + RoPE + cache append in one kernel; residual add + the following RMSNorm in one kernel);
// the KV cache, the RoPE tables and all intermediates are owned by the model object.
#include <utility>
#include <vector>

#include "smc_common.cuh"

struct smc_model {
    smc_model_desc d{};
    int max_batch = 0;
    int rows = 0;  // rows the activation scratch holds: max_batch, or the longest prompt chunk seen so far
    std::vector<const smc_weight *> wq, wk, wv, wo, wgu, wdown;
    std::vector<smc_weight *> wqkv;  // rows of Wq, Wk, Wv in one matrix (owned), when the three could be joined
    float *qkv = nullptr;            // [batch][qDim + 2 kvDim]
    float *x2 = nullptr;             // second residual buffer of the one-sequence path (the stream ping-pongs)
    std::vector<const float *> norm1, norm2, qnorm, knorm;
    // optional per-layer bias vectors of the linear layers (LinearLayer.AddBiasInPlace); bqkv = [bq | bk | bv] (owned)
    std::vector<const float *> bq, bk, bv, bo, bgu, bdown;
    std::vector<float *> bqkv;
    bool has_bias = false;
    float *kcache = nullptr, *vcache = nullptr;  // [layer][batch][kvHeads][max_seq][head_dim]
    // kv_dtype == SMC_KV_Q8_0: the caches are Q8_0 rows instead (QuantizedKVCache), as int8 planes of the same shape and
    // fp16 block scales [layer][batch][kvHeads][max_seq][head_dim / 32]
    bool kv_q8 = false;
    int8_t *kq8 = nullptr, *vq8 = nullptr;
    __half *kd8 = nullptr, *vd8 = nullptr;
    float *cosT = nullptr, *sinT = nullptr;
    float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *tmp = nullptr,
          *gu = nullptr, *act = nullptr;
    smc_q8act *qa = nullptr, *qb = nullptr;  // quantised activations for batch > 1 (hidden-sized / widest row)
};

namespace {

void free_model(smc_ctx *ctx, smc_model *m)
{
    if (!m) return;
    float *bufs[] = {m->kcache, m->vcache, m->cosT, m->sinT, m->x, m->xn, m->q, m->k, m->v, m->att, m->tmp, m->gu, m->act, m->qkv, m->x2};
    for (float *p : bufs) cudaFree(p);
    cudaFree(m->kq8), cudaFree(m->vq8), cudaFree(m->kd8), cudaFree(m->vd8);
    for (smc_weight *w : m->wqkv)
        if (w) smc_weight_release(ctx, w);
    for (float *b : m->bqkv) cudaFree(b);
    smc_q8act_free(m->qa);
    smc_q8act_free(m->qb);
    delete m;
}

// (Re)allocates the per-row activation scratch for `rows` rows; the caches and the tables are not touched.
int alloc_rows(smc_ctx *ctx, smc_model *m, int rows)
{
    const smc_model_desc &d = m->d;
    const size_t H = d.hidden, qDim = (size_t)d.n_heads * d.head_dim, kvDim = (size_t)d.n_kv_heads * d.head_dim, F = d.ffn;
    float **bufs[] = {&m->x, &m->xn, &m->q, &m->k, &m->v, &m->att, &m->tmp, &m->gu, &m->act, &m->qkv};
    const size_t widths[] = {H, H, qDim, kvDim, kvDim, qDim, H, 2 * F, F, qDim + 2 * kvDim};
    if (m->rows) cudaDeviceSynchronize();  // the buffers being replaced may be in use
    for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); ++i) {
        cudaFree(*bufs[i]);
        *bufs[i] = nullptr;
    }
    smc_q8act_free(m->qa);
    smc_q8act_free(m->qb);
    m->qa = m->qb = nullptr;
    m->rows = 0;
    for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); ++i) {
        cudaError_t e = cudaMalloc(bufs[i], (size_t)rows * widths[i] * sizeof(float));
        if (e != cudaSuccess) return smc_fail(ctx, SMC_E_CUDA, "activation scratch for %d rows: %s", rows, cudaGetErrorString(e));
    }
    int rc = 0;
    if (H % 32 == 0) rc = smc_q8act_alloc(ctx, rows, (int)H, &m->qa);
    const size_t wide = qDim > F ? qDim : F;
    if (!rc && wide % 32 == 0) rc = smc_q8act_alloc(ctx, rows, (int)wide, &m->qb);
    if (rc) return rc;
    m->rows = rows;
    return SMC_OK;
}

// y[M, N] = x[M, K] W^T in the requested mode; for SMC_ACT_Q8 with several rows the quantised rows in
// `pre` (made by the caller from the same x) are reused instead of quantising again.
// RMSNorm of x (after x += add when `add` is given) for matmuls that read quantised activations: one pass that leaves
// the Q8_0 rows in m->qa, or the separate kernels through m->xn where the shape needs them.  Same bits either way.
int norm_into_q8(smc_ctx *ctx, smc_model *m, float *x, const float *add, const float *w, int rows, int H, float eps, cudaStream_t s)
{
    int rc = smc_launch_add_rmsnorm_q8(ctx, x, add, w, nullptr, rows, H, eps, m->qa, s);
    if (rc != SMC_E_UNSUPPORTED) return rc;
    rc = add ? smc_add_rmsnorm_dev(ctx, x, add, w, m->xn, rows, H, eps, s) : smc_rmsnorm_dev(ctx, x, w, m->xn, rows, H, eps, s);
    if (rc) return rc;
    return smc_quantize_q8_dev(ctx, m->xn, rows, H, m->qa, s);
}

int linear(smc_ctx *ctx, const float *x, const smc_weight *w, float *y, int M, int mode, const smc_q8act *pre,
           cudaStream_t s, const float *bias = nullptr)
{
    int rc = (mode == SMC_ACT_Q8 && pre) ? smc_qmatmul_q8_dev(ctx, pre, w, y, s) : smc_qmatmul_dev(ctx, x, w, y, M, mode, s);
    if (rc || !bias) return rc;
    return smc_add_bias_dev(ctx, y, bias, M, w->N, s);  // InferenceLinearLayer.Forward: matmul, then AddBiasInPlace
}

// src [layers][batch][kvHeads][len][headDim] dense  ->  cache [layers][max_batch][kvHeads][max_seq][headDim]
__global__ void kv_load_kernel(const float *__restrict__ src, float *__restrict__ dst, long long total, int batch,
                               int max_batch, int kvh, int len, int max_seq, int hd)
{
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        int d = (int)(t % hd);
        long long r = t / hd;
        int p = (int)(r % len);
        r /= len;
        int h = (int)(r % kvh);
        r /= kvh;
        int b = (int)(r % batch);
        long long l = r / batch;
        dst[(((l * max_batch + b) * kvh + h) * max_seq + p) * hd + d] = src[t];
    }
}

// What follows the joined Q/K/V matmul for one new token per sequence, one warp per (sequence, head slot):
// per-head RMSNorm of Q and K (AttentionLayer.cs:300-318), RoPE at position `pos` (RoPE.Apply, RoPE.cs:168-277),
// K and V written into the cache at `pos` (KVCache.Update, KVCache.cs:84-150), Q written densely for the
// attention kernel.  Lane l holds elements l, l + 32, ...: the norm sums in the order of the stand-alone norm
// kernel and the rotation uses the same unfused products, so the results are the same bits as the separate
// launches.  headDim % 64 == 0, headDim <= 256.
// A head row held as elements lane + 32 j -> Q8_0: block j is element j of every lane (QuantizeRowQ8_0,
// QuantizedKVCache.cs:191-223: d = amax / 127, 1 for a zero block, stored as fp16; q = round-half-even(x / d)).
template <int EPL>
__device__ __forceinline__ void store_row_q8(const float (&v)[EPL], int8_t *qrow, __half *drow, int lane)
{
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        float amax = fabsf(v[j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float d = __fdiv_rn(amax, 127.0f);
        if (amax == 0.0f) d = 1.0f;
        qrow[lane + 32 * j] = (int8_t)max(-128, min(127, __float2int_rn(__fdiv_rn(v[j], d))));
        if (lane == 0) drow[j] = __float2half_rn(d);
    }
}

struct Q8Planes {
    int8_t *kq, *vq;   // null: the cache is fp32
    __half *kd, *vd;
};

template <int EPL>  // elements per lane = headDim / 32
__global__ void __launch_bounds__(256) qkv_post_kernel(const float *__restrict__ qkv, float *__restrict__ q_out,
                                                       float *__restrict__ kc, float *__restrict__ vc, Q8Planes q8,
                                                       const float *__restrict__ qnorm, const float *__restrict__ knorm,
                                                       const float *__restrict__ cosT, const float *__restrict__ sinT, int batch,
                                                       int nh, int nkv, int pos, int maxSeq, float eps, int neox, int seq0)
{
    constexpr int HD = EPL * 32, PAIRS = HD / 2;
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31;
    const int slots = nh + 2 * nkv;
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= batch * slots) return;
    const int row = wid / slots, slot = wid % slots;
    const float *src = qkv + (size_t)row * slots * HD + (size_t)slot * HD;
    // decode: row r is sequence r at position pos.  Prompt (seq0 >= 0): row r is position pos + r of sequence seq0.
    const int b = seq0 >= 0 ? seq0 : row;
    pos += seq0 >= 0 ? row : 0;
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = src[lane + 32 * j];
    if (slot >= nh + nkv) {  // V: straight into the cache
        const size_t crow = ((size_t)b * nkv + (slot - nh - nkv)) * maxSeq + pos;
        if (q8.vq) {
            store_row_q8<EPL>(v, q8.vq + crow * HD, q8.vd + crow * EPL, lane);
            return;
        }
        float *dst = vc + crow * HD;
#pragma unroll
        for (int j = 0; j < EPL; ++j) dst[lane + 32 * j] = v[j];
        return;
    }
    const bool is_q = slot < nh;
    const float *nw = is_q ? qnorm : knorm;
    if (nw) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) ss = fmaf(v[j], v[j], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(ss, (float)HD) + eps));
#pragma unroll
        for (int j = 0; j < EPL; ++j) v[j] = (v[j] * inv) * nw[lane + 32 * j];
    }
    const float *ct = cosT + (size_t)pos * PAIRS, *st = sinT + (size_t)pos * PAIRS;
    if (neox) {  // pairs (i, i + headDim / 2): both halves live in this lane
#pragma unroll
        for (int j = 0; j < EPL / 2; ++j) {
            const int i = lane + 32 * j;
            const float c = __ldg(ct + i), sn = __ldg(st + i);
            const float a = v[j], bb = v[j + EPL / 2];
            v[j] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(bb, sn));
            v[j + EPL / 2] = __fadd_rn(__fmul_rn(bb, c), __fmul_rn(a, sn));
        }
    } else {  // pairs (2i, 2i + 1): the partner sits in the neighbouring lane
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int e = lane + 32 * j, i = e >> 1;
            const float c = __ldg(ct + i), sn = __ldg(st + i);
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
            v[j] = (lane & 1) ? __fadd_rn(__fmul_rn(v[j], c), __fmul_rn(other, sn))
                              : __fsub_rn(__fmul_rn(v[j], c), __fmul_rn(other, sn));
        }
    }
    if (!is_q && q8.kq) {
        const size_t crow = ((size_t)b * nkv + (slot - nh)) * maxSeq + pos;
        store_row_q8<EPL>(v, q8.kq + crow * HD, q8.kd + crow * EPL, lane);
        return;
    }
    float *dst = is_q ? q_out + ((size_t)row * nh + slot) * HD : kc + (((size_t)b * nkv + (slot - nh)) * maxSeq + pos) * HD;
#pragma unroll
    for (int j = 0; j < EPL; ++j) dst[lane + 32 * j] = v[j];
}

// per-layer strides of the caches (elements of the fp32 cache = bytes of the int8 planes; block scales are 1/32 of that)
size_t layer_elems(const smc_model *m) { return (size_t)m->max_batch * m->d.n_kv_heads * m->d.max_seq * m->d.head_dim; }

int launch_qkv_post(smc_ctx *ctx, const smc_model *m, int l, float *kc, float *vc, int B, int pos, cudaStream_t s, int seq0 = -1)
{
    const smc_model_desc &d = m->d;
    Q8Planes q8{nullptr, nullptr, nullptr, nullptr};
    if (m->kv_q8) {
        const size_t le = layer_elems(m);
        q8 = Q8Planes{m->kq8 + l * le, m->vq8 + l * le, m->kd8 + l * (le / 32), m->vd8 + l * (le / 32)};
    }
    const int warps = B * (d.n_heads + 2 * d.n_kv_heads);
    const dim3 grid((warps + 7) / 8);
    const float *qn = d.qk_norm ? m->qnorm[l] : nullptr, *kn = d.qk_norm ? m->knorm[l] : nullptr;
#define SMC_QKV_POST(E)                                                                                              \
    smc_launch_dep(ctx->use_pdl, qkv_post_kernel<E>, grid, dim3(256), 0, s, (const float *)m->qkv, m->q, kc, vc, q8, qn, kn, \
                   (const float *)m->cosT, (const float *)m->sinT, B, d.n_heads, d.n_kv_heads, pos, d.max_seq, d.eps,    \
                   d.neox, seq0)
    switch (d.head_dim) {
    case 64: SMC_QKV_POST(2); break;
    case 128: SMC_QKV_POST(4); break;
    case 192: SMC_QKV_POST(6); break;
    case 256: SMC_QKV_POST(8); break;
    default: return smc_fail(ctx, SMC_E_UNSUPPORTED, "joined QKV path needs headDim in {64, 128, 192, 256}");
    }
#undef SMC_QKV_POST
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// one decode step of attention for layer l over the model's cache (fp32 or Q8_0)
int attend_decode(smc_ctx *ctx, const smc_model *m, int l, int B, int pos, float scale, cudaStream_t s)
{
    const smc_model_desc &d = m->d;
    const size_t le = layer_elems(m);
    if (m->kv_q8)
        return smc_sdpa_decode_any(ctx, m->q, m->kq8 + l * le, m->vq8 + l * le, m->kd8 + l * (le / 32), m->vd8 + l * (le / 32), m->att, B,
                                   d.n_heads, d.n_kv_heads, d.head_dim, pos + 1, d.max_seq, scale, s);
    return smc_sdpa_decode_any(ctx, m->q, m->kcache + l * le, m->vcache + l * le, nullptr, nullptr, m->att, B, d.n_heads, d.n_kv_heads,
                               d.head_dim, pos + 1, d.max_seq, scale, s);
}

// dense fp32 context rows -> Q8_0 planes of the cache: one warp per 32-element block
__global__ void __launch_bounds__(256) kv_load_q8_kernel(const float *__restrict__ src, int8_t *__restrict__ q, __half *__restrict__ dsc,
                                                         long long nblocks, int batch, int max_batch, int kvh, int len, int max_seq, int hd)
{
    const int lane = threadIdx.x & 31, bpr = hd / 32;
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); blk < nblocks; blk += stride) {
        const int bi = (int)(blk % bpr);
        long long r = blk / bpr;
        const int p = (int)(r % len);
        r /= len;
        const int h = (int)(r % kvh);
        r /= kvh;
        const int b = (int)(r % batch);
        const long long l = r / batch;
        const float x = src[blk * 32 + lane];
        float amax = fabsf(x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float dd = __fdiv_rn(amax, 127.0f);
        if (amax == 0.0f) dd = 1.0f;
        const size_t row = (((size_t)l * max_batch + b) * kvh + h) * max_seq + p;
        q[row * hd + 32 * bi + lane] = (int8_t)max(-128, min(127, __float2int_rn(__fdiv_rn(x, dd))));
        if (lane == 0) dsc[row * bpr + bi] = __float2half_rn(dd);
    }
}

}  // namespace

extern "C" {

int smc_model_kv_load(smc_ctx *ctx, smc_model *m, const float *d_k, const float *d_v, int batch, int len, void *stream)
{
    if (!ctx || !m || !d_k || !d_v || batch <= 0 || len < 0) return smc_fail(ctx, SMC_E_INVALID, "kv_load: bad arguments");
    if (batch > m->max_batch || len > m->d.max_seq) return smc_fail(ctx, SMC_E_RANGE, "kv_load: %d x %d exceeds the cache", batch, len);
    long long total = (long long)m->d.n_layers * batch * m->d.n_kv_heads * len * m->d.head_dim;
    if (total == 0) return SMC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int grid = (int)((total + 255) / 256 > ctx->sm_count * 16 ? ctx->sm_count * 16 : (total + 255) / 256);
    if (m->kv_q8) {  // the context rows are quantised as QuantizedKVCache.Update would have quantised them
        kv_load_q8_kernel<<<grid, 256, 0, s>>>(d_k, m->kq8, m->kd8, total / 32, batch, m->max_batch, m->d.n_kv_heads, len, m->d.max_seq, m->d.head_dim);
        kv_load_q8_kernel<<<grid, 256, 0, s>>>(d_v, m->vq8, m->vd8, total / 32, batch, m->max_batch, m->d.n_kv_heads, len, m->d.max_seq, m->d.head_dim);
        SMC_LAUNCH_CHECK(ctx);
        return SMC_OK;
    }
    kv_load_kernel<<<grid, 256, 0, s>>>(d_k, m->kcache, total, batch, m->max_batch, m->d.n_kv_heads, len, m->d.max_seq, m->d.head_dim);
    kv_load_kernel<<<grid, 256, 0, s>>>(d_v, m->vcache, total, batch, m->max_batch, m->d.n_kv_heads, len, m->d.max_seq, m->d.head_dim);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_model_create(smc_ctx *ctx, const smc_model_desc *desc, int max_batch, smc_model **out)
{
    if (!ctx || !desc || !out || max_batch <= 0) return smc_fail(ctx, SMC_E_INVALID, "model_create: bad arguments");
    const smc_model_desc &d = *desc;
    if (d.n_layers <= 0 || d.hidden <= 0 || d.n_heads <= 0 || d.n_kv_heads <= 0 || d.n_heads % d.n_kv_heads ||
        d.head_dim <= 0 || (d.head_dim & 1) || d.ffn <= 0 || d.vocab <= 0 || d.max_seq <= 0 || !d.wq || !d.wk || !d.wv ||
        !d.wo || !d.wgu || !d.wdown || !d.norm1 || !d.norm2 || !d.final_norm || !d.lm_head ||
        (d.qk_norm && (!d.qnorm || !d.knorm)))
        return smc_fail(ctx, SMC_E_INVALID, "model_create: incomplete description");
    if (d.head_dim > 256) return smc_fail(ctx, SMC_E_RANGE, "headDim %d exceeds FlashMaxHeadDim 256", d.head_dim);
    if (d.kv_dtype != SMC_KV_F32 && d.kv_dtype != SMC_KV_Q8_0)
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "model_create: kv_dtype %d (fp32 = 0 and Q8_0 = 8 are built)", d.kv_dtype);
    if (d.kv_dtype == SMC_KV_Q8_0 && d.head_dim != 64 && d.head_dim != 128)
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "model_create: a Q8_0 KV cache needs headDim 64 or 128");
    const int H = d.hidden, qDim = d.n_heads * d.head_dim, kvDim = d.n_kv_heads * d.head_dim, F = d.ffn;
    auto shape_ok = [&](const smc_weight *w, int n, int k) { return w && w->N == n && w->K == k; };
    for (int l = 0; l < d.n_layers; ++l) {
        if (!shape_ok(d.wq[l], qDim, H) || !shape_ok(d.wk[l], kvDim, H) || !shape_ok(d.wv[l], kvDim, H) ||
            !shape_ok(d.wo[l], H, qDim) || !shape_ok(d.wgu[l], 2 * F, H) || !shape_ok(d.wdown[l], H, F))
            return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "model_create: layer %d weight shapes do not match the description", l);
    }
    if (!shape_ok(d.lm_head, d.vocab, H) || d.lm_head->dtype != SMC_Q8_0)
        return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "model_create: lm_head / embedding must be a Q8_0 [vocab, hidden] tensor");

    cudaSetDevice(ctx->device);
    smc_model *m = new smc_model();
    m->d = d;
    m->max_batch = max_batch;
    auto copy_w = [&](std::vector<const smc_weight *> &dst, const smc_weight *const *src) { dst.assign(src, src + d.n_layers); };
    auto copy_f = [&](std::vector<const float *> &dst, const float *const *src) {
        if (src) dst.assign(src, src + d.n_layers);
    };
    copy_w(m->wq, d.wq), copy_w(m->wk, d.wk), copy_w(m->wv, d.wv), copy_w(m->wo, d.wo), copy_w(m->wgu, d.wgu),
        copy_w(m->wdown, d.wdown);
    copy_f(m->norm1, d.norm1), copy_f(m->norm2, d.norm2), copy_f(m->qnorm, d.qnorm), copy_f(m->knorm, d.knorm);
    auto copy_b = [&](std::vector<const float *> &dst, const float *const *src) {
        dst.assign(d.n_layers, nullptr);
        if (!src) return;
        for (int l = 0; l < d.n_layers; ++l) {
            dst[l] = src[l];
            m->has_bias = m->has_bias || src[l] != nullptr;
        }
    };
    copy_b(m->bq, d.bq), copy_b(m->bk, d.bk), copy_b(m->bv, d.bv), copy_b(m->bo, d.bo), copy_b(m->bgu, d.bgu), copy_b(m->bdown, d.bdown);
    const size_t B = (size_t)max_batch;
    const size_t cache = (size_t)d.n_layers * B * d.n_kv_heads * d.max_seq * d.head_dim;
    const size_t half = (size_t)d.max_seq * (d.head_dim / 2);
    cudaError_t e = cudaSuccess;
    auto alloc = [&](float **p, size_t n) {
        if (e == cudaSuccess) e = cudaMalloc(p, n * sizeof(float));
    };
    m->kv_q8 = d.kv_dtype == SMC_KV_Q8_0;
    if (m->kv_q8) {
        if (e == cudaSuccess) e = cudaMalloc(&m->kq8, cache);
        if (e == cudaSuccess) e = cudaMalloc(&m->vq8, cache);
        if (e == cudaSuccess) e = cudaMalloc(&m->kd8, cache / 32 * sizeof(__half));
        if (e == cudaSuccess) e = cudaMalloc(&m->vd8, cache / 32 * sizeof(__half));
        if (e == cudaSuccess) e = cudaMemset(m->kq8, 0, cache);
        if (e == cudaSuccess) e = cudaMemset(m->vq8, 0, cache);
        if (e == cudaSuccess) e = cudaMemset(m->kd8, 0, cache / 32 * sizeof(__half));
        if (e == cudaSuccess) e = cudaMemset(m->vd8, 0, cache / 32 * sizeof(__half));
    } else {
        alloc(&m->kcache, cache), alloc(&m->vcache, cache);
        if (e == cudaSuccess) e = cudaMemset(m->kcache, 0, cache * sizeof(float));
        if (e == cudaSuccess) e = cudaMemset(m->vcache, 0, cache * sizeof(float));
    }
    alloc(&m->cosT, half), alloc(&m->sinT, half);
    alloc(&m->x2, (size_t)H);
    if (e != cudaSuccess) {
        free_model(ctx, m);
        return smc_fail(ctx, SMC_E_CUDA, "model_create: allocation failed: %s", cudaGetErrorString(e));
    }
    int rc = alloc_rows(ctx, m, max_batch);
    if (rc) {
        free_model(ctx, m);
        return rc;
    }
    // one matmul for Q, K and V where the three matrices can be joined (same format, vector layout) and the
    // head size suits the kernel that follows it
    m->wqkv.assign(d.n_layers, nullptr);
    const bool hd_ok = d.head_dim == 64 || d.head_dim == 128 || d.head_dim == 192 || d.head_dim == 256;
    for (int l = 0; l < d.n_layers && hd_ok && !rc; ++l) {
        const smc_weight *parts[3] = {m->wq[l], m->wk[l], m->wv[l]};
        if (!(parts[0]->fast && parts[1]->fast && parts[2]->fast && parts[0]->dtype == parts[1]->dtype &&
              parts[0]->dtype == parts[2]->dtype))
            continue;
        rc = smc_weight_concat_rows(ctx, parts, 3, &m->wqkv[l]);
        if (rc == SMC_E_UNSUPPORTED) rc = SMC_OK, m->wqkv[l] = nullptr;  // parts that cannot be joined stay three matmuls
    }
    // the joined matmul takes the three bias vectors joined the same way (zeros where a projection has none)
    m->bqkv.assign(d.n_layers, nullptr);
    for (int l = 0; l < d.n_layers && !rc; ++l) {
        if (!m->wqkv[l] || !(m->bq[l] || m->bk[l] || m->bv[l])) continue;
        cudaError_t ce = cudaMalloc(&m->bqkv[l], (size_t)(qDim + 2 * kvDim) * sizeof(float));
        if (ce == cudaSuccess) ce = cudaMemset(m->bqkv[l], 0, (size_t)(qDim + 2 * kvDim) * sizeof(float));
        const float *src[3] = {m->bq[l], m->bk[l], m->bv[l]};
        const int off[3] = {0, qDim, qDim + kvDim}, len[3] = {qDim, kvDim, kvDim};
        for (int i = 0; i < 3 && ce == cudaSuccess; ++i)
            if (src[i]) ce = cudaMemcpy(m->bqkv[l] + off[i], src[i], (size_t)len[i] * sizeof(float), cudaMemcpyDeviceToDevice);
        if (ce != cudaSuccess) rc = smc_fail(ctx, SMC_E_CUDA, "model_create: bias: %s", cudaGetErrorString(ce));
    }
    if (rc) {
        free_model(ctx, m);
        return rc;
    }
    rc = smc_rope_tables(ctx, d.rope_theta, d.head_dim, d.max_seq, m->cosT, m->sinT);
    // the attention's scratch for every step this model can run: decoding never allocates
    if (!rc && (d.head_dim == 64 || d.head_dim == 128)) rc = smc_sdpa_decode_reserve(ctx, max_batch, d.n_heads, d.n_kv_heads, d.head_dim, d.max_seq);
    if (rc) {
        free_model(ctx, m);
        return rc;
    }
    *out = m;
    return SMC_OK;
}

int smc_model_destroy(smc_ctx *ctx, smc_model *m)
{
    if (!ctx || !m) return smc_fail(ctx, SMC_E_INVALID, "model_destroy: bad arguments");
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    free_model(ctx, m);
    return SMC_OK;
}

int smc_model_kv(smc_ctx *ctx, smc_model *m, float **d_k, float **d_v)
{
    if (!ctx || !m || !d_k || !d_v) return smc_fail(ctx, SMC_E_INVALID, "model_kv: bad arguments");
    if (m->kv_q8) return smc_fail(ctx, SMC_E_UNSUPPORTED, "model_kv: the model's cache holds Q8_0 rows, not floats");
    *d_k = m->kcache;
    *d_v = m->vcache;
    return SMC_OK;
}

int smc_decode_step(smc_ctx *ctx, smc_model *m, const int *d_tokens, int batch, int pos, int mode, float *d_logits,
                    int *d_argmax, void *stream)
{
    if (!ctx || !m || !d_tokens || !d_logits || batch <= 0) return smc_fail(ctx, SMC_E_INVALID, "decode_step: bad arguments");
    if (batch > m->max_batch) return smc_fail(ctx, SMC_E_RANGE, "decode_step: batch %d exceeds the model's %d", batch, m->max_batch);
    const smc_model_desc &d = m->d;
    if (pos < 0 || pos + 1 > d.max_seq)  // KVCache.Update throws on overflow (KVCache.cs:89-91)
        return smc_fail(ctx, SMC_E_RANGE, "KVCache overflow: position %d + seqLen 1 exceeds capacity %d", pos, d.max_seq);
    if (mode != SMC_ACT_F32 && mode != SMC_ACT_Q8 && mode != SMC_REF_ORDER)
        return smc_fail(ctx, SMC_E_INVALID, "decode_step: unknown mode %d", mode);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int H = d.hidden, nh = d.n_heads, nkv = d.n_kv_heads, hd = d.head_dim, F = d.ffn;
    const int qDim = nh * hd, kvDim = nkv * hd, B = batch;
    const float scale = 1.0f / sqrtf((float)hd);
    const size_t layer_stride = (size_t)m->max_batch * nkv * d.max_seq * hd;
    // several rows in SMC_ACT_Q8: quantise an activation once and feed every matmul that reads it
    const bool reuse = mode == SMC_ACT_Q8 && B > 1 && m->qa && m->qb;
    int rc;
#define SMC_TRY(call)        \
    do {                     \
        rc = (call);         \
        if (rc) return rc;   \
    } while (0)

    // One sequence with quantised activations: every elementwise step between two matmuls rides in the staging of
    // the matmul that consumes it (residual add + RMSNorm, SiLU-gate), so a layer is eight launches: joined QKV,
    // per-head norm + RoPE + append, attention, Wo, gate||up, down (+ the next layer's QKV takes its residual).
    // (an FFN wider than ctx->ffn_fuse_max, 16384 by default, keeps its SiLU-gate as a launch of its own: the
    // down-projection's row is then too long to be worth staging through the gate on every SM pair)
    bool one_row = mode == SMC_ACT_Q8 && B == 1 && H <= 8192 && !m->has_bias && smc_tma_supported(d.lm_head, 1) &&
                   (F <= ctx->ffn_fuse_max || m->qb);
    for (int l = 0; l < d.n_layers && one_row; ++l)
        one_row = m->wqkv[l] && smc_tma_supported(m->wqkv[l], 1) && smc_tma_supported(m->wgu[l], 1) && m->wdown[l]->fast &&
                  (F > ctx->ffn_fuse_max || smc_tma_supported(m->wdown[l], 1));
    if (one_row) {
        float *cur = m->x, *other = m->x2;
        const float *pending = nullptr;  // output of the previous block's down-projection, not yet added to the stream
        SMC_TRY(smc_embed_q8_0_dev(ctx, d.lm_head, d_tokens, 1, cur, s));
        for (int l = 0; l < d.n_layers; ++l) {
            float *kc = m->kcache + (size_t)l * layer_stride, *vc = m->vcache + (size_t)l * layer_stride;
            smc_norm_prologue p1{pending, m->norm1[l], pending ? other : nullptr, d.eps};
            SMC_TRY(smc_launch_gemv_tma_addnorm(ctx, cur, &p1, m->wqkv[l], m->qkv, s));
            if (pending) std::swap(cur, other);
            SMC_TRY(launch_qkv_post(ctx, m, l, kc, vc, 1, pos, s));
            SMC_TRY(attend_decode(ctx, m, l, 1, pos, scale, s));
            SMC_TRY(smc_qmatmul_dev(ctx, m->att, m->wo[l], m->tmp, 1, mode, s));
            smc_norm_prologue p2{m->tmp, m->norm2[l], other, d.eps};
            SMC_TRY(smc_launch_gemv_tma_addnorm(ctx, cur, &p2, m->wgu[l], m->gu, s));
            std::swap(cur, other);
            if (F <= ctx->ffn_fuse_max) {
                SMC_TRY(smc_launch_gemv_tma_swiglu(ctx, m->gu, m->gu + F, m->wdown[l], m->tmp, s));
            } else {
                SMC_TRY(smc_launch_swiglu_quantize_q8(ctx, m->gu, m->gu + F, 1, F, 2 * F, m->qb, s));
                SMC_TRY(smc_qmatmul_q8_dev(ctx, m->qb, m->wdown[l], m->tmp, s));
            }
            pending = m->tmp;
        }
        smc_norm_prologue pf{pending, d.final_norm, nullptr, d.eps};
        SMC_TRY(smc_launch_gemv_tma_addnorm(ctx, cur, &pf, d.lm_head, d_logits, s));
        if (d_argmax) SMC_TRY(smc_argmax_dev(ctx, d_logits, 1, d.vocab, d_argmax, s));
        return SMC_OK;
    }
    SMC_TRY(smc_embed_q8_0_dev(ctx, d.lm_head, d_tokens, B, m->x, s));
    if (reuse) SMC_TRY(norm_into_q8(ctx, m, m->x, nullptr, m->norm1[0], B, H, d.eps, s));
    else SMC_TRY(smc_rmsnorm_dev(ctx, m->x, m->norm1[0], m->xn, B, H, d.eps, s));
    for (int l = 0; l < d.n_layers; ++l) {
        // m->xn (m->qa with quantised activations) holds RMSNorm(x) with this layer's first norm, made by the previous layer's tail
        float *kc = m->kcache + (size_t)l * layer_stride, *vc = m->vcache + (size_t)l * layer_stride;
        // the joined matrix carries no GGUF-layout copy unless its parts kept theirs: reference order needs it
        const smc_weight *joined = m->wqkv[l];
        if (joined && (mode != SMC_REF_ORDER || joined->d_raw)) {
            SMC_TRY(linear(ctx, m->xn, joined, m->qkv, B, mode, reuse ? m->qa : nullptr, s, m->bqkv[l]));
            SMC_TRY(launch_qkv_post(ctx, m, l, kc, vc, B, pos, s));
        } else {
            if (m->kv_q8) return smc_fail(ctx, SMC_E_UNSUPPORTED, "decode_step: a Q8_0 KV cache needs the joined Q/K/V path (layer %d has none usable in mode %d)", l, mode);
            SMC_TRY(linear(ctx, m->xn, m->wq[l], m->q, B, mode, reuse ? m->qa : nullptr, s, m->bq[l]));
            SMC_TRY(linear(ctx, m->xn, m->wk[l], m->k, B, mode, reuse ? m->qa : nullptr, s, m->bk[l]));
            SMC_TRY(linear(ctx, m->xn, m->wv[l], m->v, B, mode, reuse ? m->qa : nullptr, s, m->bv[l]));
            if (d.qk_norm) {
                SMC_TRY(smc_rmsnorm_dev(ctx, m->q, m->qnorm[l], m->q, B * nh, hd, d.eps, s));
                SMC_TRY(smc_rmsnorm_dev(ctx, m->k, m->knorm[l], m->k, B * nkv, hd, d.eps, s));
            }
            // every sequence is one token at position `pos`: [1, B*heads, headDim] with offset pos
            SMC_TRY(smc_rope_dev(ctx, m->q, 1, B * nh, hd, hd, pos, m->cosT, m->sinT, d.neox, s));
            SMC_TRY(smc_rope_dev(ctx, m->k, 1, B * nkv, hd, hd, pos, m->cosT, m->sinT, d.neox, s));
            SMC_TRY(smc_kv_append_dev(ctx, m->k, m->v, kc, vc, B, nkv, hd, pos, d.max_seq, s));
        }
        SMC_TRY(attend_decode(ctx, m, l, B, pos, scale, s));
        if (reuse) SMC_TRY(smc_quantize_q8_dev(ctx, m->att, B, qDim, m->qb, s));
        SMC_TRY(linear(ctx, m->att, m->wo[l], m->tmp, B, mode, reuse ? m->qb : nullptr, s, m->bo[l]));
        if (reuse) SMC_TRY(norm_into_q8(ctx, m, m->x, m->tmp, m->norm2[l], B, H, d.eps, s));
        else SMC_TRY(smc_add_rmsnorm_dev(ctx, m->x, m->tmp, m->norm2[l], m->xn, B, H, d.eps, s));
        SMC_TRY(linear(ctx, m->xn, m->wgu[l], m->gu, B, mode, reuse ? m->qa : nullptr, s, m->bgu[l]));
        if (mode == SMC_ACT_Q8 && B == 1 && F <= 8192 && !m->bdown[l] && m->wdown[l]->fast && smc_tma_supported(m->wdown[l], 1)) {
            // one row: SiLU(gate) * up is formed and quantised while the down-projection stages its activations
            SMC_TRY(smc_launch_gemv_tma_swiglu(ctx, m->gu, m->gu + F, m->wdown[l], m->tmp, s));
        } else {
            if (reuse) {  // SiLU-gate and quantisation in one pass: the fp32 product is not written out
                SMC_TRY(smc_launch_swiglu_quantize_q8(ctx, m->gu, m->gu + F, B, F, 2 * F, m->qb, s));
            } else {
                SMC_TRY(smc_swiglu_dev(ctx, m->gu, m->gu + F, m->act, B, F, 2 * F, s));
            }
            SMC_TRY(linear(ctx, m->act, m->wdown[l], m->tmp, B, mode, reuse ? m->qb : nullptr, s, m->bdown[l]));
        }
        // residual add, then the next block's first norm (the final norm after the last block)
        const float *next_norm = l + 1 < d.n_layers ? m->norm1[l + 1] : d.final_norm;
        if (reuse) SMC_TRY(norm_into_q8(ctx, m, m->x, m->tmp, next_norm, B, H, d.eps, s));
        else SMC_TRY(smc_add_rmsnorm_dev(ctx, m->x, m->tmp, next_norm, m->xn, B, H, d.eps, s));
    }
    SMC_TRY(linear(ctx, m->xn, d.lm_head, d_logits, B, mode, reuse ? m->qa : nullptr, s));
    if (d_argmax) SMC_TRY(smc_argmax_dev(ctx, d_logits, B, d.vocab, d_argmax, s));
    return SMC_OK;
}

// all_rows == 0: Transformer.ForwardLastLogits (logits of the last position); != 0: Transformer.Forward (logits of every
// position, [seqLen, vocab]), with the final-normed hidden states copied to d_hidden [seqLen, hidden] when given.
static int forward_tokens(smc_ctx *ctx, smc_model *m, const int *d_tokens, int seqLen, int seq, int pos, int mode, float *d_logits,
                          int *d_argmax, int all_rows, float *d_hidden, void *stream);

int smc_forward_last_logits(smc_ctx *ctx, smc_model *m, const int *d_tokens, int seqLen, int seq, int pos, int mode,
                            float *d_logits, int *d_argmax, void *stream)
{
    return forward_tokens(ctx, m, d_tokens, seqLen, seq, pos, mode, d_logits, d_argmax, 0, nullptr, stream);
}

int smc_forward_logits(smc_ctx *ctx, smc_model *m, const int *d_tokens, int seqLen, int seq, int pos, int mode, float *d_logits,
                       int *d_argmax, float *d_hidden, void *stream)
{
    return forward_tokens(ctx, m, d_tokens, seqLen, seq, pos, mode, d_logits, d_argmax, 1, d_hidden, stream);
}

static int forward_tokens(smc_ctx *ctx, smc_model *m, const int *d_tokens, int seqLen, int seq, int pos, int mode, float *d_logits,
                          int *d_argmax, int all_rows, float *d_hidden, void *stream)
{
    if (!ctx || !m || !d_tokens || !d_logits || seqLen <= 0) return smc_fail(ctx, SMC_E_INVALID, "forward_last_logits: bad arguments");
    if (seq < 0 || seq >= m->max_batch) return smc_fail(ctx, SMC_E_RANGE, "forward_last_logits: sequence %d outside [0, %d)", seq, m->max_batch);
    const smc_model_desc &d = m->d;
    if (pos < 0 || (long long)pos + seqLen > d.max_seq)  // KVCache.Update throws on overflow (KVCache.cs:89-91)
        return smc_fail(ctx, SMC_E_RANGE, "KVCache overflow: position %d + seqLen %d exceeds capacity %d", pos, seqLen, d.max_seq);
    if (mode != SMC_ACT_F32 && mode != SMC_ACT_Q8 && mode != SMC_REF_ORDER)
        return smc_fail(ctx, SMC_E_INVALID, "forward_last_logits: unknown mode %d", mode);
    if (d.head_dim != 64 && d.head_dim != 128)
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "forward_last_logits: headDim %d (64 and 128 are built)", d.head_dim);
    for (int l = 0; l < d.n_layers; ++l)
        if (!m->wqkv[l] || (mode == SMC_REF_ORDER && !m->wqkv[l]->d_raw))
            return smc_fail(ctx, SMC_E_UNSUPPORTED, "forward_last_logits: layer %d has no joined Q/K/V matrix usable in mode %d", l, mode);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int T = seqLen, H = d.hidden, nh = d.n_heads, nkv = d.n_kv_heads, hd = d.head_dim, F = d.ffn, qDim = nh * hd;
    int rc;
    if (T > m->rows) {  // first prompt chunk of this length: allocates (keep it outside stream capture)
        std::lock_guard<std::mutex> lock(ctx->mu_scratch);
        if ((rc = alloc_rows(ctx, m, T > m->max_batch ? T : m->max_batch))) return rc;
    }
    const float scale = 1.0f / sqrtf((float)hd);
    const size_t layer_stride = (size_t)m->max_batch * nkv * d.max_seq * hd, seq_off = (size_t)seq * nkv * d.max_seq * hd;
    const bool reuse = mode == SMC_ACT_Q8 && T > 1 && m->qa && m->qb;
    SMC_TRY(smc_embed_q8_0_dev(ctx, d.lm_head, d_tokens, T, m->x, s));
    if (reuse) SMC_TRY(norm_into_q8(ctx, m, m->x, nullptr, m->norm1[0], T, H, d.eps, s));
    else SMC_TRY(smc_rmsnorm_dev(ctx, m->x, m->norm1[0], m->xn, T, H, d.eps, s));
    for (int l = 0; l < d.n_layers; ++l) {
        float *kc = m->kcache + (size_t)l * layer_stride, *vc = m->vcache + (size_t)l * layer_stride;
        SMC_TRY(linear(ctx, m->xn, m->wqkv[l], m->qkv, T, mode, reuse ? m->qa : nullptr, s, m->bqkv[l]));
        // row t: per-head norm, rotation by position pos + t, K and V appended to sequence `seq`
        SMC_TRY(launch_qkv_post(ctx, m, l, kc, vc, T, pos, s, seq));
        if (m->kv_q8) {
            const size_t le = layer_elems(m);
            SMC_TRY(smc_launch_sdpa_q8_rows(ctx, m->q, m->kq8 + l * le + seq_off, m->kd8 + (l * le + seq_off) / 32, m->vq8 + l * le + seq_off,
                                            m->vd8 + (l * le + seq_off) / 32, m->att, 1, T, nh, nkv, hd, pos + T, d.max_seq, scale, s));
        } else {
            SMC_TRY(smc_launch_sdpa_prefill(ctx, m->q, kc + seq_off, vc + seq_off, m->att, T, nh, nkv, hd, pos, d.max_seq, scale, s));
        }
        if (reuse) SMC_TRY(smc_quantize_q8_dev(ctx, m->att, T, qDim, m->qb, s));
        SMC_TRY(linear(ctx, m->att, m->wo[l], m->tmp, T, mode, reuse ? m->qb : nullptr, s, m->bo[l]));
        if (reuse) SMC_TRY(norm_into_q8(ctx, m, m->x, m->tmp, m->norm2[l], T, H, d.eps, s));
        else SMC_TRY(smc_add_rmsnorm_dev(ctx, m->x, m->tmp, m->norm2[l], m->xn, T, H, d.eps, s));
        SMC_TRY(linear(ctx, m->xn, m->wgu[l], m->gu, T, mode, reuse ? m->qa : nullptr, s, m->bgu[l]));
        if (reuse) {
            SMC_TRY(smc_launch_swiglu_quantize_q8(ctx, m->gu, m->gu + F, T, F, 2 * F, m->qb, s));
        } else {
            SMC_TRY(smc_swiglu_dev(ctx, m->gu, m->gu + F, m->act, T, F, 2 * F, s));
        }
        SMC_TRY(linear(ctx, m->act, m->wdown[l], m->tmp, T, mode, reuse ? m->qb : nullptr, s, m->bdown[l]));
        const float *next_norm = l + 1 < d.n_layers ? m->norm1[l + 1] : d.final_norm;
        // the last block's output meets the LM head as fp32 rows; the others are only ever read quantised
        if (reuse && l + 1 < d.n_layers) SMC_TRY(norm_into_q8(ctx, m, m->x, m->tmp, next_norm, T, H, d.eps, s));
        else SMC_TRY(smc_add_rmsnorm_dev(ctx, m->x, m->tmp, next_norm, m->xn, T, H, d.eps, s));
    }
    if (all_rows) {  // Transformer.Forward: the LM head meets every position (draft verification reads all of them)
        if (d_hidden) SMC_CUDA(ctx, cudaMemcpyAsync(d_hidden, m->xn, (size_t)T * H * sizeof(float), cudaMemcpyDeviceToDevice, s));
        SMC_TRY(smc_qmatmul_dev(ctx, m->xn, d.lm_head, d_logits, T, mode, s));
        if (d_argmax) SMC_TRY(smc_argmax_dev(ctx, d_logits, T, d.vocab, d_argmax, s));
        return SMC_OK;
    }
    // only the last position's logits are formed (Transformer.ForwardLastLogits)
    SMC_TRY(smc_qmatmul_dev(ctx, m->xn + (size_t)(T - 1) * H, d.lm_head, d_logits, 1, mode, s));
    if (d_argmax) SMC_TRY(smc_argmax_dev(ctx, d_logits, 1, d.vocab, d_argmax, s));
#undef SMC_TRY
    return SMC_OK;
}

// ---- draft verification (MedusaGenerator.cs:262-283) and the Medusa heads (MedusaHeads.PredictQuantized, MedusaHeads.cs:80-130) ----
namespace {

// accepted = 1 + the longest prefix i with argmax[i] == draft[i + 1]  (token 0 was the model's own greedy choice)
__global__ void verify_greedy_kernel(const int *__restrict__ argmax, const int *__restrict__ draft, int heads, int *__restrict__ accepted)
{
    smc_grid_dep_sync();
    if (threadIdx.x || blockIdx.x) return;
    int a = 1;
    for (int i = 0; i < heads; ++i) {
        if (argmax[i] != draft[i + 1]) break;
        ++a;
    }
    *accepted = a;
}

// h'[head][i] = SiLU(b[i] + sum_j hidden[j] * W[j * H + i]), the sum taken sequentially in fp32 with unfused products as
// the reference's loop does; one thread per (head, i), consecutive threads read consecutive i of a weight row.
__global__ void __launch_bounds__(256) medusa_heads_kernel(const float *__restrict__ hidden, const float *__restrict__ w,
                                                          const float *__restrict__ b, float *__restrict__ out, int k, int H)
{
    smc_grid_dep_sync();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= k * H) return;
    const int head = t / H, i = t - head * H;
    const float *wh = w + (size_t)head * H * H;
    float sum = b[(size_t)head * H + i];
    for (int j = 0; j < H; ++j) sum = __fadd_rn(sum, __fmul_rn(hidden[j], wh[(size_t)j * H + i]));
    out[t] = __fdiv_rn(sum, 1.0f + expf(-sum));
}

}  // namespace

int smc_verify_greedy_dev(smc_ctx *ctx, const int *d_argmax, const int *d_draft, int heads, int *d_accepted, void *stream)
{
    if (!ctx || !d_argmax || !d_draft || !d_accepted || heads < 0) return smc_fail(ctx, SMC_E_INVALID, "verify_greedy: bad arguments");
    smc_launch_dep(ctx->use_pdl, verify_greedy_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), d_argmax, d_draft, heads, d_accepted);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_medusa_predict_dev(smc_ctx *ctx, const float *d_hidden, const float *d_head_w, const float *d_head_b, int k, int hidden,
                           const smc_weight *lm_head, float *d_work, int *d_tokens, void *stream)
{
    if (!ctx || !d_hidden || !d_head_w || !d_head_b || !lm_head || !d_work || !d_tokens || k < 0 || hidden <= 0)
        return smc_fail(ctx, SMC_E_INVALID, "medusa_predict: bad arguments");
    if (lm_head->K != hidden) return smc_fail(ctx, SMC_E_SIZE_MISMATCH, "medusa_predict: lm_head has K = %d, hidden is %d", lm_head->K, hidden);
    if (k == 0) return SMC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float *heads_out = d_work, *logits = d_work + (size_t)k * hidden;  // d_work holds k * (hidden + vocab) floats
    smc_launch_dep(ctx->use_pdl, medusa_heads_kernel, dim3((k * hidden + 255) / 256), dim3(256), 0, s, d_hidden, d_head_w, d_head_b, heads_out, k,
                   hidden);
    SMC_LAUNCH_CHECK(ctx);
    // QuantizedMatMulQ8_0(headsInput, rawEmbedding, logits, k, hidden, vocab) in the scalar tier's order, then Argmax per head
    int rc = smc_qmatmul_dev(ctx, heads_out, lm_head, logits, k, lm_head->d_raw ? SMC_REF_ORDER : SMC_ACT_F32, stream);
    if (rc) return rc;
    return smc_argmax_dev(ctx, logits, k, lm_head->N, d_tokens, stream);
}

}  // extern "C"
