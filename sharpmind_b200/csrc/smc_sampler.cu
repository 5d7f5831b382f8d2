// Token sampling on the device, so that a non-greedy decode step does not have to copy [batch, vocab] logits to the
// host: Sampler.Sample (SharpMind.Inference/Sampler.cs:16-46) and RepetitionPenalty.Apply
// (SharpMind.Inference/RepetitionPenalty.cs:15-27).
//
// Order of operations as in the reference: temperature, guarded softmax, min-p, top-k, top-p, normalise, one
// categorical draw.  The uniform number of the draw is an INPUT (one per row): the reference takes it from a .NET
// Random the host owns, so the host keeps drawing from that generator and hands the number over, and the device
// result is a pure function of (logits, config, r).
//
// One CTA of 1024 threads works on one row; every pass re-reads the row's probabilities from a caller-supplied work
// buffer (L2-resident: 600 KB for a 152k vocabulary).  Where the reference sorts or heap-selects, the kernel finds
// the cut as a threshold VALUE by building its bit pattern from the top bit down (31 counting or summing passes):
//   top-k  the largest t with  #{p >= t} >= k      (probabilities below t are zeroed)
//   top-p  the largest t with  sum{p >= t} >= topP (likewise)
// which keeps exactly the reference's set except that probabilities bit-equal to the cut value are all kept (the
// reference keeps as many of them as its heap / sort order happens to leave; which ones is not defined by its code).
// All reductions use one fixed tree, so a result does not change from run to run; sums are taken in another order than
// the reference's sequential loops, so a draw that lies within rounding (1e-6 of the total mass) of a boundary between
// two tokens may pick the neighbour.
#include "smc_common.cuh"

namespace {

constexpr int ST = 1024;  // threads per row

__device__ __forceinline__ float block_sum(float v, float *sh)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = sh[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}
__device__ __forceinline__ float block_max(float v, float *sh)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = sh[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    return t;
}
__device__ __forceinline__ int block_isum(int v, int *sh)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    int t = sh[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}
__device__ __forceinline__ int block_imin(int v, int *sh)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    int t = sh[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
    return t;
}
__device__ __forceinline__ int block_imax(int v, int *sh) { return -block_imin(-v, sh); }

__global__ void __launch_bounds__(ST) sample_kernel(const float *__restrict__ logits, float *__restrict__ work, int n, float inv_temp,
                                                    int topK, float topP, float minP, const float *__restrict__ uniform,
                                                    int *__restrict__ out)
{
    __shared__ float shf[32];
    __shared__ int shi[32];
    smc_grid_dep_sync();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float *x = logits + (size_t)row * n;
    float *p = work + (size_t)row * n;
    // temperature, and the softmax's guard: any infinity or NaN makes the row a point mass on token 0
    float mx = -INFINITY;
    int bad = 0;
    for (int i = tid; i < n; i += ST) {
        const float v = x[i] * inv_temp;
        bad |= (isinf(v) || isnan(v)) ? 1 : 0;
        mx = fmaxf(mx, v);
    }
    bad = block_isum(bad, shi);
    if (bad) {
        if (tid == 0) out[row] = 0;  // one token holds all the mass: every later step keeps it, every draw picks it
        return;
    }
    mx = block_max(mx, shf);
    float s = 0.f;
    for (int i = tid; i < n; i += ST) {
        float e = x[i] * inv_temp - mx;
        e = fminf(80.f, fmaxf(-80.f, e));
        const float v = expf(e);
        p[i] = v;
        s += v;
    }
    s = block_sum(s, shf);
    const float inv = __fdiv_rn(1.0f, s);
    float pmax = 0.f;
    for (int i = tid; i < n; i += ST) {
        const float v = p[i] * inv;
        p[i] = v;
        pmax = fmaxf(pmax, v);
    }
    if (minP > 0.f) {
        pmax = block_max(pmax, shf);
        const float thr = minP * pmax;
        for (int i = tid; i < n; i += ST)
            if (p[i] < thr) p[i] = 0.f;
    }
    __syncthreads();
    if (topK > 0 && topK < n) {
        unsigned cur = 0;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = cur | (1u << bit);
            int c = 0;
            for (int i = tid; i < n; i += ST) c += (__float_as_uint(p[i]) >= cand) ? 1 : 0;
            if (block_isum(c, shi) >= topK) cur = cand;
        }
        for (int i = tid; i < n; i += ST)
            if (__float_as_uint(p[i]) < cur) p[i] = 0.f;
        __syncthreads();
    }
    if (topP < 1.0f && topP > 0.f) {
        unsigned cur = 0;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = cur | (1u << bit);
            float m = 0.f;
            for (int i = tid; i < n; i += ST) {
                const float v = p[i];
                m += (__float_as_uint(v) >= cand) ? v : 0.f;
            }
            if (block_sum(m, shf) >= topP) cur = cand;
        }
        for (int i = tid; i < n; i += ST)
            if (__float_as_uint(p[i]) < cur) p[i] = 0.f;
        __syncthreads();
    }
    // normalise what is left
    float tot = 0.f;
    for (int i = tid; i < n; i += ST) tot += p[i];
    tot = block_sum(tot, shf);
    const float ninv = tot > 0.f ? __fdiv_rn(1.0f, tot) : 1.0f;
    // the draw: thread t owns the contiguous chunk [t*c, (t+1)*c); chunk sums in index order, a scan over the chunks,
    // and the thread whose chunk the number falls into walks it
    const int c = (n + ST - 1) / ST, b0 = min(n, tid * c), b1 = min(n, b0 + c);
    float cs = 0.f;
    int last_pos = -1;
    for (int i = b0; i < b1; ++i) {
        const float v = p[i] * ninv;
        cs += v;
        if (v > 0.f) last_pos = i;
    }
    // inclusive scan of the chunk sums: within a warp by shuffles, warp totals by warp 0
    float incl = cs;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += t;
    }
    __syncthreads();
    if ((tid & 31) == 31) shf[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
        float w = shf[tid];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, w, o);
            if (tid >= o) w += t;
        }
        shf[tid] = w;
    }
    __syncthreads();
    const float before = (tid >> 5) ? shf[(tid >> 5) - 1] : 0.f;
    incl += before;
    const float excl = incl - cs;
    const float r = uniform[row];
    const int first = block_imin((r <= incl && b1 > b0) ? tid : ST, shi);
    const int fallback = block_imax(last_pos, shi);  // the last token that kept any mass
    if (first == ST) {
        if (tid == 0) out[row] = fallback < 0 ? 0 : fallback;
        return;
    }
    if (tid == first) {
        float cum = excl;
        int tok = last_pos;  // rounding between the scan and this walk: the chunk's last token with mass
        for (int i = b0; i < b1; ++i) {
            cum += p[i] * ninv;
            if (r <= cum) {
                tok = i;
                break;
            }
        }
        out[row] = tok < 0 ? (fallback < 0 ? 0 : fallback) : tok;
    }
}

// RepetitionPenalty.Apply per row: every distinct id of the row's window scales its logit once.  ids < 0 or >= n are
// skipped (padding / out of range, as the reference skips them).
__global__ void __launch_bounds__(256) repetition_penalty_kernel(float *__restrict__ logits, int n, const int *__restrict__ ids,
                                                                 int window, float penalty)
{
    smc_grid_dep_sync();
    const int row = blockIdx.x;
    const int *w = ids + (size_t)row * window;
    float *x = logits + (size_t)row * n;
    for (int i = threadIdx.x; i < window; i += blockDim.x) {
        const int id = w[i];
        if (id < 0 || id >= n) continue;
        bool seen = false;
        for (int j = 0; j < i && !seen; ++j) seen = w[j] == id;  // the first occurrence applies the penalty
        if (seen) continue;
        const float v = x[id];
        x[id] = v >= 0.f ? __fdiv_rn(v, penalty) : v * penalty;
    }
}

}  // namespace

extern "C" {

int smc_sample_dev(smc_ctx *ctx, const float *d_logits, int rows, int n, const smc_sampling *cfg, const float *d_uniform,
                   float *d_work, int *d_tokens, void *stream)
{
    if (!ctx || !d_logits || !cfg || !d_tokens || rows < 0 || n <= 0) return smc_fail(ctx, SMC_E_INVALID, "sample: bad arguments");
    if (rows == 0) return SMC_OK;
    if (cfg->temperature <= 0.f)  // the greedy shortcut (Sampler.cs:19-20)
        return smc_argmax_dev(ctx, d_logits, rows, n, d_tokens, stream);
    if (!d_uniform || !d_work) return smc_fail(ctx, SMC_E_INVALID, "sample: temperature > 0 needs the uniform numbers and a work buffer");
    smc_launch_dep(ctx->use_pdl, sample_kernel, dim3(rows), dim3(ST), 0, static_cast<cudaStream_t>(stream), d_logits, d_work, n,
                   1.0f / cfg->temperature, cfg->top_k, cfg->top_p, cfg->min_p, d_uniform, d_tokens);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_repetition_penalty_dev(smc_ctx *ctx, float *d_logits, int rows, int n, const int *d_ids, int window, float penalty,
                               void *stream)
{
    if (!ctx || !d_logits || !d_ids || rows < 0 || n <= 0 || window < 0 || !(penalty > 0.f))
        return smc_fail(ctx, SMC_E_INVALID, "repetition_penalty: bad arguments");
    if (rows == 0 || window == 0 || penalty == 1.0f) return SMC_OK;
    smc_launch_dep(ctx->use_pdl, repetition_penalty_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), d_logits, n,
                   d_ids, window, penalty);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

}  // extern "C"
