// fp32 attention over an fp32 KV cache.
//
//  * sdpa_decode_split_kernel: one query token per sequence (decode).  The cache
//    sweep is the only traffic that matters (2 * kvLen * headDim * 4 bytes per KV head), so the
//    key range is split across CTAs to fill the GPU at batch 1, the query heads that share a KV
//    head are processed together (K and V are read once per group), and eight lanes share a key so
//    that every load is a coalesced 128-bit access.  Each eight-lane group keeps its own online-
//    softmax state; states are merged in shared memory per CTA, and the CTA that finishes a (sequence, KV head)
//    last merges the CTAs' records in split order.
//  * sdpa_tile_kernel: any seqLen / kvLen / headDim <= 256 / strides / causal / ALiBi, written in the
//    reference's own order (tiles of 64 keys, sequential fp32 dot, running max and sum), used by the
//    host-pointer `attention` slot and for head sizes the split kernel does not take.
//
// References: ScaledDotProductFlash{Scalar,FMA} SharpMind.Model/Layers/Attention/AttentionKernels.cs:315-475,
// AttentionLayer.Forward's per-(batch, head) loop AttentionLayer.cs:326-413, KVCache layout and Update
// SharpMind.Model/KVCache.cs:13-36,84-150.
#include <math.h>

#include "smc_common.cuh"

namespace {

constexpr int LPK = 8;          // lanes per key
constexpr int MAXG = 8;         // query heads per KV head handled by one CTA pass
constexpr int SPLIT_THREADS = 128;

constexpr int MERGE_MAX_SPLITS = 128;

// Per (batch, head) the split kernel leaves `splits` partial results laid out for this merge:
// [splits][4] floats (m, l, -, -) followed by [splits][HD] partial outputs, every row 16-byte aligned.
__host__ __device__ inline size_t head_record_floats(int splits, int hd) { return (size_t)splits * (hd + 4); }

// Combines the records of the G consecutive heads of one CTA's (sequence, KV head):
// out = sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M).  Built for few round trips to L2 (the records were written by
// other CTAs of the same launch): one for all (m, l) pairs, then every thread streams float4 pieces of the partial
// outputs of its (head, quarter of the dims, subset of splits) with the loads of a subset in flight together.
// The subsets (split s belongs to subset s mod P) are added in subset order, each in split order: the result
// depends on the split count only.  `scratch` (16-byte aligned) holds 3 * G * splits + 3 + (blockDim / (HD / 4)) * HD floats.
template <int G, int HD>
__device__ __forceinline__ void merge_heads(const float *rec0, float *out0, int splits, float *scratch)
{
    constexpr int NQ = HD / 4;                   // float4 pieces per head
    const int tid = threadIdx.x, nthr = blockDim.x;
    float *sm_m = scratch, *sm_l = sm_m + G * splits, *sm_w = sm_l + G * splits;
    float *sm_o = scratch + ((3 * G * splits + 3) & ~3);  // float4 rows: 16-byte aligned (scratch itself is)
    __shared__ float sL[G];
    const size_t hstride = head_record_floats(splits, HD);
    for (int i = tid; i < G * splits; i += nthr) {
        const int g = i / splits, sp = i - g * splits;
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(rec0 + g * hstride + 4 * sp));
        sm_m[i] = ml.x, sm_l[i] = ml.y;
    }
    __syncthreads();
    const int lane = tid & 31, warp = tid >> 5;
    for (int g = warp; g < G; g += nthr >> 5) {  // one warp per head: maximum, weights, then the denominator in split order
        float m = -INFINITY;
        for (int sp = lane; sp < splits; sp += 32) m = fmaxf(m, sm_m[g * splits + sp]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        for (int sp = lane; sp < splits; sp += 32) {
            const float ms = sm_m[g * splits + sp];
            sm_w[g * splits + sp] = (ms == -INFINITY) ? 0.f : expf(ms - m);
        }
        __syncwarp();
        if (lane == 0) {
            float L = 0.f;
            for (int sp = 0; sp < splits; ++sp) L = fmaf(sm_l[g * splits + sp], sm_w[g * splits + sp], L);
            sL[g] = L;
        }
    }
    __syncthreads();
    const int groups = nthr / NQ;                // thread groups of one head's width
    const int P = groups >= G ? groups / G : 1;  // split subsets per head
    const int gid = tid / NQ, quad = tid - gid * NQ;
    if (gid < G * P) {  // one (head, subset) per thread
        const int g = gid % G, part = gid / G;
        const float *src = rec0 + g * hstride + 4 * (size_t)splits + 4 * quad;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int sp = part;
        for (; sp + 3 * P < splits; sp += 4 * P) {
            const float4 a = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)sp * HD));
            const float4 b = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)(sp + P) * HD));
            const float4 c = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)(sp + 2 * P) * HD));
            const float4 e = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)(sp + 3 * P) * HD));
            const float wa = sm_w[g * splits + sp], wb = sm_w[g * splits + sp + P], wc = sm_w[g * splits + sp + 2 * P],
                        we = sm_w[g * splits + sp + 3 * P];
            acc.x = fmaf(a.x, wa, acc.x), acc.y = fmaf(a.y, wa, acc.y), acc.z = fmaf(a.z, wa, acc.z), acc.w = fmaf(a.w, wa, acc.w);
            acc.x = fmaf(b.x, wb, acc.x), acc.y = fmaf(b.y, wb, acc.y), acc.z = fmaf(b.z, wb, acc.z), acc.w = fmaf(b.w, wb, acc.w);
            acc.x = fmaf(c.x, wc, acc.x), acc.y = fmaf(c.y, wc, acc.y), acc.z = fmaf(c.z, wc, acc.z), acc.w = fmaf(c.w, wc, acc.w);
            acc.x = fmaf(e.x, we, acc.x), acc.y = fmaf(e.y, we, acc.y), acc.z = fmaf(e.z, we, acc.z), acc.w = fmaf(e.w, we, acc.w);
        }
        for (; sp < splits; sp += P) {
            const float4 a = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)sp * HD));
            const float wa = sm_w[g * splits + sp];
            acc.x = fmaf(a.x, wa, acc.x), acc.y = fmaf(a.y, wa, acc.y), acc.z = fmaf(a.z, wa, acc.z), acc.w = fmaf(a.w, wa, acc.w);
        }
        *reinterpret_cast<float4 *>(sm_o + ((size_t)part * G + g) * HD + 4 * quad) = acc;
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += nthr) {
        const int g = i / HD, d = i - g * HD;
        float O = sm_o[(size_t)g * HD + d];
        for (int part = 1; part < P; ++part) O += sm_o[((size_t)part * G + g) * HD + d];
        const float L = sL[g];
        out0[(size_t)g * HD + d] = L > 0.f ? __fdiv_rn(O, L) : 0.f;
    }
}

// partial results per (batch, head): see head_record_floats
// Q8: the cache holds Q8_0 rows (QuantizedKVCache, SharpMind.Model/QuantizedKVCache.cs) as two planes per tensor: int8
// quants [.., maxSeq, HD] in kc / vc and fp16 block scales [.., maxSeq, HD/32] in kd / vd.  A lane's dims lie inside one
// 32-element block; bytes become floats through a PRMT + FADD pair, and the block scale multiplies the lane's partial
// dot (keys) or the softmax weight (values) once instead of every element: what ScaledDotProductFlashQ8_0*
// (AttentionKernels.cs:489-813) computes, at a quarter of the fp32 cache's bytes.
template <int DPL, int G, bool Q8>  // DPL = dims per lane = headDim / 8, G = query heads per KV head
__global__ void __launch_bounds__(SPLIT_THREADS) sdpa_decode_split_kernel(
    const float *__restrict__ q, const void *__restrict__ kc_, const void *__restrict__ vc_, const __half *__restrict__ kd,
    const __half *__restrict__ vd, float *part, int heads, int kvHeads, int kvLen, int maxSeq, float scale, int splits,
    float *__restrict__ out, unsigned *tickets, int hshare)
{
    // kvHeads counts virtual KV heads: `hshare` consecutive ones read the same cached head, each for its own G
    // query heads (a group of 8 query heads runs as 4 x 2, so that the per-thread state of G heads stays in registers)
    constexpr int HD = DPL * LPK;
    smc_grid_dep_sync();
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grp = lane / LPK, sub = lane % LPK;        // 4 key groups per warp
    const int ngroups = (SPLIT_THREADS / 32) * (32 / LPK);
    const int gid = warp * (32 / LPK) + grp;

    const int chunk = (kvLen + splits - 1) / splits;
    const int k0 = split * chunk, k1 = min(kvLen, k0 + chunk);

    const size_t cached_head = (size_t)b * (kvHeads / hshare) + kvh / hshare;
    const float *kbase = static_cast<const float *>(kc_) + cached_head * (size_t)maxSeq * HD;
    const float *vbase = static_cast<const float *>(vc_) + cached_head * (size_t)maxSeq * HD;
    const int8_t *kq = static_cast<const int8_t *>(kc_) + cached_head * (size_t)maxSeq * HD + sub * DPL;
    const int8_t *vq = static_cast<const int8_t *>(vc_) + cached_head * (size_t)maxSeq * HD + sub * DPL;
    const __half *kdb = Q8 ? kd + cached_head * (size_t)maxSeq * (HD / 32) + (sub * DPL) / 32 : nullptr;
    const __half *vdb = Q8 ? vd + cached_head * (size_t)maxSeq * (HD / 32) + (sub * DPL) / 32 : nullptr;

    float qr[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float *qp = q + ((size_t)b * heads + (size_t)kvh * G + g) * HD + sub * DPL;
#pragma unroll
        for (int d = 0; d < DPL; d += 4) {
            float4 t = *reinterpret_cast<const float4 *>(qp + d);
            qr[g][d] = t.x, qr[g][d + 1] = t.y, qr[g][d + 2] = t.z, qr[g][d + 3] = t.w;
        }
    }
    float m[G], l[G], o[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[g][d] = 0.f;
    }

    // every lane group runs the same number of iterations so the shuffles below stay converged
    const int iters = k1 > k0 ? (k1 - k0 + ngroups - 1) / ngroups : 0;
    for (int it = 0; it < iters; ++it) {
        const int j = k0 + it * ngroups + gid;
        const bool live = j < k1;
        const int jj = live ? j : k0;
        float kr[DPL], vr[DPL];
        float dk = 1.f, dv = 1.f;  // block scales of the lane's dims (Q8)
        if (Q8) {
            uint32_t kw[DPL / 4], vw[DPL / 4];
            if (DPL == 16) {
                const uint4 a = smc_ldg_stream16(kq + (size_t)jj * HD), c = smc_ldg_stream16(vq + (size_t)jj * HD);
                kw[0] = a.x, kw[1] = a.y, kw[DPL / 4 - 2] = a.z, kw[DPL / 4 - 1] = a.w;
                vw[0] = c.x, vw[1] = c.y, vw[DPL / 4 - 2] = c.z, vw[DPL / 4 - 1] = c.w;
            } else {
                const uint2 a = smc_ldg_stream8(kq + (size_t)jj * HD), c = smc_ldg_stream8(vq + (size_t)jj * HD);
                kw[0] = a.x, kw[1] = a.y, vw[0] = c.x, vw[1] = c.y;
            }
            dk = __half2float(__ldg(kdb + (size_t)jj * (HD / 32)));
            dv = __half2float(__ldg(vdb + (size_t)jj * (HD / 32)));
#pragma unroll
            for (int d = 0; d < DPL; ++d) {  // signed byte -> float: flip to unsigned, magic-number convert, take 128 off
                kr[d] = __uint_as_float(__byte_perm(kw[d >> 2] ^ 0x80808080u, 0x4B000000u, 0x7540u | (d & 3))) - 8388736.0f;
                vr[d] = __uint_as_float(__byte_perm(vw[d >> 2] ^ 0x80808080u, 0x4B000000u, 0x7540u | (d & 3))) - 8388736.0f;
            }
        } else {
#pragma unroll
            for (int d = 0; d < DPL; d += 4) {
                float4 t = smc_ldg_stream16f(kbase + (size_t)jj * HD + sub * DPL + d);
                kr[d] = t.x, kr[d + 1] = t.y, kr[d + 2] = t.z, kr[d + 3] = t.w;
                float4 u = smc_ldg_stream16f(vbase + (size_t)jj * HD + sub * DPL + d);
                vr[d] = u.x, vr[d + 1] = u.y, vr[d + 2] = u.z, vr[d + 3] = u.w;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float dot = 0.f;
#pragma unroll
            for (int d = 0; d < DPL; ++d) dot = fmaf(qr[g][d], kr[d], dot);
            if (Q8) dot *= dk;
            dot = smc_group_sum<LPK>(dot);
            if (live) {
                float s = dot * scale;
                float mn = fmaxf(m[g], s);
                float alpha = expf(m[g] - mn);  // exp(-inf) = 0 on the first key
                float p = expf(s - mn);
                l[g] = fmaf(l[g], alpha, p);
                const float pv = Q8 ? p * dv : p;
#pragma unroll
                for (int d = 0; d < DPL; ++d) o[g][d] = fmaf(pv, vr[d], o[g][d] * alpha);
                m[g] = mn;
            }
        }
    }

    // merge the lane groups of the CTA: shared memory holds (m, l) per group and o per group
    extern __shared__ __align__(16) float sm[];
    float *sm_m = sm;                                   // [ngroups][G]
    float *sm_l = sm_m + ngroups * G;                   // [ngroups][G]
    float *sm_o = sm_l + ngroups * G;                   // [ngroups][G][HD]
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (sub == 0) sm_m[gid * G + g] = m[g], sm_l[gid * G + g] = l[g];
#pragma unroll
        for (int d = 0; d < DPL; ++d) sm_o[((size_t)gid * G + g) * HD + sub * DPL + d] = o[g][d];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * HD; idx += SPLIT_THREADS) {
        int g = idx / HD, d = idx % HD;
        float M = -INFINITY;
        for (int r = 0; r < ngroups; ++r) M = fmaxf(M, sm_m[r * G + g]);
        float L = 0.f, O = 0.f;
        for (int r = 0; r < ngroups; ++r) {
            float mr = sm_m[r * G + g];
            float w = (mr == -INFINITY) ? 0.f : expf(mr - M);
            L = fmaf(sm_l[r * G + g], w, L);
            O = fmaf(sm_o[((size_t)r * G + g) * HD + d], w, O);
        }
        float *rec = part + ((size_t)b * heads + (size_t)kvh * G + g) * head_record_floats(splits, HD);
        if (d == 0) rec[4 * split] = M, rec[4 * split + 1] = L;
        rec[4 * (size_t)splits + (size_t)split * HD + d] = O;
    }
    // the CTA that finishes a (sequence, KV head) last combines the records of its query heads
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        unsigned *tk = tickets + (size_t)b * kvHeads + kvh;
        s_last = atomicAdd(tk, 1u) == (unsigned)splits - 1 ? 1 : 0;
        if (s_last) *tk = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // the shared memory of the group merge above is free again (every thread passed the barrier after its last read)
    const size_t head0 = (size_t)b * heads + (size_t)kvh * G;
    merge_heads<G, HD>(part + head0 * head_record_floats(splits, HD), out + head0 * HD, splits, sm);
}

// Reference-order attention: one CTA per query row, 256 threads, tiles of 64 keys.
__global__ void __launch_bounds__(256) sdpa_tile_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                                        const float *__restrict__ v, float *__restrict__ out, int seqLen,
                                                        int kvLen, int hd, float scale, int causal, int qStride,
                                                        int oStride, float alibi)
{
    __shared__ float tile[64];
    __shared__ float sq[256];
    __shared__ float stat[4];  // newMax, scaleOld, newL
    const int i = blockIdx.x, t = threadIdx.x;
    const float *qi = q + (size_t)i * qStride;
    const int queryBase = causal ? kvLen - seqLen : 0;
    const int absQ = queryBase + i;
    const int eff = causal ? min(absQ + 1, kvLen) : kvLen;
    if (t < hd) sq[t] = qi[t];
    float o = 0.f;
    float mMax = -INFINITY, lSum = 0.f;  // kept identically by every thread
    __syncthreads();
    for (int start = 0; start < eff; start += 64) {
        const int len = min(64, eff - start);
        if (t < len) {
            const float *kj = k + (size_t)(start + t) * hd;
            float dot = 0.f;
            for (int d = 0; d < hd; ++d) dot = __fadd_rn(dot, __fmul_rn(sq[d], kj[d]));
            dot = __fsub_rn(__fmul_rn(dot, scale), __fmul_rn(alibi, (float)(absQ - (start + t))));
            tile[t] = dot;
        }
        __syncthreads();
        if (t == 0) {
            float tmax = -INFINITY;
            for (int j = 0; j < len; ++j) tmax = fmaxf(tmax, tile[j]);
            float newMax = fmaxf(mMax, tmax);
            float scaleOld = expf(mMax - newMax);
            float scaleNew = 0.f;
            for (int j = 0; j < len; ++j) {
                tile[j] = expf(tile[j] - newMax);
                scaleNew = __fadd_rn(scaleNew, tile[j]);
            }
            stat[0] = newMax;
            stat[1] = scaleOld;
            stat[2] = __fadd_rn(__fmul_rn(scaleOld, lSum), scaleNew);
        }
        __syncthreads();
        mMax = stat[0];
        lSum = stat[2];
        if (t < hd) {
            o = __fmul_rn(o, stat[1]);
            for (int j = 0; j < len; ++j) o = __fadd_rn(o, __fmul_rn(tile[j], v[(size_t)(start + j) * hd + t]));
        }
        __syncthreads();
    }
    if (t < hd) out[(size_t)i * oStride + t] = lSum > 0.f ? __fdiv_rn(o, lSum) : 0.f;
}

__global__ void kv_append_kernel(const float *__restrict__ k, const float *__restrict__ v, float *__restrict__ kc,
                                 float *__restrict__ vc, int batch, int kvHeads, int hd, int pos, int maxSeq)
{
    long long total = (long long)batch * kvHeads * hd;
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= total) return;
    int d = (int)(t % hd);
    long long bh = t / hd;  // b * kvHeads + h
    size_t dst = ((size_t)bh * maxSeq + pos) * hd + d;
    kc[dst] = k[t];
    vc[dst] = v[t];
}

template <int DPL, bool Q8>
int launch_split_g(smc_ctx *ctx, int G, dim3 grid, size_t smem, cudaStream_t s, const float *q, const void *k,
                   const void *v, const __half *kd, const __half *vd, float *part, int heads, int kvHeads, int kvLen, int maxSeq,
                   float scale, int splits, float *out, unsigned *tickets, int hshare)
{
#define SMC_SPLIT_CASE(GV)                                                                                         \
    case GV:                                                                                                       \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(sdpa_decode_split_kernel<DPL, GV, Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                 (int)smem);                                                                       \
        smc_launch_dep(ctx->use_pdl, sdpa_decode_split_kernel<DPL, GV, Q8>, grid, dim3(SPLIT_THREADS), smem, s, q, k, v, kd, vd, part, heads, \
                       kvHeads, kvLen, maxSeq, scale, splits, out, tickets, hshare);        \
        break;
    switch (G) {
        SMC_SPLIT_CASE(1)
        SMC_SPLIT_CASE(2)
        SMC_SPLIT_CASE(4)
    default: return smc_fail(ctx, SMC_E_UNSUPPORTED, "sdpa_decode: %d query heads per KV head", G);
    }
#undef SMC_SPLIT_CASE
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// Causal attention of T consecutive query tokens of ONE sequence against its fp32 cache (the new tokens' K and V
// already appended): query t sits at position pos0 + t and sees keys 0 .. pos0 + t.  A CTA takes one head and
// 8 * R consecutive query rows, R per warp; K and V go through shared memory in tiles of 32 keys shared by all of
// them (rows padded to HD + 4 floats: a lane's 16-byte reads of its own key row, and all lanes' reads of one value
// row, are conflict free).  Lane j scores key j of the tile for each of the warp's R rows from one read of the key
// (the R query rows are broadcast reads), the running max / sum are per row, and lane i accumulates output dims
// 4i .. 4i + 3 (HD = 128) or 2i, 2i + 1 (HD = 64) of every row from one read of the value row.
template <int HD, int R>
__global__ void __launch_bounds__(256) sdpa_prefill_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                                                           const float *__restrict__ vc, float *__restrict__ out, int T,
                                                           int nh, int nkv, int pos0, int maxSeq, float scale)
{
    constexpr int LD = HD + 4, DPL = HD / 32, ROWS = 8 * R;
    extern __shared__ __align__(16) float sm_att[];
    float *sk = sm_att, *sv = sk + 32 * LD, *sq = sv + 32 * LD;  // sq [ROWS][HD]
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y, kvh = h / (nh / nkv);
    const int t0 = blockIdx.x * ROWS, tw = t0 + warp * R;  // first row of the CTA, of this warp
    const int cta_len = pos0 + min(T, t0 + ROWS);
    int len[R];  // keys row r sees; 0 for rows past the chunk
#pragma unroll
    for (int r = 0; r < R; ++r) len[r] = tw + r < T ? pos0 + tw + r + 1 : 0;
    const int warp_len = tw < T ? pos0 + min(T, tw + R) : 0;
    const float *kbase = kc + (size_t)kvh * maxSeq * HD, *vbase = vc + (size_t)kvh * maxSeq * HD;
    for (int e = threadIdx.x; e < ROWS * HD; e += 256) {
        const int r = e / HD, d = e % HD;
        sq[e] = t0 + r < T ? q[((size_t)(t0 + r) * nh + h) * HD + d] : 0.f;
    }
    float o[R][DPL], m[R], l[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m[r] = -INFINITY, l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[r][i] = 0.f;
    }
    for (int start = 0; start < cta_len; start += 32) {
        __syncthreads();  // the previous tile has been consumed (and sq is written before the first use)
        for (int e = threadIdx.x; e < 32 * (HD / 4); e += 256) {
            const int r = e / (HD / 4), c = e % (HD / 4);
            float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
            if (start + r < cta_len) {
                kk = *reinterpret_cast<const float4 *>(kbase + (size_t)(start + r) * HD + 4 * c);
                vv = *reinterpret_cast<const float4 *>(vbase + (size_t)(start + r) * HD + 4 * c);
            }
            *reinterpret_cast<float4 *>(sk + r * LD + 4 * c) = kk;
            *reinterpret_cast<float4 *>(sv + r * LD + 4 * c) = vv;
        }
        __syncthreads();
        if (start >= warp_len) continue;  // warp uniform: every row's causal bound lies before the tile
        float dot[R];
#pragma unroll
        for (int r = 0; r < R; ++r) dot[r] = 0.f;
#pragma unroll 4
        for (int c = 0; c < HD / 4; ++c) {
            const float4 b = *reinterpret_cast<const float4 *>(sk + lane * LD + 4 * c);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float4 a = *reinterpret_cast<const float4 *>(sq + (warp * R + r) * HD + 4 * c);
                dot[r] = fmaf(a.x, b.x, dot[r]), dot[r] = fmaf(a.y, b.y, dot[r]);
                dot[r] = fmaf(a.z, b.z, dot[r]), dot[r] = fmaf(a.w, b.w, dot[r]);
            }
        }
        float p[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            p[r] = 0.f;
            if (start >= len[r]) continue;  // warp uniform per row
            const bool valid = start + lane < len[r];
            const float sc = valid ? dot[r] * scale : -INFINITY;
            float tmax = sc;
#pragma unroll
            for (int x = 16; x > 0; x >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, x));
            const float nm = fmaxf(m[r], tmax);  // finite: key `start` is inside the bound
            p[r] = valid ? expf(sc - nm) : 0.f;
            float ps = p[r];
#pragma unroll
            for (int x = 16; x > 0; x >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, x);
            const float corr = expf(m[r] - nm);  // exp(-inf) = 0 on the first tile
            l[r] = fmaf(l[r], corr, ps);
            m[r] = nm;
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[r][i] *= corr;
        }
#pragma unroll 4
        for (int j = 0; j < 32; ++j) {
            float vv[4];
            if (DPL == 4) {
                const float4 t4 = *reinterpret_cast<const float4 *>(sv + j * LD + 4 * lane);
                vv[0] = t4.x, vv[1] = t4.y, vv[2] = t4.z, vv[3] = t4.w;
            } else {
                const float2 t2 = *reinterpret_cast<const float2 *>(sv + j * LD + 2 * lane);
                vv[0] = t2.x, vv[1] = t2.y, vv[2] = vv[3] = 0.f;
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float pj = __shfl_sync(0xffffffffu, p[r], j);
#pragma unroll
                for (int i = 0; i < DPL; ++i) o[r][i] = fmaf(pj, vv[i], o[r][i]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (tw + r >= T) continue;
        float *dst = out + ((size_t)(tw + r) * nh + h) * HD + DPL * lane;
#pragma unroll
        for (int i = 0; i < DPL; ++i) dst[i] = l[r] > 0.f ? o[r][i] / l[r] : 0.f;
    }
}

}  // namespace

int smc_launch_sdpa_prefill(smc_ctx *ctx, const float *q, const float *kc, const float *vc, float *out, int T, int nh, int nkv,
                            int hd, int pos0, int maxSeq, float scale, cudaStream_t s)
{
    if (hd != 64 && hd != 128) return smc_fail(ctx, SMC_E_UNSUPPORTED, "prefill attention needs headDim 64 or 128, got %d", hd);
    if (nh % nkv) return smc_fail(ctx, SMC_E_INVALID, "prefill attention: heads %d not a multiple of KV heads %d", nh, nkv);
    // the contractions on the tensor cores (bf16 MMAs on three-way split operands: fp32-grade accuracy) unless switched off
    if (ctx->attn_mma && smc_sdpa_prefill_mma_supported(nh, nkv, hd))
        return smc_launch_sdpa_prefill_mma(ctx, q, kc, vc, out, T, nh, nkv, hd, pos0, maxSeq, scale, s);
    // query rows per warp: four, or two while that leaves fewer than three CTAs per SM (a CTA waits on its K/V
    // tile loads with nothing else to do, so the SM needs other CTAs to run meanwhile)
    auto go = [&](auto kernel, int R) {
        const dim3 grid((T + 8 * R - 1) / (8 * R), nh);
        const size_t smem = ((size_t)2 * 32 * (hd + 4) + (size_t)8 * R * hd) * sizeof(float);
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        smc_launch_dep(ctx->use_pdl, kernel, grid, dim3(256), smem, s, q, kc, vc, out, T, nh, nkv, pos0, maxSeq, scale);
    };
    const bool four = (long long)((T + 31) / 32) * nh >= 3LL * ctx->sm_count;
    if (hd == 128) four ? go(sdpa_prefill_kernel<128, 4>, 4) : go(sdpa_prefill_kernel<128, 2>, 2);
    else four ? go(sdpa_prefill_kernel<64, 4>, 4) : go(sdpa_prefill_kernel<64, 2>, 2);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_launch_sdpa_tile(smc_ctx *ctx, const float *q, const float *k, const float *v, float *o, int seqLen, int kvLen,
                         int hd, float scale, int causal, int qStride, int oStride, float alibi, cudaStream_t s)
{
    sdpa_tile_kernel<<<seqLen, 256, 0, s>>>(q, k, v, o, seqLen, kvLen, hd, scale, causal, qStride, oStride, alibi);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// Scratch of the split-KV decode attention: a fixed header of tickets (one per (sequence, virtual KV head), zeroed at
// allocation and left at zero by every launch), then one record per (sequence, head, split).  It is sized for the most
// splits the shape can ever use (the count grows with kvLen until the whole cache of maxSeq positions is in play), so
// that decoding further into a sequence never reallocates: growth happens only for a larger batch, more heads or a
// larger maxSeq, after a device-wide synchronisation (make the first call of such a shape outside stream capture;
// smc_model_create reserves for the model's own shape).  Caller holds ctx->mu_scratch.
constexpr size_t TICKET_BYTES = 65536 * sizeof(unsigned);
static int reserve_split_scratch(smc_ctx *ctx, int batch, int heads, int kvHeadsVirtual, int headDim, int maxSeq)
{
    const int pairs = batch * kvHeadsVirtual;
    if ((size_t)pairs > 65536) return smc_fail(ctx, SMC_E_RANGE, "sdpa_decode: more than 65536 (sequence, KV head) pairs");
    int worst = (2 * ctx->sm_count + pairs - 1) / pairs;
    if (worst > (maxSeq + 63) / 64) worst = (maxSeq + 63) / 64;
    if (worst < 1) worst = 1;
    if (worst > MERGE_MAX_SPLITS) worst = MERGE_MAX_SPLITS;
    const size_t need = TICKET_BYTES + (size_t)batch * heads * head_record_floats(worst, headDim) * sizeof(float);
    if (need <= ctx->attn_part_cap) return SMC_OK;
    if (ctx->d_attn_part) {
        cudaDeviceSynchronize();
        cudaFree(ctx->d_attn_part);
    }
    ctx->d_attn_part = nullptr;
    ctx->attn_part_cap = 0;
    SMC_CUDA(ctx, cudaMalloc(&ctx->d_attn_part, need));
    SMC_CUDA(ctx, cudaMemset(ctx->d_attn_part, 0, TICKET_BYTES));
    ctx->attn_part_cap = need;
    return SMC_OK;
}

// Reserves the decode attention's scratch for every batch size up to `max_batch` of a model shape.
int smc_sdpa_decode_reserve(smc_ctx *ctx, int max_batch, int heads, int kvHeads, int headDim, int maxSeq)
{
    const int Gall = heads / kvHeads;
    const int G = Gall > 2 ? (Gall % 2 == 0 ? 2 : 1) : Gall;
    const int kvVirtual = kvHeads * (Gall / G);
    std::lock_guard<std::mutex> lock(ctx->mu_scratch);
    for (int b = 1; b <= max_batch; ++b) {  // the record count is not monotonic in the batch size (fewer splits per pair)
        int rc = reserve_split_scratch(ctx, b, heads, kvVirtual, headDim, maxSeq);
        if (rc) return rc;
    }
    return SMC_OK;
}

extern "C" {

int smc_sdpa_decode_dev(smc_ctx *ctx, const float *d_q, const float *d_k, const float *d_v, float *d_out, int batch,
                        int heads, int kvHeads, int headDim, int kvLen, int maxSeq, float scale, void *stream)
{
    return smc_sdpa_decode_any(ctx, d_q, d_k, d_v, nullptr, nullptr, d_out, batch, heads, kvHeads, headDim, kvLen, maxSeq, scale,
                               static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// fp32 cache (d_kd == null: d_k / d_v are fp32 [batch, kvHeads, maxSeq, headDim]) or Q8_0 cache (d_k / d_v are the int8
// planes of that shape, d_kd / d_vd the fp16 block scales [batch, kvHeads, maxSeq, headDim / 32]).
int smc_sdpa_decode_any(smc_ctx *ctx, const float *d_q, const void *d_k, const void *d_v, const __half *d_kd, const __half *d_vd,
                        float *d_out, int batch, int heads, int kvHeads, int headDim, int kvLen, int maxSeq, float scale,
                        cudaStream_t stream)
{
    const bool q8 = d_kd != nullptr;
    if (!ctx || !d_q || !d_k || !d_v || !d_out || batch < 0 || heads <= 0 || kvHeads <= 0 || heads % kvHeads ||
        headDim <= 0 || kvLen <= 0 || kvLen > maxSeq || (q8 && !d_vd))
        return smc_fail(ctx, SMC_E_INVALID, "sdpa_decode: bad arguments");
    if (headDim > 256) return smc_fail(ctx, SMC_E_RANGE, "sdpa_decode: headDim %d exceeds 256", headDim);
    if (batch == 0) return SMC_OK;
    cudaStream_t s = stream;
    const int Gall = heads / kvHeads;
    // query heads per CTA: at most two, so that the running state of its heads stays in registers; a larger group is
    // spread over CTAs that read the same cached head (the second read comes from L2).  Measured on a Llama-3-8B
    // shape (4 per KV head, context 2048): 2.40 -> 2.16 ms per step at batch 1 together with the wide-FFN path,
    // 6.0 -> 5.2 ms at batch 8, 12.9 -> 11.8 ms at batch 32 against all four heads in one CTA.
    int G = Gall;
    if (Gall > 2) G = Gall % 2 == 0 ? 2 : 1;
    const int hshare = Gall / G;
    const int kvReal = kvHeads;
    kvHeads *= hshare;  // virtual KV heads from here on
    const bool split_ok = (headDim == 64 || headDim == 128) && (G == 1 || G == 2 || G == 4) &&
                          ((reinterpret_cast<uintptr_t>(d_q) | reinterpret_cast<uintptr_t>(d_k) |
                            reinterpret_cast<uintptr_t>(d_v)) & 15) == 0;
    if (!split_ok) {
        if (q8) return smc_fail(ctx, SMC_E_UNSUPPORTED, "sdpa_decode: a Q8_0 cache needs headDim 64 or 128 and 16-byte aligned buffers");
        // reference-order kernel, one launch per (batch, head) group is avoided by treating each
        // (batch, head) as its own single-query problem through grid.y
        for (int b = 0; b < batch; ++b)
            for (int h = 0; h < heads; ++h) {
                const float *kp = static_cast<const float *>(d_k) + ((size_t)b * kvReal + h / Gall) * (size_t)maxSeq * headDim;
                const float *vp = static_cast<const float *>(d_v) + ((size_t)b * kvReal + h / Gall) * (size_t)maxSeq * headDim;
                int rc = smc_launch_sdpa_tile(ctx, d_q + ((size_t)b * heads + h) * headDim, kp, vp,
                                              d_out + ((size_t)b * heads + h) * headDim, 1, kvLen, headDim, scale, 1,
                                              headDim, headDim, 0.f, s);
                if (rc) return rc;
            }
        return SMC_OK;
    }
    int pairs = batch * kvHeads;
    int splits = (2 * ctx->sm_count + pairs - 1) / pairs;
    int max_splits = (kvLen + 63) / 64;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > MERGE_MAX_SPLITS) splits = MERGE_MAX_SPLITS;
    std::lock_guard<std::mutex> scratch_lock(ctx->mu_scratch);  // held until the launch is queued (one stream per context)
    {
        int rc = reserve_split_scratch(ctx, batch, heads, kvHeads, headDim, maxSeq);
        if (rc) return rc;
    }
    unsigned *tickets = reinterpret_cast<unsigned *>(ctx->d_attn_part);
    float *records = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ctx->d_attn_part) + TICKET_BYTES);
    const int ngroups = (SPLIT_THREADS / 32) * (32 / LPK);
    size_t smem = ((size_t)ngroups * G * 2 + (size_t)ngroups * G * headDim) * sizeof(float);
    dim3 grid(splits, kvHeads, batch);
    int rc;
    if (headDim == 128)
        rc = q8 ? launch_split_g<16, true>(ctx, G, grid, smem, s, d_q, d_k, d_v, d_kd, d_vd, records, heads, kvHeads, kvLen, maxSeq,
                                           scale, splits, d_out, tickets, hshare)
                : launch_split_g<16, false>(ctx, G, grid, smem, s, d_q, d_k, d_v, d_kd, d_vd, records, heads, kvHeads, kvLen, maxSeq,
                                            scale, splits, d_out, tickets, hshare);
    else
        rc = q8 ? launch_split_g<8, true>(ctx, G, grid, smem, s, d_q, d_k, d_v, d_kd, d_vd, records, heads, kvHeads, kvLen, maxSeq,
                                          scale, splits, d_out, tickets, hshare)
                : launch_split_g<8, false>(ctx, G, grid, smem, s, d_q, d_k, d_v, d_kd, d_vd, records, heads, kvHeads, kvLen, maxSeq,
                                           scale, splits, d_out, tickets, hshare);
    if (rc) return rc;
    return SMC_OK;
}

extern "C" {

int smc_kv_append_dev(smc_ctx *ctx, const float *d_k, const float *d_v, float *d_kcache, float *d_vcache, int batch,
                      int kvHeads, int headDim, int pos, int maxSeq, void *stream)
{
    if (!ctx || !d_k || !d_v || !d_kcache || !d_vcache || batch < 0 || kvHeads <= 0 || headDim <= 0)
        return smc_fail(ctx, SMC_E_INVALID, "kv_append: bad arguments");
    if (pos < 0 || pos >= maxSeq)  // KVCache.Update throws on overflow (KVCache.cs:89-91)
        return smc_fail(ctx, SMC_E_RANGE, "KVCache overflow: position %d + seqLen 1 exceeds capacity %d", pos, maxSeq);
    long long total = (long long)batch * kvHeads * headDim;
    if (total == 0) return SMC_OK;
    kv_append_kernel<<<(unsigned)((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        d_k, d_v, d_kcache, d_vcache, batch, kvHeads, headDim, pos, maxSeq);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

}  // extern "C"
