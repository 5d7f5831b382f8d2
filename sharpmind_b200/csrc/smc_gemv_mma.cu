// Small-batch (2..32 rows, larger batches in passes of 32) quantised-activation matmul on the int8 tensor-core
// path: out[t, r] = sum_blocks (dw * dx) * isum(block) (- the Q4_K min term), the arithmetic of SMC_ACT_Q8.
//
// Why MMA here: with a handful of activation rows the dp4a kernels issue one integer dot per (row, token,
// 4 bytes) and become instruction-bound long before HBM is busy.  One mma.m16n8k32 (s8 x s8 -> s32) covers
// 16 weight rows x 8 tokens x one 32-element block, so the per-block integer sums of 32 rows x 32 tokens cost
// 8 instructions per warp; the per-block scaling (int -> float, dw * dx, fused multiply-add) stays on the
// CUDA cores and is what remains.  Integer block sums are exact, so they equal the dp4a kernels' sums; each
// output adds its scaled block sums in k order within a warp's k range and the eight warps of a CTA (which
// split K) are added in warp order: the result of a row does not depend on the batch size or on the other
// rows (for any batch >= 2; the one-row kernels use a different summation tree).
//
// Layout choices.  A CTA owns 32 weight rows (two m16 tiles) and all tokens; its 8 warps take interleaved
// k groups and meet in shared memory at the end.  Fragments are loaded straight from global memory as 8-byte
// words: the dot product does not care about the order of k inside a block, so MMA k index 4*tg + i is bound to
// byte 8*tg + i and 16 + 4*tg + i to byte 8*tg + 4 + i of the block, for weights and activations alike; a
// quad of lanes then reads one whole 32-byte sector per row.  Scales are loaded once per lane (lane = row for
// the weights, lane = token for the activations) and handed round with shuffles.
#include "smc_common.cuh"

#include <type_traits>

namespace {

constexpr int MMA_ROWS = 32;   // weight rows per CTA
constexpr int MMA_WARPS = 8;
// floats per token of the warps' partial tiles in shared memory: a lane (g, tg) of an accumulator fragment writes token
// 2 * tg (+ 1), row g (+ 8), so 2 * RED_LD = 8 (mod 32) puts the 32 lanes of a store on 32 banks (33 left them 4 deep)
constexpr int RED_LD = 36;

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ uint2 ldg8(const void *p)
{
    uint2 v;
    asm("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));  // not volatile: free to be hoisted
    return v;
}

// Adds the warps' partial tiles in warp order and stores out[t, r]; red is [NW warps][TOK tokens][RED_LD], TOK >= 8 * NT.
template <int NT, int NW = MMA_WARPS, int TOK = 32>
__device__ __forceinline__ void reduce_and_store(float (*red)[TOK][RED_LD], const float (&acc)[2][NT][4], float *out, int N, int M,
                                                 int r0, int t0)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[warp][8 * t + 2 * tg + (i & 1)][mt * 16 + g + ((i >> 1) << 3)] = acc[mt][t][i];
    __syncthreads();
    for (int o = threadIdx.x; o < 32 * 8 * NT; o += blockDim.x) {
        const int row = o & 31, tok = o >> 5;
        float s = red[0][tok][row];
#pragma unroll
        for (int w = 1; w < NW; ++w) s += red[w][tok][row];
        if (r0 + row < N && t0 + tok < M) out[(size_t)(t0 + tok) * N + r0 + row] = s;
    }
    __syncthreads();
}

// ------------------------------------------------------------------------------------------ Q8_0
// Planes: quants [N][K] int8, scales [N][K/32] fp16.  K % 128 == 0; a warp works on groups of four blocks.
template <int NT>
__global__ void __launch_bounds__(256, NT > 4 ? 1 : 2)
gemv_mma_q8_0_kernel(const int8_t *__restrict__ wq, const __half *__restrict__ wd, const int8_t *__restrict__ xq,
                     const float *__restrict__ xd, float *__restrict__ out, int N, int K, int M)
{
    // NT token tiles of 8 per pass: 1, 2, 4 for up to 32 rows; 8 for prompt-sized batches (64 tokens share every weight
    // fragment and scale, which halves the passes over the matrix)
    constexpr int TOK = NT > 4 ? 64 : 32, XR = TOK / 32;
    extern __shared__ __align__(16) float red_q8[];
    float (*red)[TOK][RED_LD] = reinterpret_cast<float (*)[TOK][RED_LD]>(red_q8);
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
    const int r0 = blockIdx.x * MMA_ROWS;
    const int nb = K / 32, ngroups = nb / 4;
    // rows past the end are clamped for loads and masked at the store
    const int8_t *arow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) arow[j] = wq + (size_t)min(r0 + (j >> 1) * 16 + g + (j & 1) * 8, N - 1) * K + 8 * tg;
    const __half *drow = wd + (size_t)min(r0 + lane, N - 1) * nb;
    {  // one pass of 8 * NT tokens per CTA: blockIdx.y picks the pass (a batch of more than 32 rows fills the grid with passes)
        const int t0 = blockIdx.y * 8 * NT;
        const int8_t *brow[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) brow[t] = xq + (size_t)min(t0 + 8 * t + g, M - 1) * K + 8 * tg;
        const float *xrow[XR];  // this lane's tokens: lane, and lane + 32 in a 64-token pass
#pragma unroll
        for (int x = 0; x < XR; ++x) xrow[x] = xd + (size_t)min(t0 + 32 * x + lane, M - 1) * nb;
        float acc[2][NT][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][t][i] = 0.f;
        for (int gi = warp; gi < ngroups; gi += MMA_WARPS) {
            // all weight bytes of the group are requested before any of them is used: 4 KB in flight per warp
            uint2 aq[4][4];
#pragma unroll
            for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                for (int j = 0; j < 4; ++j) aq[kb][j] = ldg8(arow[j] + (gi * 4 + kb) * 32);
            const uint2 dwp = *reinterpret_cast<const uint2 *>(drow + gi * 4);   // this lane's row, 4 blocks
            float4 dxp[XR];                                                      // this lane's tokens, 4 blocks
#pragma unroll
            for (int x = 0; x < XR; ++x) dxp[x] = *reinterpret_cast<const float4 *>(xrow[x] + gi * 4);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                const int koff = (gi * 4 + kb) * 32;
                uint2 b[NT];
                const uint2 (&a)[4] = aq[kb];
#pragma unroll
                for (int t = 0; t < NT; ++t) b[t] = ldg8(brow[t] + koff);
                const uint32_t dword = (kb & 2) ? dwp.y : dwp.x;
                float dxl[XR];
#pragma unroll
                for (int x = 0; x < XR; ++x) dxl[x] = kb == 0 ? dxp[x].x : kb == 1 ? dxp[x].y : kb == 2 ? dxp[x].z : dxp[x].w;
                float dw[2][2];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t wv = __shfl_sync(0xffffffffu, dword, (j >> 1) * 16 + g + (j & 1) * 8);
                    dw[j >> 1][j & 1] = smc_h2f((uint16_t)((kb & 1) ? (wv >> 16) : (wv & 0xFFFFu)));
                }
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float dx0 = __shfl_sync(0xffffffffu, dxl[t >> 2], 8 * (t & 3) + 2 * tg);
                    const float dx1 = __shfl_sync(0xffffffffu, dxl[t >> 2], 8 * (t & 3) + 2 * tg + 1);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        int c[4];
                        mma_s8(c, a[2 * mt].x, a[2 * mt + 1].x, a[2 * mt].y, a[2 * mt + 1].y, b[t].x, b[t].y);
                        acc[mt][t][0] = fmaf((float)c[0], dw[mt][0] * dx0, acc[mt][t][0]);
                        acc[mt][t][1] = fmaf((float)c[1], dw[mt][0] * dx1, acc[mt][t][1]);
                        acc[mt][t][2] = fmaf((float)c[2], dw[mt][1] * dx0, acc[mt][t][2]);
                        acc[mt][t][3] = fmaf((float)c[3], dw[mt][1] * dx1, acc[mt][t][3]);
                    }
                }
            }
        }
        reduce_and_store<NT, MMA_WARPS, TOK>(red, acc, out, N, M, r0, t0);
    }
}

// Prompt-sized batches (hundreds of rows): the same sums with no shared-memory reduction.  The kernel above splits K
// over the eight warps of a CTA (warp w takes the groups w, w + 8, ...) and adds the eight partial tiles in warp order;
// with this many tokens there is parallelism enough without that split, so here one warp owns a 32 x 64 output tile and
// walks the eight group classes one after the other, adding each finished class to its running total: the same
// partial sums added in the same order, hence the same bits, without the barriers, the 64 KB of partial tiles and the
// 8-way re-read that cost the split kernel a quarter of its instructions on K = 1024.  A CTA = eight token tiles of
// one 32-row strip, which share the weight fragments through L1.
__global__ void __launch_bounds__(256, 1)
gemv_mma_q8_0_tile_kernel(const int8_t *__restrict__ wq, const __half *__restrict__ wd, const int8_t *__restrict__ xq,
                          const float *__restrict__ xd, float *__restrict__ out, int N, int K, int M)
{
    constexpr int NT = 8;
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
    const int r0 = blockIdx.x * MMA_ROWS;
    const int t0 = (blockIdx.y * (blockDim.x >> 5) + warp) * 8 * NT;  // the launcher picks 1..8 warps (token tiles) per CTA
    if (t0 >= M) return;  // no barrier below
    const int nb = K / 32, ngroups = nb / 4;
    const int8_t *abase = wq + 8 * tg;
    uint32_t aoff[4];  // 32-bit offsets (the launcher keeps N * K and M * K below 2^32): pointers would not fit the register file
#pragma unroll
    for (int j = 0; j < 4; ++j) aoff[j] = (uint32_t)min(r0 + (j >> 1) * 16 + g + (j & 1) * 8, N - 1) * (uint32_t)K;
    const __half *drow = wd + (size_t)min(r0 + lane, N - 1) * nb;
    const int8_t *bbase = xq + 8 * tg;
    uint32_t boff[NT];  // rows past the end are clamped for loads and masked at the store
#pragma unroll
    for (int t = 0; t < NT; ++t) boff[t] = (uint32_t)min(t0 + 8 * t + g, M - 1) * (uint32_t)K;
    const float *xrow[2] = {xd + (size_t)min(t0 + lane, M - 1) * nb, xd + (size_t)min(t0 + 32 + lane, M - 1) * nb};
    float total[2][NT][4];
#pragma unroll 1
    for (int cls = 0; cls < MMA_WARPS; ++cls) {
        float acc[2][NT][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][t][i] = 0.f;
#pragma unroll 1
        for (int gi = cls; gi < ngroups; gi += MMA_WARPS) {
            uint2 aq[4][4];
#pragma unroll
            for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                for (int j = 0; j < 4; ++j) aq[kb][j] = ldg8(abase + aoff[j] + (uint32_t)(gi * 4 + kb) * 32u);
            const uint2 dwp = *reinterpret_cast<const uint2 *>(drow + gi * 4);
            const float4 dxp[2] = {*reinterpret_cast<const float4 *>(xrow[0] + gi * 4), *reinterpret_cast<const float4 *>(xrow[1] + gi * 4)};
            // the activation fragments of block kb + 1 are requested before block kb is multiplied (those of block 0 go
            // out with the weight fragments above): one exposed load latency per group instead of five
            uint2 bn[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) bn[t] = ldg8(bbase + boff[t] + (uint32_t)(gi * 4) * 32u);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                uint2 b[NT];
                const uint2 (&a)[4] = aq[kb];
#pragma unroll
                for (int t = 0; t < NT; ++t) b[t] = bn[t];
                if (kb < 3) {
#pragma unroll
                    for (int t = 0; t < NT; ++t) bn[t] = ldg8(bbase + boff[t] + (uint32_t)(gi * 4 + kb + 1) * 32u);
                }
                const uint32_t dword = (kb & 2) ? dwp.y : dwp.x;
                float dxl[2];
#pragma unroll
                for (int x = 0; x < 2; ++x) dxl[x] = kb == 0 ? dxp[x].x : kb == 1 ? dxp[x].y : kb == 2 ? dxp[x].z : dxp[x].w;
                float dw[2][2];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t wv = __shfl_sync(0xffffffffu, dword, (j >> 1) * 16 + g + (j & 1) * 8);
                    dw[j >> 1][j & 1] = smc_h2f((uint16_t)((kb & 1) ? (wv >> 16) : (wv & 0xFFFFu)));
                }
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float dx0 = __shfl_sync(0xffffffffu, dxl[t >> 2], 8 * (t & 3) + 2 * tg);
                    const float dx1 = __shfl_sync(0xffffffffu, dxl[t >> 2], 8 * (t & 3) + 2 * tg + 1);
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        int c[4];
                        mma_s8(c, a[2 * mt].x, a[2 * mt + 1].x, a[2 * mt].y, a[2 * mt + 1].y, b[t].x, b[t].y);
                        acc[mt][t][0] = fmaf((float)c[0], dw[mt][0] * dx0, acc[mt][t][0]);
                        acc[mt][t][1] = fmaf((float)c[1], dw[mt][0] * dx1, acc[mt][t][1]);
                        acc[mt][t][2] = fmaf((float)c[2], dw[mt][1] * dx0, acc[mt][t][2]);
                        acc[mt][t][3] = fmaf((float)c[3], dw[mt][1] * dx1, acc[mt][t][3]);
                    }
                }
            }
        }
        // the split kernel's fold: s = partial of warp 0; s += partial of warp 1; ...
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) total[mt][t][i] = cls == 0 ? acc[mt][t][i] : total[mt][t][i] + acc[mt][t][i];
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = t0 + 8 * t + 2 * tg + (i & 1), row = r0 + mt * 16 + g + ((i >> 1) << 3);
                if (row < N && tok < M) out[(size_t)tok * N + row] = total[mt][t][i];
            }
}

// ------------------------------------------------------------------------------------------ Q4_K
// GGUF blocks of 144 bytes: d, dmin (fp16), 12 packed scale / min bytes, 128 nibble bytes; the 32 bytes of
// group gq hold sub-block 2*gq in the low nibbles and 2*gq + 1 in the high ones.  K % 256 == 0; a warp works
// on whole 256-element blocks.  out += d*sc_j * dx * isum  -  dmin*m_j * (dx * sum(xq))  per sub-block.
template <int NT>
__global__ void __launch_bounds__(256, NT > 2 ? 1 : 2)
gemv_mma_q4_K_kernel(const uint8_t *__restrict__ raw, const int8_t *__restrict__ xq, const float *__restrict__ xd,
                     const float *__restrict__ xsd, float *__restrict__ out, int N, int K, int M)
{
    __shared__ float red[MMA_WARPS][32][RED_LD];
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
    const int r0 = blockIdx.x * MMA_ROWS;
    const int nb = K / 32, nsb = K / 256;
    const size_t row_bytes = (size_t)nsb * 144;
    const uint8_t *arow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) arow[j] = raw + (size_t)min(r0 + (j >> 1) * 16 + g + (j & 1) * 8, N - 1) * row_bytes + 16 + 8 * tg;
    const uint8_t *hrow = raw + (size_t)min(r0 + lane, N - 1) * row_bytes;
    {  // one pass of 8 * NT tokens per CTA: blockIdx.y picks the pass (a batch of more than 32 rows fills the grid with passes)
        const int t0 = blockIdx.y * 8 * NT;
        const int8_t *brow[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) brow[t] = xq + (size_t)min(t0 + 8 * t + g, M - 1) * K + 8 * tg;
        const float *xrow = xd + (size_t)min(t0 + lane, M - 1) * nb;
        const float *srow = xsd + (size_t)min(t0 + lane, M - 1) * nb;
        float acc[2][NT][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][t][i] = 0.f;
        for (int sb = warp; sb < nsb; sb += MMA_WARPS) {
            // this lane's row: d * sc_j and dmin * m_j of the eight sub-blocks
            const uint4 hdr = *reinterpret_cast<const uint4 *>(hrow + (size_t)sb * 144);
            const float d = smc_h2f((uint16_t)(hdr.x & 0xFFFFu)), dmin = smc_h2f((uint16_t)(hdr.x >> 16));
            float dsc[8], dmn[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int sc, mn;
                smc_k4_scale_min(hdr.y, hdr.z, hdr.w, j, sc, mn);
                dsc[j] = d * (float)sc;
                dmn[j] = dmin * (float)mn;
            }
            // this lane's token: activation scale and scale * sum(q) of the eight sub-blocks
            const float4 dxa = *reinterpret_cast<const float4 *>(xrow + sb * 8), dxb = *reinterpret_cast<const float4 *>(xrow + sb * 8 + 4);
            const float4 sxa = *reinterpret_cast<const float4 *>(srow + sb * 8), sxb = *reinterpret_cast<const float4 *>(srow + sb * 8 + 4);
            const float dxl[8] = {dxa.x, dxa.y, dxa.z, dxa.w, dxb.x, dxb.y, dxb.z, dxb.w};
            const float sxl[8] = {sxa.x, sxa.y, sxa.z, sxa.w, sxb.x, sxb.y, sxb.z, sxb.w};
            uint2 aq[4][4];
#pragma unroll
            for (int gq = 0; gq < 4; ++gq)
#pragma unroll
                for (int j = 0; j < 4; ++j) aq[gq][j] = ldg8(arow[j] + (size_t)sb * 144 + 32 * gq);
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                const uint2 (&a)[4] = aq[gq];
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const int j8 = 2 * gq + hi;  // sub-block
                    const int koff = (sb * 8 + j8) * 32;
                    uint2 b[NT];
#pragma unroll
                    for (int t = 0; t < NT; ++t) b[t] = ldg8(brow[t] + koff);
                    float ws[2][2], wm[2][2];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int src = (j >> 1) * 16 + g + (j & 1) * 8;
                        ws[j >> 1][j & 1] = __shfl_sync(0xffffffffu, dsc[j8], src);
                        wm[j >> 1][j & 1] = __shfl_sync(0xffffffffu, dmn[j8], src);
                    }
                    uint32_t an[4][2];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        an[j][0] = (hi ? (a[j].x >> 4) : a[j].x) & 0x0F0F0F0Fu;
                        an[j][1] = (hi ? (a[j].y >> 4) : a[j].y) & 0x0F0F0F0Fu;
                    }
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const float dx0 = __shfl_sync(0xffffffffu, dxl[j8], 8 * t + 2 * tg);
                        const float dx1 = __shfl_sync(0xffffffffu, dxl[j8], 8 * t + 2 * tg + 1);
                        const float sx0 = __shfl_sync(0xffffffffu, sxl[j8], 8 * t + 2 * tg);
                        const float sx1 = __shfl_sync(0xffffffffu, sxl[j8], 8 * t + 2 * tg + 1);
#pragma unroll
                        for (int mt = 0; mt < 2; ++mt) {
                            int c[4];
                            mma_s8(c, an[2 * mt][0], an[2 * mt + 1][0], an[2 * mt][1], an[2 * mt + 1][1], b[t].x, b[t].y);
                            acc[mt][t][0] = fmaf(-wm[mt][0], sx0, fmaf((float)c[0], ws[mt][0] * dx0, acc[mt][t][0]));
                            acc[mt][t][1] = fmaf(-wm[mt][0], sx1, fmaf((float)c[1], ws[mt][0] * dx1, acc[mt][t][1]));
                            acc[mt][t][2] = fmaf(-wm[mt][1], sx0, fmaf((float)c[2], ws[mt][1] * dx0, acc[mt][t][2]));
                            acc[mt][t][3] = fmaf(-wm[mt][1], sx1, fmaf((float)c[3], ws[mt][1] * dx1, acc[mt][t][3]));
                        }
                    }
                }
            }
        }
        reduce_and_store<NT>(red, acc, out, N, M, r0, t0);
    }
}

// ------------------------------------------------------------------------------------------------ Q6_K
// Weights in the unit layout of smc_common.cuh (X, Y, Z entries per lane slot, 16 int8 scales and fp16 d per block).
// A scale covers 16 elements, so the unit is mma.m16n8k16: for half h (128 elements) and sixteen `is` a lane reads
// four bytes of the X, Y and Z entries of slot (block, h, is) at byte 4*tg of each of its four rows and forms from
// them the codes of columns c = 0..3 (elements 32c + l .. l + 3 of the half, l = 16*is + 4*tg), 32 subtracted
// bytewise; out += (d * sc[8h + is + 2c]) * dx[4h + c] * isum.
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

__device__ __forceinline__ uint32_t ldg4(const void *p)
{
    uint32_t v;
    asm("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

template <int C>
__device__ __forceinline__ uint32_t q6_codes(uint32_t wx, uint32_t wy, uint32_t wz)
{
    const uint32_t M6 = 0x3F3F3F3Fu;
    uint32_t q;
    if (C == 0) q = wx & M6;
    else if (C == 1) q = wy & M6;
    else if (C == 2) q = wz & M6;
    else q = ((wx >> 6) & 0x03030303u) | ((wy >> 4) & 0x0C0C0C0Cu) | ((wz >> 2) & 0x30303030u);
    return __vsub4(q, 0x20202020u);  // codes 0..63 -> -32..31, no byte borrows into its neighbour
}

template <int NT, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 2 : 1)
gemv_mma_q6_K_kernel(const uint8_t *__restrict__ q6u, const int8_t *__restrict__ xq, const float *__restrict__ xd,
                     float *__restrict__ out, int N, int K, int M)
{
    // NW warps split K: 8 (two CTAs per SM), or 16 in one CTA per SM for rows of 8192 elements and more
    extern __shared__ __align__(16) float red_dyn[];
    float (*red)[32][RED_LD] = reinterpret_cast<float (*)[32][RED_LD]>(red_dyn);
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
    const int r0 = blockIdx.x * MMA_ROWS;
    const int nb = K / 32, nsb = K / 256;
    uint32_t rblk[4];  // block indices: a tensor has fewer than 2^32 blocks of 256
#pragma unroll
    for (int j = 0; j < 4; ++j) rblk[j] = (uint32_t)min(r0 + (j >> 1) * 16 + g + (j & 1) * 8, N - 1) * (uint32_t)nsb;
    const uint32_t hblk = (uint32_t)min(r0 + lane, N - 1) * (uint32_t)nsb;
    {  // one pass of 8 * NT tokens per CTA: blockIdx.y picks the pass (a batch of more than 32 rows fills the grid with passes)
        const int t0 = blockIdx.y * 8 * NT;
        const int8_t *brow[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) brow[t] = xq + (size_t)min(t0 + 8 * t + g, M - 1) * K + 4 * tg;
        const float *xrow = xd + (size_t)min(t0 + lane, M - 1) * nb;
        float acc[2][NT][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][t][i] = 0.f;
        for (int sb = warp; sb < nsb; sb += NW) {
            // this lane's row: d * sc of the sixteen sub-blocks
            const uint4 scw = *reinterpret_cast<const uint4 *>(q6u + smc_q6u_scales(hblk + sb));
            const float d = __half2float(*reinterpret_cast<const __half *>(q6u + smc_q6u_d(hblk + sb)));
            // this lane's token: activation scales of the eight 32-element blocks
            const float4 dxa = *reinterpret_cast<const float4 *>(xrow + sb * 8), dxb = *reinterpret_cast<const float4 *>(xrow + sb * 8 + 4);
            // up to 16 tokens both halves are unrolled and their loads overlap; beyond, the accumulators need the registers
#pragma unroll(NT <= 2 ? 2 : 1)
            for (int h = 0; h < 2; ++h) {
                const uint32_t scws[2] = {h ? scw.z : scw.x, h ? scw.w : scw.y};
                const float dxl[4] = {h ? dxb.x : dxa.x, h ? dxb.y : dxa.y, h ? dxb.z : dxa.z, h ? dxb.w : dxa.w};
#pragma unroll
                for (int is = 0; is < 2; ++is) {
                    uint32_t wa[4], wb[4], wh[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint8_t *pl = q6u + smc_q6u_slot(rblk[j] + sb, h, is) + 4 * tg;
                        wa[j] = ldg4(pl), wb[j] = ldg4(pl + SMC_Q6U_Y), wh[j] = ldg4(pl + SMC_Q6U_Z);
                    }
                    auto column = [&](auto cc) {
                        constexpr int c = decltype(cc)::value;
                        constexpr int bx = c;
                        const int si = is + 2 * c;  // scale byte within the half
                        const int koff = sb * 256 + 128 * h + 32 * c + 16 * is;
                        uint32_t b[NT], an[4];
#pragma unroll
                        for (int t = 0; t < NT; ++t) b[t] = ldg4(brow[t] + koff);
#pragma unroll
                        for (int j = 0; j < 4; ++j) an[j] = q6_codes<c>(wa[j], wb[j], wh[j]);
                        const float dsc = d * (float)(int)(int8_t)((scws[si >> 2] >> (8 * (si & 3))) & 0xFF);
                        float ws[2][2];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            ws[j >> 1][j & 1] = __shfl_sync(0xffffffffu, dsc, (j >> 1) * 16 + g + (j & 1) * 8);
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            const float dx0 = __shfl_sync(0xffffffffu, dxl[bx], 8 * t + 2 * tg);
                            const float dx1 = __shfl_sync(0xffffffffu, dxl[bx], 8 * t + 2 * tg + 1);
#pragma unroll
                            for (int mt = 0; mt < 2; ++mt) {
                                int c4[4];
                                mma_s8_k16(c4, an[2 * mt], an[2 * mt + 1], b[t]);
                                acc[mt][t][0] = fmaf((float)c4[0], ws[mt][0] * dx0, acc[mt][t][0]);
                                acc[mt][t][1] = fmaf((float)c4[1], ws[mt][0] * dx1, acc[mt][t][1]);
                                acc[mt][t][2] = fmaf((float)c4[2], ws[mt][1] * dx0, acc[mt][t][2]);
                                acc[mt][t][3] = fmaf((float)c4[3], ws[mt][1] * dx1, acc[mt][t][3]);
                            }
                        }
                    };
                    column(std::integral_constant<int, 0>{});
                    column(std::integral_constant<int, 1>{});
                    column(std::integral_constant<int, 2>{});
                    column(std::integral_constant<int, 3>{});
                }
            }
        }
        reduce_and_store<NT, NW>(red, acc, out, N, M, r0, t0);
    }
}

}  // namespace

bool smc_mma_supported(const smc_weight *w, int M)
{
    if (!w->fast || M < 2) return false;
    if (w->dtype == SMC_Q8_0) return w->K % 128 == 0 && w->q8_qs != nullptr;
    if (w->dtype == SMC_Q4_K) return w->K % 256 == 0 && w->d_raw != nullptr;
    if (w->dtype == SMC_Q6_K) return w->K % 256 == 0 && w->q6u != nullptr;
    return false;
}

int smc_launch_gemv_mma(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s)
{
    const int N = w->N, K = w->K, M = a->M;
    const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
    const dim3 grid((N + MMA_ROWS - 1) / MMA_ROWS, (M + 8 * nt - 1) / (8 * nt));
    if (w->dtype == SMC_Q8_0) {
        // prompt-sized batches: passes of 64 tokens
        const int nt8 = M >= 64 ? 8 : nt;
        const dim3 g8((N + MMA_ROWS - 1) / MMA_ROWS, (M + 8 * nt8 - 1) / (8 * nt8));
        auto go8 = [&](auto kernel, int tok) {
            const size_t smem = (size_t)MMA_WARPS * tok * RED_LD * sizeof(float);
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            smc_launch_dep(ctx->use_pdl, kernel, g8, dim3(256), smem, s, (const int8_t *)w->q8_qs, (const __half *)w->q8_d,
                           (const int8_t *)a->q, (const float *)a->d, out, N, K, M);
        };
        if (M >= 256 && (size_t)N * K < (1ull << 32) && (size_t)M * K < (1ull << 32)) {  // enough token tiles for a warp to own one: no K split, no shared memory
            // eight token tiles of a 32-row strip per CTA share its weight fragments through L1; matrices of few rows
            // take fewer per CTA so that the grid still covers the SMs twice (a warp's bits do not depend on this)
            const int strips = (N + MMA_ROWS - 1) / MMA_ROWS, tiles = (M + 63) / 64;
            int wpc = 8;
            while (wpc > 1 && strips * ((tiles + wpc - 1) / wpc) < 2 * ctx->sm_count) wpc >>= 1;
            smc_launch_dep(ctx->use_pdl, gemv_mma_q8_0_tile_kernel, dim3(strips, (tiles + wpc - 1) / wpc), dim3(32 * wpc), 0, s,
                           (const int8_t *)w->q8_qs, (const __half *)w->q8_d, (const int8_t *)a->q, (const float *)a->d, out, N, K, M);
        } else if (nt8 == 1) go8(gemv_mma_q8_0_kernel<1>, 32);
        else if (nt8 == 2) go8(gemv_mma_q8_0_kernel<2>, 32);
        else if (nt8 == 4) go8(gemv_mma_q8_0_kernel<4>, 32);
        else go8(gemv_mma_q8_0_kernel<8>, 64);
    } else if (w->dtype == SMC_Q6_K) {
        // the warp count follows from K alone, so a row's bits depend neither on the batch nor on how the rows are
        // split across GPUs; long rows are where matrices of few rows (FFN down) need the extra warps per SM
        const bool wide = K >= 8192;
        auto go = [&](auto kernel, int nw) {
            const size_t smem = (size_t)nw * 32 * RED_LD * sizeof(float);
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            smc_launch_dep(ctx->use_pdl, kernel, grid, dim3(nw * 32), smem, s, (const uint8_t *)w->q6u, (const int8_t *)a->q,
                           (const float *)a->d, out, N, K, M);
        };
        if (wide) {
            if (nt == 1) go(gemv_mma_q6_K_kernel<1, 16>, 16);
            else if (nt == 2) go(gemv_mma_q6_K_kernel<2, 16>, 16);
            else go(gemv_mma_q6_K_kernel<4, 16>, 16);
        } else {
            if (nt == 1) go(gemv_mma_q6_K_kernel<1, 8>, 8);
            else if (nt == 2) go(gemv_mma_q6_K_kernel<2, 8>, 8);
            else go(gemv_mma_q6_K_kernel<4, 8>, 8);
        }
    } else {
        if (nt == 1) smc_launch_dep(ctx->use_pdl, gemv_mma_q4_K_kernel<1>, grid, dim3(256), 0, s, (const uint8_t *)w->d_raw, (const int8_t *)a->q,
                           (const float *)a->d, (const float *)a->sd, out, N, K, M);
        else if (nt == 2) smc_launch_dep(ctx->use_pdl, gemv_mma_q4_K_kernel<2>, grid, dim3(256), 0, s, (const uint8_t *)w->d_raw, (const int8_t *)a->q,
                           (const float *)a->d, (const float *)a->sd, out, N, K, M);
        else smc_launch_dep(ctx->use_pdl, gemv_mma_q4_K_kernel<4>, grid, dim3(256), 0, s, (const uint8_t *)w->d_raw, (const int8_t *)a->q,
                           (const float *)a->d, (const float *)a->sd, out, N, K, M);
    }
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}
