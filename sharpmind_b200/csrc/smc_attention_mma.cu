// Causal prompt attention on the tensor cores with fp32-grade accuracy: S = Q K^T and O = P V as bf16 MMAs
// (mma.sync.m16n8k16, fp32 accumulate) on operands split three ways, x = hi + mid + lo with each part a bf16
// (8 + 8 + 8 mantissa bits = the 24 of fp32).  A product keeps the six terms hi*hi, hi*mid, mid*hi, hi*lo, lo*hi,
// mid*mid; what is dropped is below 2^-24 of the product, so scores and outputs carry fp32 rounding only
// (ScaledDotProductFlash*'s arithmetic up to summation order, AttentionKernels.cs:220-475).  Six MMAs of 2048
// multiply-adds replace 12 288 fp32 FMAs, i.e. 384 warp instructions: the CUDA-core kernel this replaces spent its
// time waiting on shared-memory operands of those FMAs.
//
// One CTA = 64 consecutive query rows of HPC (1 or 2) query heads that share a KV head, four warps per head, 16 rows
// per warp.  K and V go through shared memory in tiles of 32 keys, split into their three bf16 planes ONCE per CTA
// while they are staged (rows padded to an odd multiple of 16 bytes: every ldmatrix is conflict free); Q is split
// the same way once per CTA.  The score tile's accumulator layout is the A-operand layout of the next MMA for
// 16-bit types, so P goes from registers to registers.  Online softmax per row as in the scalar kernel.
// sm_100a runs mma.sync on its legacy tensor path; a tcgen05 version would keep S and O in tensor memory.
#include <cuda_bf16.h>

#include "smc_common.cuh"

namespace {

constexpr int QROWS = 64, KT = 32;

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// x = hi + mid + lo, each a bf16 (round to nearest; the remainders are exact in fp32)
__device__ __forceinline__ void split3(float x, __nv_bfloat16 &hi, __nv_bfloat16 &mid, __nv_bfloat16 &lo)
{
    hi = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(hi);
    mid = __float2bfloat16_rn(r1);
    lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
}
__device__ __forceinline__ uint32_t pack2(__nv_bfloat16 a, __nv_bfloat16 b)
{
    return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}
// the six kept terms of (a_hi + a_mid + a_lo) * (b_hi + b_mid + b_lo), smallest first
__device__ __forceinline__ void mma6(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&am)[4], const uint32_t (&al)[4],
                                     const uint32_t (&b0)[3], const uint32_t (&b1)[3])
{
    mma_bf16(c, am, b0[1], b1[1]);
    mma_bf16(c, ah, b0[2], b1[2]);
    mma_bf16(c, al, b0[0], b1[0]);
    mma_bf16(c, ah, b0[1], b1[1]);
    mma_bf16(c, am, b0[0], b1[0]);
    mma_bf16(c, ah, b0[0], b1[0]);
}

// Shared memory (bf16 planes, plane p of a tile at p * rows * LDB bytes): Q [3][HPC * 64][LD], K [3][32][LD], V [3][32][LD]
// Q8: the cache holds Q8_0 rows as int8 planes kc / vc [.., maxSeq, HD] with fp16 block scales kd / vd [.., maxSeq, HD / 32]
// (QuantizedKVCache); a staged value is d * q, a 19-bit number that its three bf16 parts hold exactly, so the contraction
// sees exactly what ScaledDotProductFlashQ8_0* reads from the cache (AttentionKernels.cs:489-813).
template <int HD, int HPC, bool Q8>
__global__ void __launch_bounds__(128 * HPC) sdpa_prefill_mma_kernel(const float *__restrict__ q, const void *__restrict__ kc,
                                                                     const void *__restrict__ vc, const __half *__restrict__ kd,
                                                                     const __half *__restrict__ vd, float *__restrict__ out, int T,
                                                                     int nh, int nkv, int pos0, int maxSeq, float scale)
{
    constexpr int LDB = HD * 2 + 16;                 // bytes per row of a plane
    constexpr int QPLANE = HPC * QROWS * LDB, KPLANE = KT * LDB;
    constexpr int NTH = 128 * HPC;
    extern __shared__ __align__(16) uint8_t sm_raw[];
    uint8_t *sq = sm_raw, *sk = sq + 3 * QPLANE, *sv = sk + 3 * KPLANE;
    const uint32_t sq_a = (uint32_t)__cvta_generic_to_shared(sq), sk_a = (uint32_t)__cvta_generic_to_shared(sk),
                   sv_a = (uint32_t)__cvta_generic_to_shared(sv);
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tg = lane & 3;
    const int hl = warp >> 2, wq = warp & 3;          // head of the CTA's group, 16-row slice of the 64 rows
    const int hg = blockIdx.x;                          // head group; the grid's fast index, so CTAs start heaviest tile first
    const int h = hg * HPC + hl, kvh = (hg * HPC) / (nh / nkv);
    const int t0 = (int)(gridDim.y - 1 - blockIdx.y) * QROWS;  // later rows see more keys: they start first
    const int cta_len = pos0 + min(T, t0 + QROWS);    // keys any row of this CTA sees
    const float *kbase = static_cast<const float *>(kc) + (size_t)kvh * maxSeq * HD, *vbase = static_cast<const float *>(vc) + (size_t)kvh * maxSeq * HD;
    const int8_t *kqb = static_cast<const int8_t *>(kc) + (size_t)kvh * maxSeq * HD, *vqb = static_cast<const int8_t *>(vc) + (size_t)kvh * maxSeq * HD;
    const __half *kdb = Q8 ? kd + (size_t)kvh * maxSeq * (HD / 32) : nullptr, *vdb = Q8 ? vd + (size_t)kvh * maxSeq * (HD / 32) : nullptr;

    // ---- Q: split once
    for (int e = threadIdx.x; e < HPC * QROWS * (HD / 4); e += NTH) {
        const int c = e % (HD / 4), r = (e / (HD / 4)) % QROWS, hh = e / (QROWS * (HD / 4));
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t0 + r < T) v = *reinterpret_cast<const float4 *>(q + ((size_t)(t0 + r) * nh + hg * HPC + hh) * HD + 4 * c);
        __nv_bfloat16 p[3][4];
        split3(v.x, p[0][0], p[1][0], p[2][0]), split3(v.y, p[0][1], p[1][1], p[2][1]);
        split3(v.z, p[0][2], p[1][2], p[2][2]), split3(v.w, p[0][3], p[1][3], p[2][3]);
#pragma unroll
        for (int pl = 0; pl < 3; ++pl)
            *reinterpret_cast<uint2 *>(sq + pl * QPLANE + (hh * QROWS + r) * LDB + 8 * c) = make_uint2(pack2(p[pl][0], p[pl][1]), pack2(p[pl][2], p[pl][3]));
    }

    // rows of this lane: g and g + 8 of the warp's 16
    const int row0 = t0 + wq * 16 + g, row1 = row0 + 8;
    const int len0 = row0 < T ? pos0 + row0 + 1 : 0, len1 = row1 < T ? pos0 + row1 + 1 : 0;  // keys each row sees
    const int warp_len = t0 + wq * 16 < T ? pos0 + min(T, t0 + wq * 16 + 16) : 0;
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // ldmatrix lane addressing
    const uint32_t a_off = (uint32_t)((hl * QROWS + wq * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDB + 16 * (lane >> 4));
    const uint32_t bk_off = (uint32_t)(((lane & 7) + 8 * (lane >> 4)) * LDB + 16 * ((lane >> 3) & 1));   // K: [key][dim], two key tiles
    const uint32_t bv_off = (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * LDB + 16 * (lane >> 4));   // V: transposed, two dim tiles

    // A tile's K and V rows are requested one iteration ahead into registers (the loads fly while the previous tile is
    // multiplied), then split into their planes and stored once everybody has finished reading that previous tile.
    constexpr int PF = KT * (HD / 4) / NTH;  // float4 pieces of K (and of V) per thread and tile
    float4 pk[PF], pv[PF];
    auto fetch = [&](int start) {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            const int e = threadIdx.x + i * NTH, r = e / (HD / 4), c = e % (HD / 4);
            pk[i] = pv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (start + r < cta_len) {
                if (Q8) {  // four codes and their block's scale: the piece is d * q
                    const size_t row = (size_t)(start + r);
                    const char4 ck = *reinterpret_cast<const char4 *>(kqb + row * HD + 4 * c), cv = *reinterpret_cast<const char4 *>(vqb + row * HD + 4 * c);
                    const float dk = __half2float(kdb[row * (HD / 32) + c / 8]), dv = __half2float(vdb[row * (HD / 32) + c / 8]);
                    pk[i] = make_float4(dk * (float)ck.x, dk * (float)ck.y, dk * (float)ck.z, dk * (float)ck.w);
                    pv[i] = make_float4(dv * (float)cv.x, dv * (float)cv.y, dv * (float)cv.z, dv * (float)cv.w);
                } else {
                    pk[i] = *reinterpret_cast<const float4 *>(kbase + (size_t)(start + r) * HD + 4 * c);
                    pv[i] = *reinterpret_cast<const float4 *>(vbase + (size_t)(start + r) * HD + 4 * c);
                }
            }
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            const int e = threadIdx.x + i * NTH, r = e / (HD / 4), c = e % (HD / 4);
            __nv_bfloat16 p[3][4];
            split3(pk[i].x, p[0][0], p[1][0], p[2][0]), split3(pk[i].y, p[0][1], p[1][1], p[2][1]);
            split3(pk[i].z, p[0][2], p[1][2], p[2][2]), split3(pk[i].w, p[0][3], p[1][3], p[2][3]);
#pragma unroll
            for (int pl = 0; pl < 3; ++pl)
                *reinterpret_cast<uint2 *>(sk + pl * KPLANE + r * LDB + 8 * c) = make_uint2(pack2(p[pl][0], p[pl][1]), pack2(p[pl][2], p[pl][3]));
            split3(pv[i].x, p[0][0], p[1][0], p[2][0]), split3(pv[i].y, p[0][1], p[1][1], p[2][1]);
            split3(pv[i].z, p[0][2], p[1][2], p[2][2]), split3(pv[i].w, p[0][3], p[1][3], p[2][3]);
#pragma unroll
            for (int pl = 0; pl < 3; ++pl)
                *reinterpret_cast<uint2 *>(sv + pl * KPLANE + r * LDB + 8 * c) = make_uint2(pack2(p[pl][0], p[pl][1]), pack2(p[pl][2], p[pl][3]));
        }
    };
    fetch(0);
    for (int start = 0; start < cta_len; start += KT) {
        __syncthreads();  // the previous tile has been consumed (and Q is in place before its first use)
        stash();
        __syncthreads();
        if (start + KT < cta_len) fetch(start + KT);  // in flight under this tile's MMAs
        if (start >= warp_len) continue;  // warp uniform: every row's causal bound lies before the tile

        // ---- S = Q K^T for 16 rows x 32 keys
        float s[KT / 8][4], s2[KT / 8][4];  // even and odd k-steps: two independent chains of dependent MMAs per key tile
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = s2[n][0] = s2[n][1] = s2[n][2] = s2[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
            uint32_t ah[4], am[4], al[4];
            ldsm4(sq_a + a_off + 32 * ks, ah);
            ldsm4(sq_a + QPLANE + a_off + 32 * ks, am);
            ldsm4(sq_a + 2 * QPLANE + a_off + 32 * ks, al);
#pragma unroll
            for (int np = 0; np < KT / 16; ++np) {  // two key tiles per ldmatrix
                uint32_t b[3][4];
#pragma unroll
                for (int pl = 0; pl < 3; ++pl) ldsm4(sk_a + pl * KPLANE + bk_off + np * 16 * LDB + 32 * ks, b[pl]);
                const uint32_t b0a[3] = {b[0][0], b[1][0], b[2][0]}, b1a[3] = {b[0][1], b[1][1], b[2][1]};
                const uint32_t b0b[3] = {b[0][2], b[1][2], b[2][2]}, b1b[3] = {b[0][3], b[1][3], b[2][3]};
                if (ks & 1) {
                    mma6(s2[2 * np], ah, am, al, b0a, b1a);
                    mma6(s2[2 * np + 1], ah, am, al, b0b, b1b);
                } else {
                    mma6(s[2 * np], ah, am, al, b0a, b1a);
                    mma6(s[2 * np + 1], ah, am, al, b0b, b1b);
                }
            }
        }
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) s[n][0] += s2[n][0], s[n][1] += s2[n][1], s[n][2] += s2[n][2], s[n][3] += s2[n][3];
        // ---- online softmax: lane holds keys start + 8n + 2tg, + 1 of rows g (s[n][0..1]) and g + 8 (s[n][2..3])
        float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) {
            const int key = start + 8 * n + 2 * tg;
            s[n][0] = key < len0 ? s[n][0] * scale : -INFINITY, s[n][1] = key + 1 < len0 ? s[n][1] * scale : -INFINITY;
            s[n][2] = key < len1 ? s[n][2] * scale : -INFINITY, s[n][3] = key + 1 < len1 ? s[n][3] * scale : -INFINITY;
            tm0 = fmaxf(tm0, fmaxf(s[n][0], s[n][1])), tm1 = fmaxf(tm1, fmaxf(s[n][2], s[n][3]));
        }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1)), tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1)), tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        const float nm0 = fmaxf(m0, tm0), nm1 = fmaxf(m1, tm1);
        // a row that sees no key of this tile (and none before) keeps m = -inf: its weights and corrections are 0
        const float c0 = nm0 > -INFINITY ? expf(m0 - nm0) : 0.f, c1 = nm1 > -INFINITY ? expf(m1 - nm1) : 0.f;
        float ps0 = 0.f, ps1 = 0.f;
        uint32_t ph[KT / 16][4], pm[KT / 16][4], pl_[KT / 16][4];  // P as A operands: k16 = two key tiles
#pragma unroll
        for (int n = 0; n < KT / 8; ++n) {
            float p[4];
            p[0] = nm0 > -INFINITY ? expf(s[n][0] - nm0) : 0.f, p[1] = nm0 > -INFINITY ? expf(s[n][1] - nm0) : 0.f;
            p[2] = nm1 > -INFINITY ? expf(s[n][2] - nm1) : 0.f, p[3] = nm1 > -INFINITY ? expf(s[n][3] - nm1) : 0.f;
            ps0 += p[0] + p[1], ps1 += p[2] + p[3];
            __nv_bfloat16 hi[4], mi[4], lo[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) split3(p[i], hi[i], mi[i], lo[i]);
            // accumulator (row g: cols 2tg, 2tg+1 | row g+8) of key tile n -> A regs: tile 2j -> a0 (row g), a1 (row g+8); tile 2j+1 -> a2, a3
            const int j = n >> 1, o2 = (n & 1) * 2;
            ph[j][o2] = pack2(hi[0], hi[1]), ph[j][o2 + 1] = pack2(hi[2], hi[3]);
            pm[j][o2] = pack2(mi[0], mi[1]), pm[j][o2 + 1] = pack2(mi[2], mi[3]);
            pl_[j][o2] = pack2(lo[0], lo[1]), pl_[j][o2 + 1] = pack2(lo[2], lo[3]);
        }
        ps0 += __shfl_xor_sync(0xffffffffu, ps0, 1), ps0 += __shfl_xor_sync(0xffffffffu, ps0, 2);
        ps1 += __shfl_xor_sync(0xffffffffu, ps1, 1), ps1 += __shfl_xor_sync(0xffffffffu, ps1, 2);
        l0 = fmaf(l0, c0, ps0), l1 = fmaf(l1, c1, ps1);
        m0 = nm0, m1 = nm1;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n) o[n][0] *= c0, o[n][1] *= c0, o[n][2] *= c1, o[n][3] *= c1;
        // ---- O += P V
#pragma unroll
        for (int j = 0; j < KT / 16; ++j) {
#pragma unroll
            for (int np = 0; np < HD / 16; ++np) {  // two dim tiles per ldmatrix
                uint32_t b[3][4];
#pragma unroll
                for (int pl = 0; pl < 3; ++pl) ldsm4t(sv_a + pl * KPLANE + bv_off + j * 16 * LDB + 32 * np, b[pl]);
                const uint32_t b0a[3] = {b[0][0], b[1][0], b[2][0]}, b1a[3] = {b[0][1], b[1][1], b[2][1]};
                const uint32_t b0b[3] = {b[0][2], b[1][2], b[2][2]}, b1b[3] = {b[0][3], b[1][3], b[2][3]};
                mma6(o[2 * np], ph[j], pm[j], pl_[j], b0a, b1a);
                mma6(o[2 * np + 1], ph[j], pm[j], pl_[j], b0b, b1b);
            }
        }
    }
    // ---- out = O / l
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        if (row0 < T) *reinterpret_cast<float2 *>(out + ((size_t)row0 * nh + h) * HD + 8 * n + 2 * tg) = make_float2(o[n][0] * i0, o[n][1] * i0);
        if (row1 < T) *reinterpret_cast<float2 *>(out + ((size_t)row1 * nh + h) * HD + 8 * n + 2 * tg) = make_float2(o[n][2] * i1, o[n][3] * i1);
    }
}

}  // namespace

bool smc_sdpa_prefill_mma_supported(int nh, int nkv, int hd) { return (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0; }

// kd == null: kc / vc are fp32 rows; else the int8 planes and fp16 block scales of a Q8_0 cache
static int launch_prefill_mma(smc_ctx *ctx, const float *q, const void *kc, const void *vc, const __half *kd, const __half *vd, float *out,
                              int T, int nh, int nkv, int hd, int pos0, int maxSeq, float scale, cudaStream_t s)
{
    const int G = nh / nkv;
    auto go = [&](auto kernel, int hpc) {
        const dim3 grid(nh / hpc, (T + QROWS - 1) / QROWS);
        const size_t ldb = (size_t)hd * 2 + 16;
        const size_t smem = 3 * ((size_t)hpc * QROWS + 2 * KT) * ldb;
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        smc_launch_dep(ctx->use_pdl, kernel, grid, dim3(128 * hpc), smem, s, q, kc, vc, kd, vd, out, T, nh, nkv, pos0, maxSeq, scale);
    };
    const bool two = G % 2 == 0 && ctx->attn_hpc != 1;
    if (kd) {
        if (hd == 128) two ? go(sdpa_prefill_mma_kernel<128, 2, true>, 2) : go(sdpa_prefill_mma_kernel<128, 1, true>, 1);
        else two ? go(sdpa_prefill_mma_kernel<64, 2, true>, 2) : go(sdpa_prefill_mma_kernel<64, 1, true>, 1);
    } else {
        if (hd == 128) two ? go(sdpa_prefill_mma_kernel<128, 2, false>, 2) : go(sdpa_prefill_mma_kernel<128, 1, false>, 1);
        else two ? go(sdpa_prefill_mma_kernel<64, 2, false>, 2) : go(sdpa_prefill_mma_kernel<64, 1, false>, 1);
    }
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_launch_sdpa_prefill_mma(smc_ctx *ctx, const float *q, const float *kc, const float *vc, float *out, int T, int nh, int nkv,
                                int hd, int pos0, int maxSeq, float scale, cudaStream_t s)
{
    return launch_prefill_mma(ctx, q, kc, vc, nullptr, nullptr, out, T, nh, nkv, hd, pos0, maxSeq, scale, s);
}

// one sequence's Q8_0 cache planes (rows pos0 .. pos0 + T - 1 are the queries' own positions)
int smc_launch_sdpa_prefill_mma_q8(smc_ctx *ctx, const float *q, const int8_t *kq, const __half *kd, const int8_t *vq, const __half *vd,
                                   float *out, int T, int nh, int nkv, int hd, int pos0, int maxSeq, float scale, cudaStream_t s)
{
    return launch_prefill_mma(ctx, q, kq, vq, kd, vd, out, T, nh, nkv, hd, pos0, maxSeq, scale, s);
}
