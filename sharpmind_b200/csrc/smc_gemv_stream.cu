// Streaming GEMV for Q8_0-quantised activations (SMC_ACT_Q8), M <= 8: the kernels the decode path
// spends its time in.  Same arithmetic as the per-unit kernels in smc_gemv.cu, restructured so that
// the instruction stream per weight byte is short enough for HBM to be the limit:
//
//   * a warp owns a contiguous range of weight rows; because rows are contiguous in every layout
//     its weight bytes form one contiguous stream, cut into "steps" of 32 lane-units
//     (Q4_K / Q6_K: 8 blocks = 2048 elements; Q8_0: 32 blocks = 1024 elements);
//   * the units of the next PF steps are already in registers (software prefetch ring of 16-byte
//     streaming loads) while the current step is computed, so 3-4 KB per warp are in flight;
//   * for M = 1 the quantised activations live in shared memory (one copy per CTA); for M > 1
//     they are read through L1;
//   * all per-lane constants (block / sub-block position, scale selectors) are hoisted out of the
//     loop, scales are unpacked two at a time with 16-bit lane arithmetic, high nibbles are dotted
//     in place (dp4a on w & 0xF0F0F0F0, exact shift by 4 afterwards).
//
// Rows need K % 2048 == 0 (K-quants) or K % 1024 == 0 (Q8_0); other shapes use smc_gemv.cu.
// References: VecDotQ4K_* SharpMind.Core/Quantization/QuantizationKernels.Q4.cs:586-747, GetScaleMinK4_*
// QuantizationKernels.cs:177-189, VecDotQ6K_* QuantizationKernels.Q6.cs:12-235, VecDotQ8_0_*
// QuantizationKernels.Q8.cs:11-138.
#include "smc_common.cuh"

namespace {

constexpr int WARPS = 8;  // per CTA

struct XPtrs {
    const int8_t *q;     // [M][K]
    const float *d;      // [M][K/32]
    const float *sd;     // [M][K/32]
    const int16_t *s16;  // [M][K/16]
};

template <bool SMEM>
__device__ __forceinline__ uint4 ld16(const void *p)
{
    if (SMEM) return *reinterpret_cast<const uint4 *>(p);
    return __ldg(reinterpret_cast<const uint4 *>(p));
}
template <bool SMEM>
__device__ __forceinline__ float2 ld8f(const float *p)
{
    if (SMEM) return *reinterpret_cast<const float2 *>(p);
    return __ldg(reinterpret_cast<const float2 *>(p));
}
template <bool SMEM>
__device__ __forceinline__ float4 ld16f(const float *p)
{
    if (SMEM) return *reinterpret_cast<const float4 *>(p);
    return __ldg(reinterpret_cast<const float4 *>(p));
}
template <bool SMEM>
__device__ __forceinline__ float ld4f(const float *p)
{
    if (SMEM) return *p;
    return __ldg(p);
}

__device__ __forceinline__ float warp_sum32(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Copies row `m` of the activation buffers into shared memory: q | d | sd | s16, each 16-byte aligned.
__device__ __forceinline__ XPtrs stage_x(const XPtrs &g, int m, int K, uint8_t *smem, bool want_sd, bool want_s16)
{
    XPtrs s;
    int8_t *sq = reinterpret_cast<int8_t *>(smem);
    float *sdx = reinterpret_cast<float *>(smem + K);
    float *ssd = sdx + K / 32;
    int16_t *ss16 = reinterpret_cast<int16_t *>(ssd + K / 32);
    const uint4 *gq = reinterpret_cast<const uint4 *>(g.q + (size_t)m * K);
    for (int i = threadIdx.x; i < K / 16; i += blockDim.x) reinterpret_cast<uint4 *>(sq)[i] = __ldg(gq + i);
    for (int i = threadIdx.x; i < K / 32; i += blockDim.x) {
        sdx[i] = __ldg(g.d + (size_t)m * (K / 32) + i);
        if (want_sd) ssd[i] = __ldg(g.sd + (size_t)m * (K / 32) + i);
    }
    if (want_s16)
        for (int i = threadIdx.x; i < K / 16; i += blockDim.x) ss16[i] = __ldg(g.s16 + (size_t)m * (K / 16) + i);
    __syncthreads();
    s.q = sq, s.d = sdx, s.sd = ssd, s.s16 = ss16;
    return s;
}

__device__ __forceinline__ void warp_rows(int N, int &r0, int &r1)
{
    const long long W = (long long)gridDim.x * WARPS;
    const long long w = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
    r0 = (int)((long long)N * w / W);
    r1 = (int)((long long)N * (w + 1) / W);
}

// =========================================================================================== Q4_K
struct U4 {
    uint4 hdr, q0, q1;
};

template <int MT, int PF>
__global__ void __launch_bounds__(256, 2) gemv_stream_q4k(const uint8_t *__restrict__ raw, XPtrs xg, float *__restrict__ out,
                                                          int N, int K, int M)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr bool XS = (MT == 1);
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * MT;
    XPtrs xs = xg;
    if (XS) xs = stage_x(xg, m0, K, smem, true, false);

    int r0, r1;
    warp_rows(N, r0, r1);
    const int spr = K >> 11;  // steps per row
    const int nsteps = (r1 - r0) * spr;
    const int b = lane >> 2, p = lane & 3;
    const uint8_t *wp = raw + ((size_t)r0 * (K >> 8) + b) * 144;

    // lane constants for the scale unpack: sub-blocks 2p and 2p+1 (GetScaleMinK4_* on 16-bit pairs)
    const int sh = (p & 1) * 16;
    const bool low = p < 2;

    auto load = [&](int t) {
        const uint8_t *s = wp + (size_t)t * (8 * 144);
        U4 u;
        u.q0 = smc_ldg_stream16(s + 16 + 32 * p);
        u.q1 = smc_ldg_stream16(s + 32 + 32 * p);
        u.hdr = smc_ldg_stream16(s);
        return u;
    };

    U4 buf[PF];
#pragma unroll
    for (int i = 0; i < PF; ++i)
        if (i < nsteps) buf[i] = load(i);

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    int part = 0, row = r0;

    for (int t = 0; t < nsteps; t += PF) {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            if (t + i < nsteps) {
                const U4 u = buf[i];
                if (t + i + PF < nsteps) buf[i] = load(t + i + PF);

                // ---- scales of sub-blocks 2p (low byte) and 2p+1 (high byte)
                const uint32_t s0 = u.hdr.y, s1 = u.hdr.z, s2 = u.hdr.w;
                const uint32_t hp = ((low ? s0 : s1) >> sh) & 0xFFFFu;   // 16-bit pair p
                const uint32_t hp2 = ((low ? s1 : s2) >> sh) & 0xFFFFu;  // pair p + 2
                const uint32_t hm2 = (s0 >> sh) & 0xFFFFu;               // pair p - 2 (p >= 2)
                const uint32_t sc = low ? (hp & 0x3F3Fu) : ((hp2 & 0x0F0Fu) | ((hm2 >> 2) & 0x3030u));
                const uint32_t mn = low ? (hp2 & 0x3F3Fu) : (((hp2 >> 4) & 0x0F0Fu) | ((hp >> 2) & 0x3030u));
                const int sc_lo = sc & 0xFF, sc_hi = sc >> 8;
                const float mn_lo = (float)(mn & 0xFF), mn_hi = (float)(mn >> 8);
                const float d = smc_h2f((uint16_t)(u.hdr.x & 0xFFFF));
                const float dmin = smc_h2f((uint16_t)(u.hdr.x >> 16));

                const uint32_t M4 = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
                const int k0 = part * 2048 + b * 256 + 64 * p;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const int mm = XS ? 0 : min(m0 + m, M - 1);
                    const int8_t *xq = xs.q + (size_t)mm * K + k0;
                    const uint4 a0 = ld16<XS>(xq), a1 = ld16<XS>(xq + 16), c0 = ld16<XS>(xq + 32), c1 = ld16<XS>(xq + 48);
                    int lo = smc_dp4a(u.q0.x & M4, a0.x, 0);
                    lo = smc_dp4a(u.q0.y & M4, a0.y, lo);
                    lo = smc_dp4a(u.q0.z & M4, a0.z, lo);
                    lo = smc_dp4a(u.q0.w & M4, a0.w, lo);
                    lo = smc_dp4a(u.q1.x & M4, a1.x, lo);
                    lo = smc_dp4a(u.q1.y & M4, a1.y, lo);
                    lo = smc_dp4a(u.q1.z & M4, a1.z, lo);
                    lo = smc_dp4a(u.q1.w & M4, a1.w, lo);
                    int hi = smc_dp4a_us(u.q0.x & MH, c0.x, 0);
                    hi = smc_dp4a_us(u.q0.y & MH, c0.y, hi);
                    hi = smc_dp4a_us(u.q0.z & MH, c0.z, hi);
                    hi = smc_dp4a_us(u.q0.w & MH, c0.w, hi);
                    hi = smc_dp4a_us(u.q1.x & MH, c1.x, hi);
                    hi = smc_dp4a_us(u.q1.y & MH, c1.y, hi);
                    hi = smc_dp4a_us(u.q1.z & MH, c1.z, hi);
                    hi = smc_dp4a_us(u.q1.w & MH, c1.w, hi);
                    hi >>= 4;  // every term carried a factor 16: the shift is exact
                    const size_t b32 = (size_t)mm * (K / 32) + (k0 >> 5);
                    const float2 dx = ld8f<XS>(xs.d + b32);
                    const float2 sdx = ld8f<XS>(xs.sd + b32);
                    const float tsum = fmaf((float)(sc_lo * lo), dx.x, (float)(sc_hi * hi) * dx.y);
                    const float msum = fmaf(mn_lo, sdx.x, mn_hi * sdx.y);
                    acc[m] = fmaf(d, tsum, acc[m]);
                    acc[m] = fmaf(-dmin, msum, acc[m]);
                }
                if (++part == spr) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float v = warp_sum32(acc[m]);
                        if (lane == 0 && m0 + m < M) out[(size_t)(m0 + m) * N + row] = v;
                        acc[m] = 0.f;
                    }
                    part = 0;
                    ++row;
                }
            }
        }
    }
}

// =========================================================================================== Q6_K
struct U6 {
    uint4 a, b, h;
    uint2 sc;
    uint32_t d;
};

template <int MT, int PF>
__global__ void __launch_bounds__(256, 2) gemv_stream_q6k(const uint8_t *__restrict__ ql, const uint8_t *__restrict__ qh,
                                                          const int8_t *__restrict__ scp, const __half *__restrict__ dp,
                                                          XPtrs xg, float *__restrict__ out, int N, int K, int M)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr bool XS = (MT == 1);
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * MT;
    XPtrs xs = xg;
    if (XS) xs = stage_x(xg, m0, K, smem, false, true);

    int r0, r1;
    warp_rows(N, r0, r1);
    const int spr = K >> 11;
    const int nsteps = (r1 - r0) * spr;
    const int b = lane >> 2, r = lane & 3, h = r >> 1, l0 = 16 * (r & 1);
    const size_t blk0 = (size_t)r0 * (K >> 8) + b;
    const uint8_t *pql = ql + blk0 * 128 + 64 * h + l0;
    const uint8_t *pqh = qh + blk0 * 64 + 32 * h + l0;
    const int8_t *psc = scp + blk0 * 16 + 8 * h;
    const __half *pd = dp + blk0;
    const int ssel = (r & 1) ? 0 : 16;  // left shift that brings the wanted int16 of a pair to the top

    auto load = [&](int t) {
        U6 u;
        u.a = smc_ldg_stream16(pql + (size_t)t * (8 * 128));
        u.b = smc_ldg_stream16(pql + (size_t)t * (8 * 128) + 32);
        u.h = smc_ldg_stream16(pqh + (size_t)t * (8 * 64));
        u.sc = smc_ldg_stream8(psc + (size_t)t * (8 * 16));
        u.d = smc_ldg_stream2(pd + (size_t)t * 8);
        return u;
    };

    U6 buf[PF];
#pragma unroll
    for (int i = 0; i < PF; ++i)
        if (i < nsteps) buf[i] = load(i);

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    int part = 0, row = r0;

    for (int t = 0; t < nsteps; t += PF) {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            if (t + i < nsteps) {
                const U6 u = buf[i];
                if (t + i + PF < nsteps) buf[i] = load(t + i + PF);

                const uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x30303030u;
                const uint32_t wa[4] = {u.a.x, u.a.y, u.a.z, u.a.w};
                const uint32_t wb[4] = {u.b.x, u.b.y, u.b.z, u.b.w};
                const uint32_t wh[4] = {u.h.x, u.h.y, u.h.z, u.h.w};
                uint32_t q[4][4];  // [column c][word j]: six-bit codes of elements 32c + l0 + 4j .. +3
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    q[0][j] = (wa[j] & M4) | ((wh[j] << 4) & M2);
                    q[1][j] = (wb[j] & M4) | ((wh[j] << 2) & M2);
                    q[2][j] = ((wa[j] >> 4) & M4) | (wh[j] & M2);
                    q[3][j] = ((wb[j] >> 4) & M4) | ((wh[j] >> 2) & M2);
                }
                // int8 scales is + {0, 2, 4, 6}, is = l0 / 16: bytes (r&1), +2, +4, +6 of the half's 8
                const uint32_t sw0 = (r & 1) ? (u.sc.x >> 8) : u.sc.x, sw1 = (r & 1) ? (u.sc.y >> 8) : u.sc.y;
                const int scl[4] = {(int)(int8_t)(sw0 & 0xFF), (int)(int8_t)((sw0 >> 16) & 0xFF),
                                    (int)(int8_t)(sw1 & 0xFF), (int)(int8_t)((sw1 >> 16) & 0xFF)};
                const float d = smc_h2f((uint16_t)u.d);
                const int k0 = part * 2048 + b * 256 + 128 * h + l0;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const int mm = XS ? 0 : min(m0 + m, M - 1);
                    const int8_t *xq = xs.q + (size_t)mm * K + k0;
                    const float4 dx = ld16f<XS>(xs.d + (size_t)mm * (K / 32) + ((k0 - l0) >> 5));
                    const uint4 sw = ld16<XS>(xs.s16 + (size_t)mm * (K / 16) + ((k0 - l0) >> 4));
                    const uint32_t sws[4] = {sw.x, sw.y, sw.z, sw.w};
                    const float dxs[4] = {dx.x, dx.y, dx.z, dx.w};
                    float rsum = 0.f;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint4 x = ld16<XS>(xq + 32 * c);
                        int s = smc_dp4a(q[c][0], x.x, 0);
                        s = smc_dp4a(q[c][1], x.y, s);
                        s = smc_dp4a(q[c][2], x.z, s);
                        s = smc_dp4a(q[c][3], x.w, s);
                        const int sx = ((int)(sws[c] << ssel)) >> 16;  // sum of the 16 activation quants
                        s -= 32 * sx;
                        rsum = fmaf((float)(scl[c] * s), dxs[c], rsum);
                    }
                    acc[m] = fmaf(d, rsum, acc[m]);
                }
                if (++part == spr) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float v = warp_sum32(acc[m]);
                        if (lane == 0 && m0 + m < M) out[(size_t)(m0 + m) * N + row] = v;
                        acc[m] = 0.f;
                    }
                    part = 0;
                    ++row;
                }
            }
        }
    }
}

// =========================================================================================== Q8_0
struct U8 {
    uint4 q0, q1;
    uint32_t d;
};

template <int MT, int PF>
__global__ void __launch_bounds__(256, 2) gemv_stream_q8_0(const int8_t *__restrict__ qs, const __half *__restrict__ dp,
                                                           XPtrs xg, float *__restrict__ out, int N, int K, int M)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr bool XS = (MT == 1);
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * MT;
    XPtrs xs = xg;
    if (XS) xs = stage_x(xg, m0, K, smem, false, false);

    int r0, r1;
    warp_rows(N, r0, r1);
    const int spr = K >> 10;  // 32 blocks per step
    const int nsteps = (r1 - r0) * spr;
    const int8_t *pq = qs + (size_t)r0 * K + 32 * lane;
    const __half *pd = dp + (size_t)r0 * (K >> 5) + lane;

    auto load = [&](int t) {
        U8 u;
        u.q0 = smc_ldg_stream16(pq + (size_t)t * 1024);
        u.q1 = smc_ldg_stream16(pq + (size_t)t * 1024 + 16);
        u.d = smc_ldg_stream2(pd + (size_t)t * 32);
        return u;
    };

    U8 buf[PF];
#pragma unroll
    for (int i = 0; i < PF; ++i)
        if (i < nsteps) buf[i] = load(i);

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    int part = 0, row = r0;

    for (int t = 0; t < nsteps; t += PF) {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            if (t + i < nsteps) {
                const U8 u = buf[i];
                if (t + i + PF < nsteps) buf[i] = load(t + i + PF);
                const float d = smc_h2f((uint16_t)u.d);
                const int k0 = part * 1024 + 32 * lane;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const int mm = XS ? 0 : min(m0 + m, M - 1);
                    const int8_t *xq = xs.q + (size_t)mm * K + k0;
                    const uint4 a0 = ld16<XS>(xq), a1 = ld16<XS>(xq + 16);
                    int s = smc_dp4a(u.q0.x, a0.x, 0);
                    s = smc_dp4a(u.q0.y, a0.y, s);
                    s = smc_dp4a(u.q0.z, a0.z, s);
                    s = smc_dp4a(u.q0.w, a0.w, s);
                    s = smc_dp4a(u.q1.x, a1.x, s);
                    s = smc_dp4a(u.q1.y, a1.y, s);
                    s = smc_dp4a(u.q1.z, a1.z, s);
                    s = smc_dp4a(u.q1.w, a1.w, s);
                    const float dx = ld4f<XS>(xs.d + (size_t)mm * (K / 32) + (k0 >> 5));
                    acc[m] = fmaf(d * dx, (float)s, acc[m]);
                }
                if (++part == spr) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const float v = warp_sum32(acc[m]);
                        if (lane == 0 && m0 + m < M) out[(size_t)(m0 + m) * N + row] = v;
                        acc[m] = 0.f;
                    }
                    part = 0;
                    ++row;
                }
            }
        }
    }
}

int stream_ctas(const smc_ctx *ctx, int N)
{
    // at most two resident CTAs per SM; every warp gets the same number of rows (+-1)
    const int wmax = ctx->sm_count * 2 * WARPS;
    int rpw = (N + wmax - 1) / wmax;
    if (rpw < 1) rpw = 1;
    int warps = (N + rpw - 1) / rpw;
    int ctas = (warps + WARPS - 1) / WARPS;
    return ctas < 1 ? 1 : ctas;
}

size_t x_smem_bytes(int K) { return (size_t)K + (size_t)(K / 32) * 8 + (size_t)(K / 16) * 2 + 64; }

}  // namespace

bool smc_stream_supported(const smc_weight *w, int M)
{
    if (!w->fast || M < 1) return false;  // M > 8 runs as ceil(M / 8) passes over the weights
    if (w->dtype == SMC_Q8_0) return w->K % 1024 == 0;
    return w->K % 2048 == 0 && x_smem_bytes(w->K) <= 200 * 1024;
}

int smc_launch_gemv_stream(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s)
{
    const int M = a->M, N = w->N, K = w->K;
    XPtrs x{a->q, a->d, a->sd, a->s16};
    const int mt = M == 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
    dim3 grid(stream_ctas(ctx, N), (M + mt - 1) / mt);
    const size_t smem = mt == 1 ? x_smem_bytes(K) : 0;

#define SMC_STREAM_LAUNCH(KERNEL, MTV, ...)                                                                   \
    do {                                                                                                      \
        if (smem > 48 * 1024)                                                                                 \
            cudaFuncSetAttribute(KERNEL<MTV, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        KERNEL<MTV, 3><<<grid, 256, smem, s>>>(__VA_ARGS__);                                                  \
    } while (0)
#define SMC_STREAM_SWITCH(KERNEL, ...)                                        \
    switch (mt) {                                                             \
    case 1: SMC_STREAM_LAUNCH(KERNEL, 1, __VA_ARGS__); break;                 \
    case 2: SMC_STREAM_LAUNCH(KERNEL, 2, __VA_ARGS__); break;                 \
    case 4: SMC_STREAM_LAUNCH(KERNEL, 4, __VA_ARGS__); break;                 \
    default: SMC_STREAM_LAUNCH(KERNEL, 8, __VA_ARGS__); break;                \
    }

    if (w->dtype == SMC_Q4_K) {
        SMC_STREAM_SWITCH(gemv_stream_q4k, w->d_raw, x, out, N, K, M)
    } else if (w->dtype == SMC_Q6_K) {
        SMC_STREAM_SWITCH(gemv_stream_q6k, w->q6_ql, w->q6_qh, w->q6_sc, w->q6_d, x, out, N, K, M)
    } else {
        SMC_STREAM_SWITCH(gemv_stream_q8_0, w->q8_qs, w->q8_d, x, out, N, K, M)
    }
#undef SMC_STREAM_SWITCH
#undef SMC_STREAM_LAUNCH
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}
