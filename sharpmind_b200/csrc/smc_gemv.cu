// Decode-sized quantized matmul (M <= 32): out[M, N] = x[M, K] * W^T with W in Q8_0 / Q4_K / Q6_K.
//
// These kernels are bound by the one pass over the weight bytes (HBM), so the design goal is
// bytes in flight, not flops:
//   * every weight byte is fetched exactly once per launch with 16-byte streaming loads
//     (ld.global.nc.L1::no_allocate), several independent loads per lane issued before any math;
//   * a row is spread over 8/16/32 lanes ("lanes per row") and reduced with warp shuffles, so
//     short rows (K = 1024) still fill a warp and long rows (K = 14336) need no shared memory;
//   * activations are tiny next to the weights and are re-read through L1;
//   * with SMC_ACT_Q8 the inner product is integer (dp4a) on Q8_0-quantised activations and only
//     one float multiply-add per 16 or 32 elements remains; with SMC_ACT_F32 bytes become floats
//     through a PRMT + FADD pair (full-rate) and feed explicit FMAs.
//
// Unit of work per lane ("unit"):
//   Q8_0  16 quants (half a block) from the repacked planes [N][K] int8 + [N][K/32] fp16
//   Q4_K  16 bytes of qs = 16 low nibbles of sub-block a and 16 high nibbles of sub-block a+1,
//         plus the 16-byte block header, straight from the GGUF layout (144 B = 9 x 16 B)
//   Q6_K  a quarter block: the 16-byte X, Y, Z entries of one lane slot of the unit layout
//         (smc_common.cuh) -> 64 six-bit values, plus the block's scales and d
//
// References: VecDotQ8_0_* QuantizationKernels.Q8.cs:11-138, VecDotQ4K_* QuantizationKernels.Q4.cs:586-747,
// VecDotQ6K_* QuantizationKernels.Q6.cs:12-235, QuantizedMatMul_*_Wrapper QuantizationKernels.cs:11-42
// (paths under SharpMind.Core/Quantization/).
#include "smc_common.cuh"

namespace {

struct ActPtrs {
    const float *x;        // fp32 activations [M][K]
    const int8_t *q;       // Q8_0 activations [M][K]
    const float *d;        // [M][K/32]
    const float *sd;       // [M][K/32]
    const int16_t *s16;    // [M][K/16]
};

struct WPtrs {
    const uint8_t *raw;    // Q4_K blocks
    const int8_t *q8_qs;
    const __half *q8_d;
    const uint8_t *q6u;    // Q6_K units (smc_common.cuh)
};

__device__ __forceinline__ float4 ldx4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ uint4 ldq16(const int8_t *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }

__device__ __forceinline__ float dot4_ubytes(uint32_t w, float4 x, float bias, float acc)
{
    // acc += sum_j x_j * (byte_j(w) - bias'), the bias folded into the magic constant
    acc = fmaf(x.x, __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u)) - bias, acc);
    acc = fmaf(x.y, __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541u)) - bias, acc);
    acc = fmaf(x.z, __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542u)) - bias, acc);
    acc = fmaf(x.w, __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543u)) - bias, acc);
    return acc;
}
__device__ __forceinline__ float sum4(float4 x, float acc) { return acc + ((x.x + x.y) + (x.z + x.w)); }

// ------------------------------------------------------------------------------------------ Q8_0
struct FmtQ8_0 {
    struct Unit {
        uint4 w;
        float d;
    };
    static __host__ __device__ int units_per_row(int K) { return K / 16; }
    static __device__ __forceinline__ Unit zero() { return Unit{make_uint4(0, 0, 0, 0), 0.f}; }
    static __device__ __forceinline__ Unit load(const WPtrs &p, int row, int u, int K)
    {
        Unit t;
        t.w = smc_ldg_stream16(p.q8_qs + (size_t)row * K + 16 * (size_t)u);
        t.d = smc_h2f(smc_ldg_stream2(p.q8_d + (size_t)row * (K / 32) + (u >> 1)));
        return t;
    }
    static __device__ __forceinline__ float dot_q8(const Unit &t, const ActPtrs &a, int m, int u, int K)
    {
        uint4 x = ldq16(a.q + (size_t)m * K + 16 * (size_t)u);
        int s = smc_dp4a(t.w.x, x.x, 0);
        s = smc_dp4a(t.w.y, x.y, s);
        s = smc_dp4a(t.w.z, x.z, s);
        s = smc_dp4a(t.w.w, x.w, s);
        float dx = __ldg(a.d + (size_t)m * (K / 32) + (u >> 1));
        return (t.d * dx) * (float)s;
    }
    static __device__ __forceinline__ float dot_f32(const Unit &t, const ActPtrs &a, int m, int u, int K)
    {
        const float *x = a.x + (size_t)m * K + 16 * (size_t)u;
        const float bias = 8388608.0f + 128.0f;  // bytes are flipped to unsigned (q + 128)
        float p = 0.f;
        p = dot4_ubytes(t.w.x ^ 0x80808080u, ldx4(x), bias, p);
        p = dot4_ubytes(t.w.y ^ 0x80808080u, ldx4(x + 4), bias, p);
        p = dot4_ubytes(t.w.z ^ 0x80808080u, ldx4(x + 8), bias, p);
        p = dot4_ubytes(t.w.w ^ 0x80808080u, ldx4(x + 12), bias, p);
        return t.d * p;
    }
};

// ------------------------------------------------------------------------------------------ Q4_K
struct FmtQ4_K {
    struct Unit {
        uint4 hdr;  // d | dmin<<16, scales[0..3], scales[4..7], scales[8..11]
        uint4 qs;
    };
    static __host__ __device__ int units_per_row(int K) { return (K / 256) * 8; }
    static __device__ __forceinline__ Unit zero() { return Unit{make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}; }
    static __device__ __forceinline__ Unit load(const WPtrs &p, int row, int u, int K)
    {
        size_t blk = (size_t)row * (K / 256) + (u >> 3);
        const uint8_t *b = p.raw + blk * 144;
        Unit t;
        t.qs = smc_ldg_stream16(b + 16 + 16 * (u & 7));
        t.hdr = smc_ldg_stream16(b);
        return t;
    }
    static __device__ __forceinline__ void scales(const Unit &t, int a, float &d, float &dmin, int &sc0, int &mn0,
                                                  int &sc1, int &mn1)
    {
        d = smc_h2f((uint16_t)(t.hdr.x & 0xFFFF));
        dmin = smc_h2f((uint16_t)(t.hdr.x >> 16));
        smc_k4_scale_min(t.hdr.y, t.hdr.z, t.hdr.w, a, sc0, mn0);
        smc_k4_scale_min(t.hdr.y, t.hdr.z, t.hdr.w, a + 1, sc1, mn1);
    }
    static __device__ __forceinline__ float dot_q8(const Unit &t, const ActPtrs &a, int m, int u, int K)
    {
        int kb = u >> 3, part = u & 7, sa = part & ~1, e = 16 * (part & 1);
        float d, dmin;
        int sc0, mn0, sc1, mn1;
        scales(t, sa, d, dmin, sc0, mn0, sc1, mn1);
        const int8_t *xq = a.q + (size_t)m * K + (size_t)kb * 256 + 32 * sa + e;
        uint4 xl = ldq16(xq), xh = ldq16(xq + 32);
        const uint32_t M4 = 0x0F0F0F0Fu;
        int lo = smc_dp4a(t.qs.x & M4, xl.x, 0);
        lo = smc_dp4a(t.qs.y & M4, xl.y, lo);
        lo = smc_dp4a(t.qs.z & M4, xl.z, lo);
        lo = smc_dp4a(t.qs.w & M4, xl.w, lo);
        int hi = smc_dp4a((t.qs.x >> 4) & M4, xh.x, 0);
        hi = smc_dp4a((t.qs.y >> 4) & M4, xh.y, hi);
        hi = smc_dp4a((t.qs.z >> 4) & M4, xh.z, hi);
        hi = smc_dp4a((t.qs.w >> 4) & M4, xh.w, hi);
        size_t b32 = (size_t)m * (K / 32) + (size_t)kb * 8;
        float2 dx = __ldg(reinterpret_cast<const float2 *>(a.d + b32 + sa));
        float sdp = __ldg(a.sd + b32 + part);  // this lane carries the min term of sub-block `part`
        float t0 = fmaf((float)(sc0 * lo), dx.x, (float)(sc1 * hi) * dx.y);
        float mnp = (float)((part & 1) ? mn1 : mn0);
        return fmaf(d, t0, -(dmin * mnp) * sdp);
    }
    static __device__ __forceinline__ float dot_f32(const Unit &t, const ActPtrs &a, int m, int u, int K)
    {
        int kb = u >> 3, part = u & 7, sa = part & ~1, e = 16 * (part & 1);
        float d, dmin;
        int sc0, mn0, sc1, mn1;
        scales(t, sa, d, dmin, sc0, mn0, sc1, mn1);
        const float *x = a.x + (size_t)m * K + (size_t)kb * 256 + 32 * sa + e;
        const uint32_t M4 = 0x0F0F0F0Fu;
        const float bias = 8388608.0f;
        float dl = 0.f, sl = 0.f, dh = 0.f, sh = 0.f;
        const uint32_t w[4] = {t.qs.x, t.qs.y, t.qs.z, t.qs.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float4 xl = ldx4(x + 4 * j), xh = ldx4(x + 32 + 4 * j);
            dl = dot4_ubytes(w[j] & M4, xl, bias, dl);
            dh = dot4_ubytes((w[j] >> 4) & M4, xh, bias, dh);
            sl = sum4(xl, sl);
            sh = sum4(xh, sh);
        }
        // value = (s*d)*v - (m*dmin), as the FMA tier forms it (QuantizationKernels.Q4.cs:715-732)
        float r = ((float)sc0 * d) * dl;
        r = fmaf((float)sc1 * d, dh, r);
        r = fmaf(-((float)mn0 * dmin), sl, r);
        r = fmaf(-((float)mn1 * dmin), sh, r);
        return r;
    }
};

// ------------------------------------------------------------------------------------------ Q6_K
struct FmtQ6_K {
    struct Unit {
        uint4 a, b, h;  // the X, Y, Z entries of lane slot (block, half, sixteen)
        uint2 sc;       // the 8 int8 scales of that half
        float d;
    };
    static __host__ __device__ int units_per_row(int K) { return (K / 256) * 4; }
    static __device__ __forceinline__ Unit zero()
    {
        uint4 z = make_uint4(0, 0, 0, 0);
        return Unit{z, z, z, make_uint2(0, 0), 0.f};
    }
    static __device__ __forceinline__ Unit load(const WPtrs &p, int row, int u, int K)
    {
        size_t blk = (size_t)row * (K / 256) + (u >> 2);
        int h = (u >> 1) & 1;
        const uint8_t *slot = p.q6u + smc_q6u_slot(blk, h, u & 1);
        Unit t;
        t.a = smc_ldg_stream16(slot);
        t.b = smc_ldg_stream16(slot + SMC_Q6U_Y);
        t.h = smc_ldg_stream16(slot + SMC_Q6U_Z);
        t.sc = smc_ldg_stream8(p.q6u + smc_q6u_scales(blk) + 8 * h);
        t.d = smc_h2f(smc_ldg_stream2(p.q6u + smc_q6u_d(blk)));
        return t;
    }
    // six-bit codes of column c (0..3) of the half, word j (0..3): elements 32c + l0 + 4j .. +3
    static __device__ __forceinline__ uint32_t codes(uint32_t a, uint32_t b, uint32_t h, int c)
    {
        uint32_t q[4];
        smc_q6u_codes(a, b, h, q);
        return q[c];
    }
    static __device__ __forceinline__ int scale_of(const Unit &t, int u, int c)
    {
        int idx = (u & 1) + 2 * c;  // is + {0, 2, 4, 6}
        uint32_t wsel = idx < 4 ? t.sc.x : t.sc.y;
        return (int)(int8_t)((wsel >> (8 * (idx & 3))) & 0xFF);
    }
    static __device__ __forceinline__ float dot_q8(const Unit &t, const ActPtrs &a, int m, int u, int K)
    {
        int kb = u >> 2, h = (u >> 1) & 1, l0 = 16 * (u & 1);
        size_t k0 = (size_t)kb * 256 + 128 * h + l0;
        const int8_t *xq = a.q + (size_t)m * K + k0;
        const float *dx = a.d + (size_t)m * (K / 32) + (size_t)kb * 8 + 4 * h;
        const int16_t *s16 = a.s16 + (size_t)m * (K / 16) + k0 / 16;
        const uint32_t wa[4] = {t.a.x, t.a.y, t.a.z, t.a.w};
        const uint32_t wb[4] = {t.b.x, t.b.y, t.b.z, t.b.w};
        const uint32_t wh[4] = {t.h.x, t.h.y, t.h.z, t.h.w};
        float r = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint4 x = ldq16(xq + 32 * c);
            const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
            int s = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) s = smc_dp4a(codes(wa[j], wb[j], wh[j], c), xs[j], s);
            s -= 32 * (int)__ldg(s16 + 2 * c);  // sum (q - 32) * x = sum q*x - 32 * sum x
            r = fmaf((float)(scale_of(t, u, c) * s), __ldg(dx + c), r);
        }
        return t.d * r;
    }
    static __device__ __forceinline__ float dot_f32(const Unit &t, const ActPtrs &a, int m, int u, int K)
    {
        int kb = u >> 2, h = (u >> 1) & 1, l0 = 16 * (u & 1);
        const float *x = a.x + (size_t)m * K + (size_t)kb * 256 + 128 * h + l0;
        const uint32_t wa[4] = {t.a.x, t.a.y, t.a.z, t.a.w};
        const uint32_t wb[4] = {t.b.x, t.b.y, t.b.z, t.b.w};
        const uint32_t wh[4] = {t.h.x, t.h.y, t.h.z, t.h.w};
        const float bias = 8388608.0f + 32.0f;
        float r = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float p = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) p = dot4_ubytes(codes(wa[j], wb[j], wh[j], c), ldx4(x + 32 * c + 4 * j), bias, p);
            r = fmaf(t.d * (float)scale_of(t, u, c), p, r);
        }
        return r;
    }
};

// ------------------------------------------------------------------------------------------ kernel
// One launch covers weight rows [0, N) and activation rows m0 = blockIdx.y * MT .. m0 + MT - 1.
// A warp owns 32/lpr consecutive rows at a time; lane `sub` of a row takes units sub, sub + lpr, ...
template <class Fmt, int MT, int UNR, bool Q8ACT>
__global__ void __launch_bounds__(256) gemv_kernel(WPtrs wp, ActPtrs ap, float *__restrict__ out, int N, int K, int M,
                                                   int lpr)
{
    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * (blockDim.x >> 5);
    const int rpw = 32 / lpr;
    const int sub = lane % lpr;
    const int U = Fmt::units_per_row(K);
    const int m0 = blockIdx.y * MT;
    const int ngroups = (N + rpw - 1) / rpw;

    for (int g = warp; g < ngroups; g += nwarps) {
        const int row = g * rpw + lane / lpr;
        const bool row_ok = row < N;
        const int rrow = row_ok ? row : N - 1;
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;

        for (int u0 = sub; u0 < U; u0 += lpr * UNR) {
            typename Fmt::Unit t[UNR];
#pragma unroll
            for (int j = 0; j < UNR; ++j) {
                int u = u0 + j * lpr;
                t[j] = (u < U) ? Fmt::load(wp, rrow, u, K) : Fmt::zero();
            }
#pragma unroll
            for (int j = 0; j < UNR; ++j) {
                int u = u0 + j * lpr;
                if (u < U) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        int mm = min(m0 + m, M - 1);
                        acc[m] += Q8ACT ? Fmt::dot_q8(t[j], ap, mm, u, K) : Fmt::dot_f32(t[j], ap, mm, u, K);
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = smc_group_sum_rt(acc[m], lpr);
            if (sub == 0 && row_ok && m0 + m < M) out[(size_t)(m0 + m) * N + row] = v;
        }
    }
}

int pick_lpr(int units)
{
    if (units >= 64) return 32;
    if (units >= 32) return 16;
    return 8;
}

template <class Fmt, int UNR, bool Q8ACT>
int launch_fmt(smc_ctx *ctx, const WPtrs &wp, const ActPtrs &ap, float *out, int N, int K, int M, cudaStream_t s)
{
    const int U = Fmt::units_per_row(K);
    const int lpr = pick_lpr(U);
    const int rpw = 32 / lpr;
    const int groups = (N + rpw - 1) / rpw;
    const int warps_per_cta = 8;
    int ctas = (groups + warps_per_cta - 1) / warps_per_cta;
    const int max_ctas = ctx->sm_count * 8;
    if (ctas > max_ctas) ctas = max_ctas;
    if (ctas < 1) ctas = 1;
    // rows of x per pass: as many as keep the weights read once for small M
    int mt = Q8ACT ? (M >= 8 ? 8 : (M >= 4 ? 4 : (M >= 2 ? 2 : 1))) : (M >= 4 ? 4 : (M >= 2 ? 2 : 1));
    dim3 grid(ctas, (M + mt - 1) / mt);
    switch (mt) {
    case 8:
        if (Q8ACT) gemv_kernel<Fmt, 8, UNR, Q8ACT><<<grid, 256, 0, s>>>(wp, ap, out, N, K, M, lpr);
        break;
    case 4: gemv_kernel<Fmt, 4, UNR, Q8ACT><<<grid, 256, 0, s>>>(wp, ap, out, N, K, M, lpr); break;
    case 2: gemv_kernel<Fmt, 2, UNR, Q8ACT><<<grid, 256, 0, s>>>(wp, ap, out, N, K, M, lpr); break;
    default: gemv_kernel<Fmt, 1, UNR, Q8ACT><<<grid, 256, 0, s>>>(wp, ap, out, N, K, M, lpr); break;
    }
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

WPtrs wptrs(const smc_weight *w)
{
    WPtrs p;
    p.raw = w->d_raw;
    p.q8_qs = w->q8_qs;
    p.q8_d = w->q8_d;
    p.q6u = w->q6u;
    return p;
}

// ------------------------------------------------------------------------------------------ SMC_REF_ORDER
// One thread per output element, walking the row exactly as the scalar tier does: fp32 products
// and weights rounded where the reference rounds them, running sum in fp64, flat-tensor block
// addressing and the reference's own loop bounds for rows that start or end inside a block.
__device__ float ref_vecdot_q8_0(const float *x, const uint8_t *raw, int col, int K)
{
    int nb = (K + 31) / 32;
    double sum = 0.0;
    for (int b = 0; b < nb; ++b) {
        const uint8_t *blk = raw + ((size_t)col * nb + b) * 34;
        float d = smc_h2f((uint16_t)(blk[0] | (blk[1] << 8)));
        const int8_t *q = reinterpret_cast<const int8_t *>(blk + 2);
        int end = min(32, K - b * 32);
        for (int i = 0; i < end; ++i) {
            float w = __fmul_rn((float)q[i], d);
            sum += (double)__fmul_rn(x[b * 32 + i], w);
        }
    }
    return (float)sum;
}

__device__ int ref_k4_scale(int j, const uint8_t *sc)
{
    return j < 4 ? (sc[j] & 0x3F) : ((sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4));
}
__device__ int ref_k4_min(int j, const uint8_t *sc)
{
    return j < 4 ? (sc[j + 4] & 0x3F) : ((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
}

__device__ float ref_vecdot_q4_K(const float *x, const uint8_t *raw, int col, int K)
{
    long long flat = (long long)col * K;
    long long startBlock = flat / 256;
    int cbs = (int)(flat % 256);
    int nb = (K + 255) / 256;
    double sum = 0.0;
    for (int b = 0; b < nb; ++b) {
        const uint8_t *blk = raw + (size_t)(startBlock + b) * 144;
        float dS = smc_h2f((uint16_t)(blk[0] | (blk[1] << 8)));
        float mS = smc_h2f((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *sc = blk + 4, *qs = blk + 16;
        int cur = b == 0 ? cbs : 0;
        int end = min(256, K + cbs - b * 256);
        for (int n16 = cur; n16 < end; n16 += 128)
            for (int j = 0; j < 4 && n16 + j * 32 < end; ++j) {
                int base = n16 + j * 32;
                int isc = (n16 / 128) * 4 + j;
                float s = (float)ref_k4_scale(isc, sc), m = (float)ref_k4_min(isc, sc);
                for (int l = 0; l < 32 && base + l < end; ++l) {
                    int idx = base + l;
                    int v = (qs[(idx / 64) * 32 + (idx % 32)] >> (((idx % 64) / 32) * 4)) & 0x0F;
                    float w = __fsub_rn(__fmul_rn(__fmul_rn(s, (float)v), dS), __fmul_rn(m, mS));
                    sum += (double)__fmul_rn(x[b * 256 + idx - cbs], w);
                }
            }
    }
    return (float)sum;
}

// `avail` = floats readable from x: when a row ends inside a 128-element half the reference's loop
// still reads the l+64 / l+96 partners, up to 96 floats past the row (into the next input row, or
// past the tensor for the last row).  Reads inside the activation tensor are reproduced; reads past
// its end return 0 instead of touching memory the caller never handed over.
__device__ float ref_vecdot_q6_K(const float *x, const uint8_t *raw, int col, int K, long long avail)
{
    auto X = [&](int i) { return i < avail ? x[i] : 0.0f; };
    long long flat = (long long)col * K;
    long long startBlock = flat / 256;
    int cbs = (int)(flat % 256);
    int nb = (K + 255) / 256;
    double sum = 0.0;
    for (int b = 0; b < nb; ++b) {
        const uint8_t *blk = raw + (size_t)(startBlock + b) * 210;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *scales = reinterpret_cast<const int8_t *>(blk + 192);
        float d = smc_h2f((uint16_t)(blk[208] | (blk[209] << 8)));
        int cur = b == 0 ? cbs : 0;
        int end = min(256, K + cbs - b * 256);
        for (int nOff = cur; nOff < end; nOff += 128) {
            const uint8_t *pql = ql + (nOff == 0 ? 0 : 64);
            const uint8_t *pqh = qh + (nOff == 0 ? 0 : 32);
            const int8_t *psc = scales + (nOff == 0 ? 0 : 8);
            int halfRem = min(128, end - nOff);
            for (int l = 0; l < 32 && l < halfRem; ++l) {
                int is = l / 16;
                int q1 = (pql[l] & 0x0F) | ((pqh[l] & 0x03) << 4);
                int q2 = (pql[l + 32] & 0x0F) | (((pqh[l] >> 2) & 0x03) << 4);
                int q3 = ((pql[l] >> 4) & 0x0F) | (((pqh[l] >> 4) & 0x03) << 4);
                int q4 = ((pql[l + 32] >> 4) & 0x0F) | (((pqh[l] >> 6) & 0x03) << 4);
                int i1 = b * 256 + nOff + l - cbs, i2 = i1 + 32;
                int lim = b * 256 + end - cbs;
                float w1 = __fmul_rn(__fmul_rn(d, (float)psc[is + 0]), (float)(q1 - 32));
                if (i2 >= lim) {
                    if (i1 < lim) sum += (double)__fmul_rn(X(i1), w1);
                    break;
                }
                float w2 = __fmul_rn(__fmul_rn(d, (float)psc[is + 2]), (float)(q2 - 32));
                float w3 = __fmul_rn(__fmul_rn(d, (float)psc[is + 4]), (float)(q3 - 32));
                float w4 = __fmul_rn(__fmul_rn(d, (float)psc[is + 6]), (float)(q4 - 32));
                sum += (double)__fmul_rn(X(i1), w1);
                sum += (double)__fmul_rn(X(i2), w2);
                sum += (double)__fmul_rn(X(i1 + 64), w3);
                sum += (double)__fmul_rn(X(i1 + 96), w4);
            }
        }
    }
    return (float)sum;
}

__global__ void gemv_ref_kernel(const float *__restrict__ x, const uint8_t *__restrict__ raw, float *__restrict__ out,
                                int dtype, int N, int K, int M, int col0, int col1)
{
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    int ncols = col1 - col0;
    if (t >= (long long)M * ncols) return;
    int m = (int)(t / ncols), col = col0 + (int)(t % ncols);
    const float *xr = x + (size_t)m * K;
    float r;
    if (dtype == SMC_Q8_0) r = ref_vecdot_q8_0(xr, raw, col, K);
    else if (dtype == SMC_Q4_K) r = ref_vecdot_q4_K(xr, raw, col, K);
    else r = ref_vecdot_q6_K(xr, raw, col, K, (long long)(M - m) * K);
    out[(size_t)m * N + col] = r;
}

// Per-block integer sums for verification: one thread per (column, 32-element block).
__global__ void block_isums_kernel(const int8_t *__restrict__ xq, const uint8_t *__restrict__ raw, int dtype, int K,
                                   int col0, int col1, int32_t *__restrict__ sums)
{
    int nb32 = K / 32;
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)(col1 - col0) * nb32) return;
    int col = col0 + (int)(t / nb32), b = (int)(t % nb32);
    int s = 0;
    if (dtype == SMC_Q8_0) {
        const int8_t *qw = reinterpret_cast<const int8_t *>(raw + ((size_t)col * nb32 + b) * 34 + 2);
        for (int i = 0; i < 32; ++i) s += (int)qw[i] * (int)xq[b * 32 + i];
    } else {
        size_t blk = (size_t)col * (K / 256) + b / 8;
        int sb = b % 8;
        for (int i = 0; i < 32; ++i) {
            int e = sb * 32 + i, code;
            if (dtype == SMC_Q4_K) {
                const uint8_t *qs = raw + blk * 144 + 16;
                code = (qs[(e / 64) * 32 + (e % 32)] >> (((e % 64) / 32) * 4)) & 0x0F;
            } else {
                const uint8_t *bp = raw + blk * 210;
                int h = e / 128, local = e % 128, l = local % 32, c = local / 32;
                const uint8_t *pql = bp + 64 * h, *pqh = bp + 128 + 32 * h;
                int lo = (c & 1) ? pql[l + 32] : pql[l];
                lo = (c >= 2) ? (lo >> 4) & 0x0F : lo & 0x0F;
                code = (lo | (((pqh[l] >> (2 * c)) & 0x03) << 4)) - 32;
            }
            s += code * (int)xq[b * 32 + i];
        }
    }
    sums[t] = s;
}

}  // namespace

int smc_launch_gemv_f32(smc_ctx *ctx, const float *x, const smc_weight *w, float *out, int M, cudaStream_t s)
{
    ActPtrs ap{};
    ap.x = x;
    WPtrs wp = wptrs(w);
    switch (w->dtype) {
    case SMC_Q8_0: return launch_fmt<FmtQ8_0, 4, false>(ctx, wp, ap, out, w->N, w->K, M, s);
    case SMC_Q4_K: return launch_fmt<FmtQ4_K, 4, false>(ctx, wp, ap, out, w->N, w->K, M, s);
    case SMC_Q6_K: return launch_fmt<FmtQ6_K, 2, false>(ctx, wp, ap, out, w->N, w->K, M, s);
    }
    return smc_fail(ctx, SMC_E_UNSUPPORTED, "dtype %d has no matmul kernel", w->dtype);
}

int smc_launch_gemv_q8(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s)
{
    // two or more rows: per-block integer sums on the int8 tensor-core path; weights through the bulk-copy ring where
    // the shape allows it (whole steps per row, whole 16-row tiles), else fragments fetched from global memory
    // (measured: alone, the ring kernel wins by 10 % for Q4_K at 8 rows on a 28672-row matrix and nowhere else; inside a
    // stack of launches it loses, so it is taken only when the option asks for it: 1 = Q4_K, 2 = every format)
    if ((ctx->mt_ring == 2 || (ctx->mt_ring == 1 && w->dtype == SMC_Q4_K)) && smc_mt_supported(w, a->M))
        return smc_launch_gemv_mt(ctx, a, w, out, s);
    if (smc_mma_supported(w, a->M)) return smc_launch_gemv_mma(ctx, a, w, out, s);
    // one row: the bulk-copy kernel, fed the rows quantised beforehand
    if (smc_tma_supported(w, a->M)) return smc_launch_gemv_tma(ctx, a, w, out, s);
    ActPtrs ap{};
    ap.q = a->q;
    ap.d = a->d;
    ap.sd = a->sd;
    ap.s16 = a->s16;
    WPtrs wp = wptrs(w);
    switch (w->dtype) {
    case SMC_Q8_0: return launch_fmt<FmtQ8_0, 4, true>(ctx, wp, ap, out, w->N, w->K, a->M, s);
    case SMC_Q4_K: return launch_fmt<FmtQ4_K, 4, true>(ctx, wp, ap, out, w->N, w->K, a->M, s);
    case SMC_Q6_K: return launch_fmt<FmtQ6_K, 2, true>(ctx, wp, ap, out, w->N, w->K, a->M, s);
    }
    return smc_fail(ctx, SMC_E_UNSUPPORTED, "dtype %d has no matmul kernel", w->dtype);
}

int smc_launch_gemv_ref(smc_ctx *ctx, const float *x, const smc_weight *w, float *out, int M, int col0, int col1,
                        cudaStream_t s)
{
    if (!w->d_raw) return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight was registered without SMC_W_KEEP_RAW");
    long long total = (long long)M * (col1 - col0);
    if (total <= 0) return SMC_OK;
    int threads = 128;
    long long blocks = (total + threads - 1) / threads;
    gemv_ref_kernel<<<(unsigned)blocks, threads, 0, s>>>(x, w->d_raw, out, w->dtype, w->N, w->K, M, col0, col1);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_launch_block_isums(smc_ctx *ctx, const smc_q8act *a, int m, const smc_weight *w, int col0, int col1,
                           int32_t *sums, cudaStream_t s)
{
    if (!w->d_raw) return smc_fail(ctx, SMC_E_UNSUPPORTED, "weight was registered without SMC_W_KEEP_RAW");
    long long total = (long long)(col1 - col0) * (w->K / 32);
    if (total <= 0) return SMC_OK;
    int threads = 128;
    block_isums_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, s>>>(
        a->q + (size_t)m * a->K, w->d_raw, w->dtype, w->K, col0, col1, sums);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}
