// TMA-staged streaming GEMV for Q8_0-quantised activations, the decode hot kernel.
//
// Each warp owns a contiguous range of weight rows, i.e. one contiguous byte stream per weight
// array, and consumes it in "steps" of 32 lane-units (Q4_K / Q6_K: 8 blocks = 2048 elements,
// Q8_0: 32 blocks = 1024 elements).  The bytes of a step are brought into a warp-private ring of
// shared-memory slots by bulk asynchronous copies (cp.async.bulk global -> shared, completion on an
// mbarrier) issued by one lane, up to `slots` steps ahead of the math:
//   * memory-level parallelism is set by shared memory, not by registers (6-8 slots x 8 warps x
//     2-3 CTAs keep more than 100 KB per SM in flight, against the ~45 KB Little's law asks for);
//   * HBM and L2 see whole contiguous ranges, never half-used sectors;
//   * the lanes read their unit with conflict-free 128-bit shared loads, and for M = 1 the
//     activation row is in shared memory too (16-byte chunks permuted per format so that the
//     strided reads of eight lanes fall in eight different bank groups): the inner loop issues no
//     global loads at all.
// The kernels are bound by instruction issue before they are bound by HBM, so the inner loop is
// written for a short instruction stream: 32-bit shared addresses and explicit ld.shared, every
// lane-constant offset hoisted, Q4_K scale / min bytes unpacked with two PRMTs, high nibbles dotted
// in place (dp4a on w & 0xF0F0F0F0, exact shift by 4 afterwards), independent dp4a chains.
// A slot is re-armed only after __syncwarp(): every lane has passed its wait and read its data, so
// no lane can be left waiting on a phase that has already been reused.  Every wait is bounded; on
// expiry the warp raises a flag in device memory (read back by smc_device_status) and stops.
//
// Arithmetic is identical to the other SMC_ACT_Q8 kernels: exact int32 block dots (dp4a), one fp32
// multiply-add per 32-element block.  Shapes: K % 2048 == 0 (K-quants) / K % 1024 == 0 (Q8_0).
// References: VecDotQ4K_* SharpMind.Core/Quantization/QuantizationKernels.Q4.cs:586-747, GetScaleMinK4_*
// QuantizationKernels.cs:177-189, VecDotQ6K_* QuantizationKernels.Q6.cs:12-235, VecDotQ8_0_*
// QuantizationKernels.Q8.cs:11-138.
#include <stdlib.h>

#include "smc_common.cuh"
#include "smc_gather.cuh"

namespace {

constexpr int WARPS = 8;
constexpr unsigned WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (unsigned i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// explicit shared-space loads on 32-bit addresses
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16u(uint32_t a)
{
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

__device__ __forceinline__ float warp_sum32(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct XPtrs {
    const int8_t *q;
    const float *d;
    const float *sd;
    const int16_t *s16;
    const float *xf;  // when set (M = 1): fp32 activations, quantised to Q8_0 while they are staged
    const float *xu;  // when set too: the staged row is SiLU(xf[i]) * xu[i] (FfnKernels.Gated's activation)
    // when nw is set: the staged row is RMSNorm(xf + xadd) * nw (xadd may be null), and CTA 0 writes xf + xadd to
    // xsum: the residual add and the norm of a decoder block folded into the matmul that consumes them
    const float *xadd, *nw;
    float *xsum;
    float eps;
};

// Shared layout of the staged activation row: q | d | sd | s16.  The quants are stored in 16-byte
// chunks permuted by Math::swz so that the 128-bit reads of a quarter warp (eight lanes, each format
// with its own stride pattern) fall in eight different bank groups.
template <class Math>
__device__ __forceinline__ void stage_x(const XPtrs &g, int m, int K, uint8_t *sx)
{
    uint4 *sq = reinterpret_cast<uint4 *>(sx);
    float *sdx = reinterpret_cast<float *>(sx + K);
    float *ssd = sdx + K / 32;
    int16_t *ss16 = reinterpret_cast<int16_t *>(ssd + K / 32);
    const uint4 *gq = reinterpret_cast<const uint4 *>(g.q + (size_t)m * K);
    for (int i = threadIdx.x; i < K / 16; i += blockDim.x) sq[Math::swz(i)] = __ldg(gq + i);
    for (int i = threadIdx.x; i < K / 32; i += blockDim.x) {
        sdx[i] = __ldg(g.d + (size_t)m * (K / 32) + i);
        if (Math::SD) ssd[i] = __ldg(g.sd + (size_t)m * (K / 32) + i);
    }
    if (Math::S16)
        for (int i = threadIdx.x; i < K / 16; i += blockDim.x) ss16[i] = __ldg(g.s16 + (size_t)m * (K / 16) + i);
}
// Quantises the eight values of chunk c (lanes 4b .. 4b+3 hold the four chunks of block b) and stores them, their
// block scale and sums in the staged layout: the rules of QuantizedKVCache.QuantizeRowQ8_0 (d = amax/127, 1 for a
// zero block, stored through fp16; q = round-half-even(x/d)).
template <class Math>
__device__ __forceinline__ void quant_chunk(const float (&v)[8], int c, int K, uint8_t *sx)
{
    float *sdx = reinterpret_cast<float *>(sx + K);
    float *ssd = sdx + K / 32;
    int16_t *ss16 = reinterpret_cast<int16_t *>(ssd + K / 32);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float scale = __fdiv_rn(amax, 127.0f);
    if (amax == 0.0f) scale = 1.0f;
    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[i] = max(-128, min(127, __float2int_rn(__fdiv_rn(v[i], scale))));
        s += q[i];
    }
    uint2 packed;
    packed.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    packed.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
    *reinterpret_cast<uint2 *>(sx + 16 * Math::swz(c >> 1) + 8 * (c & 1)) = packed;
    const int s16v = s + __shfl_xor_sync(0xffffffffu, s, 1);
    const int total = s16v + __shfl_xor_sync(0xffffffffu, s16v, 2);
    const int blk = c >> 2;
    if (Math::S16 && (c & 1) == 0) ss16[blk * 2 + ((c >> 1) & 1)] = (int16_t)s16v;
    if ((c & 3) == 0) {
        const float df = __half2float(__float2half_rn(scale));
        sdx[blk] = df;
        if (Math::SD) ssd[blk] = df * (float)total;
    }
}

// Same layout, filled by quantising an fp32 row on the fly.  Four consecutive lanes share a 32-element block,
// eight elements each; all loads of a batch are issued before any arithmetic so the row costs one memory
// latency, not one per block.  With `up` the row is SiLU(x) * up in the arithmetic of the stand-alone kernel.
template <class Math>
__device__ __forceinline__ void stage_x_quant(const float *x, const float *up, int K, uint8_t *sx)
{
    const int nchunks = K / 8;  // K is a multiple of 1024, so whole warps stay converged
    constexpr int UB = 4;
    for (int c0 = threadIdx.x; c0 < nchunks; c0 += UB * blockDim.x) {
        float4 va[UB], vb[UB];
#pragma unroll
        for (int j = 0; j < UB; ++j) {
            const int c = c0 + j * blockDim.x;
            if (c < nchunks) {
                va[j] = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c);
                vb[j] = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c + 1);
            }
        }
#pragma unroll
        for (int j = 0; j < UB; ++j) {
            const int c = c0 + j * blockDim.x;
            if (c < nchunks) {  // uniform per warp: nchunks is a multiple of 128
                float v[8] = {va[j].x, va[j].y, va[j].z, va[j].w, vb[j].x, vb[j].y, vb[j].z, vb[j].w};
                if (up) {  // g / (1 + exp(-g)) * u
                    const float4 ua = __ldg(reinterpret_cast<const float4 *>(up) + 2 * c), ub = __ldg(reinterpret_cast<const float4 *>(up) + 2 * c + 1);
                    const float u[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = __fdiv_rn(v[i], 1.0f + expf(-v[i])) * u[i];
                }
                quant_chunk<Math>(v, c, K, sx);
            }
        }
    }
}

// The residual add and the RMSNorm that precede a matmul in a decoder block, done while its activation row is
// staged: v = x + add (add may be null), xsum = v (written by the CTA that is given a pointer), row = v * rsqrt(mean
// v^2 + eps) * w, quantised as above.  K <= 8192: a thread keeps its (at most four) chunks in registers between the
// sum of squares and the scaling.  The sum of squares is taken in a fixed order (thread chunks in order, warp
// butterfly, warps in order), which is not the order of the stand-alone norm kernel: results agree to rounding.
template <class Math>
__device__ __forceinline__ void stage_x_addnorm_quant(const float *x, const float *add, const float *w, float eps, float *xsum,
                                                      int K, uint8_t *sx)
{
    __shared__ float red[8];
    const int nchunks = K / 8;
    constexpr int UB = 4;
    float v[UB][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < UB; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nchunks) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c), b = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c + 1);
            v[j][0] = a.x, v[j][1] = a.y, v[j][2] = a.z, v[j][3] = a.w, v[j][4] = b.x, v[j][5] = b.y, v[j][6] = b.z, v[j][7] = b.w;
            if (add) {
                const float4 p = __ldg(reinterpret_cast<const float4 *>(add) + 2 * c), q = __ldg(reinterpret_cast<const float4 *>(add) + 2 * c + 1);
                v[j][0] += p.x, v[j][1] += p.y, v[j][2] += p.z, v[j][3] += p.w, v[j][4] += q.x, v[j][5] += q.y, v[j][6] += q.z, v[j][7] += q.w;
            }
            if (xsum) {
                reinterpret_cast<float4 *>(xsum)[2 * c] = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
                reinterpret_cast<float4 *>(xsum)[2 * c + 1] = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[j][i], v[j][i], ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = red[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
    const float inv = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(tot, (float)K) + eps));
#pragma unroll
    for (int j = 0; j < UB; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nchunks) {
            const float4 g0 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * c), g1 = __ldg(reinterpret_cast<const float4 *>(w) + 2 * c + 1);
            const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float r[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = (v[j][i] * inv) * g[i];
            quant_chunk<Math>(r, c, K, sx);
        }
    }
}
__host__ __device__ inline size_t x_bytes(int K) { return (size_t)K + (size_t)(K / 32) * 8 + (size_t)(K / 16) * 2; }

// Where the weight arrays of a format start (piece sizes and slot offsets are Math constants).
struct StepSrc {
    const uint8_t *base[4];  // first step of row 0 in each weight array
};

// Fetches stage `g` (SS consecutive steps, contiguous in every weight array) into a slot.  PIECES and
// the per-piece sizes are compile-time so that the elected lane spends a handful of instructions here.
template <class Math, int SS>
__device__ __forceinline__ void issue_stage(const StepSrc &s, long long g, uint32_t slot_addr, uint32_t bar)
{
    mbar_expect_tx(bar, Math::STEP_BYTES * SS);
#pragma unroll
    for (int i = 0; i < Math::PIECES; ++i)
        bulk_g2s(slot_addr + Math::piece_off(i) * SS, s.base[i] + (size_t)g * (Math::piece_bytes(i) * SS),
                 Math::piece_bytes(i) * SS, bar);
}

// Context handed to the per-format math: where the activations are.
struct XCtx {
    uint32_t sx;   // shared address of the staged row (M = 1)
    int K, m0, M;
    XPtrs g;       // global buffers (M > 1)
};

// ------------------------------------------------------------------------------------------------ Q4_K
struct MathQ4K {
    static constexpr int STEP_ELEMS = 2048;
    static constexpr int PIECES = 1;
    static constexpr uint32_t STEP_BYTES = 1152;  // 8 blocks x 144 B
    static __host__ __device__ constexpr uint32_t piece_bytes(int) { return 1152; }
    static __host__ __device__ constexpr uint32_t piece_off(int) { return 0; }
    static constexpr bool SD = true, S16 = false;
    // a quarter warp reads chunks 16*b + 4*p + j (two blocks b, four p, fixed j)
    static __host__ __device__ __forceinline__ int swz(int c) { return c ^ ((c >> 3) & 7); }

    uint32_t blk_off, q_off;   // lane's block and qs bytes inside a slot
    uint32_t xo[4];            // swizzled byte offsets of the lane's four activation chunks inside a step
    uint32_t dx_off;           // byte offset of the lane's two block scales inside a step
    uint32_t selR, selT;       // PRMT selectors of the scale unpack
    bool low;
    int k_lane;                // element offset of the lane's unit inside a step

    __device__ __forceinline__ void init(int lane)
    {
        const int b = lane >> 2, p = lane & 3, pp = p & 1;
        blk_off = b * 144;
        q_off = blk_off + 16 + 32 * p;
        const int c = 16 * b + 4 * p;
#pragma unroll
        for (int j = 0; j < 4; ++j) xo[j] = 16 * swz(c + j);  // the permutation never crosses a 128-chunk step
        dx_off = (8 * b + 2 * p) * 4;
        selR = (2 * pp) | ((2 * pp + 1) << 4) | ((4 + 2 * pp) << 8) | ((5 + 2 * pp) << 12);
        selT = (2 * pp) | ((2 * pp + 1) << 4) | ((2 * pp) << 8) | ((2 * pp + 1) << 12);
        low = p < 2;
        k_lane = b * 256 + 64 * p;
    }

    template <int MT, bool XS, int SS>
    __device__ __forceinline__ void step(uint32_t slot, int i, int part, const XCtx &xc, float *acc) const
    {
        slot += i * 1152;
        const uint4 hdr = lds128(slot + blk_off), q0 = lds128(slot + q_off), q1 = lds128(slot + q_off + 16);
        // [sc(2p), sc(2p+1), mn(2p), mn(2p+1)] as four bytes (GetScaleMinK4_*): R holds scales[2pp..], scales[4+2pp..];
        // for sub-blocks >= 4 the low nibbles / high nibbles of T = scales[8+2pp..] are joined with the top two bits of R
        const uint32_t R = __byte_perm(hdr.y, hdr.z, selR);
        const uint32_t T = __byte_perm(hdr.w, hdr.w, selT);
        const uint32_t hi_form = (T & 0x00000F0Fu) | ((T >> 4) & 0x0F0F0000u) | ((R >> 2) & 0x30303030u);
        const uint32_t sm = low ? (R & 0x3F3F3F3Fu) : hi_form;
        const int sc_lo = sm & 0xFF, sc_hi = (sm >> 8) & 0xFF;
        const float mn_lo = (float)((sm >> 16) & 0xFF), mn_hi = (float)(sm >> 24);
        const float d = smc_h2f((uint16_t)(hdr.x & 0xFFFF));
        const float dmin = smc_h2f((uint16_t)(hdr.x >> 16));
        const uint32_t M4 = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
        const uint32_t l0 = q0.x & M4, l1 = q0.y & M4, l2 = q0.z & M4, l3 = q0.w & M4;
        const uint32_t l4 = q1.x & M4, l5 = q1.y & M4, l6 = q1.z & M4, l7 = q1.w & M4;
        const uint32_t h0 = q0.x & MH, h1 = q0.y & MH, h2 = q0.z & MH, h3 = q0.w & MH;
        const uint32_t h4 = q1.x & MH, h5 = q1.y & MH, h6 = q1.z & MH, h7 = q1.w & MH;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint4 a0, a1, c0, c1;
            float2 dx, sdx;
            if (XS) {
                const uint32_t xb = xc.sx + part * 2048;
                a0 = lds128(xb + xo[0]), a1 = lds128(xb + xo[1]), c0 = lds128(xb + xo[2]), c1 = lds128(xb + xo[3]);
                const uint32_t db = xc.sx + xc.K + part * 256 + dx_off;
                const uint2 t0 = lds64(db), t1 = lds64(db + (xc.K >> 3));
                dx = make_float2(__uint_as_float(t0.x), __uint_as_float(t0.y));
                sdx = make_float2(__uint_as_float(t1.x), __uint_as_float(t1.y));
            } else {
                const int mm = min(xc.m0 + m, xc.M - 1);
                const int k0 = part * 2048 + k_lane;
                const uint4 *xq = reinterpret_cast<const uint4 *>(xc.g.q + (size_t)mm * xc.K + k0);
                a0 = __ldg(xq), a1 = __ldg(xq + 1), c0 = __ldg(xq + 2), c1 = __ldg(xq + 3);
                const size_t b32 = (size_t)mm * (xc.K / 32) + (k0 >> 5);
                dx = __ldg(reinterpret_cast<const float2 *>(xc.g.d + b32));
                sdx = __ldg(reinterpret_cast<const float2 *>(xc.g.sd + b32));
            }
            int lo = smc_dp4a(l0, a0.x, 0), lo2 = smc_dp4a(l1, a0.y, 0);
            lo = smc_dp4a(l2, a0.z, lo), lo2 = smc_dp4a(l3, a0.w, lo2);
            lo = smc_dp4a(l4, a1.x, lo), lo2 = smc_dp4a(l5, a1.y, lo2);
            lo = smc_dp4a(l6, a1.z, lo), lo2 = smc_dp4a(l7, a1.w, lo2);
            int hi = smc_dp4a_us(h0, c0.x, 0), hi2 = smc_dp4a_us(h1, c0.y, 0);
            hi = smc_dp4a_us(h2, c0.z, hi), hi2 = smc_dp4a_us(h3, c0.w, hi2);
            hi = smc_dp4a_us(h4, c1.x, hi), hi2 = smc_dp4a_us(h5, c1.y, hi2);
            hi = smc_dp4a_us(h6, c1.z, hi), hi2 = smc_dp4a_us(h7, c1.w, hi2);
            lo += lo2;
            hi = (hi + hi2) >> 4;  // every term carried a factor 16: exact
            const float tsum = fmaf((float)(sc_lo * lo), dx.x, (float)(sc_hi * hi) * dx.y);
            const float msum = fmaf(mn_lo, sdx.x, mn_hi * sdx.y);
            acc[m] = fmaf(d, tsum, acc[m]);
            acc[m] = fmaf(-dmin, msum, acc[m]);
        }
    }
};

// ------------------------------------------------------------------------------------------------ Q6_K
struct MathQ6K {
    static constexpr int STEP_ELEMS = 2048;
    static constexpr int PIECES = 4;  // ql, qh, scales, d of 8 blocks
    static constexpr uint32_t STEP_BYTES = 1680;
    static __host__ __device__ constexpr uint32_t piece_bytes(int i) { return i == 0 ? 1024 : (i == 1 ? 512 : (i == 2 ? 128 : 16)); }
    static __host__ __device__ constexpr uint32_t piece_off(int i) { return i == 0 ? 0 : (i == 1 ? 1024 : (i == 2 ? 1536 : 1664)); }
    static constexpr bool SD = false, S16 = true;
    // a quarter warp reads chunks 16*b + 8*h + e + 2*cc (two b, two h, two e, fixed cc)
    static __host__ __device__ __forceinline__ int swz(int c) { return c ^ (((c >> 3) & 3) << 1); }

    uint32_t a_off, h_off, sc_off, d_off;
    uint32_t xo[4], dx_off, s16_off;
    int odd, ssel, k_half, l0;

    __device__ __forceinline__ void init(int lane)
    {
        const int b = lane >> 2, r = lane & 3, h = r >> 1;
        odd = r & 1;
        l0 = 16 * odd;
        a_off = b * 128 + 64 * h + l0;   // offsets inside each piece of one step
        h_off = b * 64 + 32 * h + l0;
        sc_off = b * 16 + 8 * h;
        d_off = 2 * b;
        const int c = 16 * b + 8 * h + odd;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) xo[cc] = 16 * swz(c + 2 * cc);
        dx_off = (8 * b + 4 * h) * 4;
        s16_off = (16 * b + 8 * h) * 2;
        ssel = odd ? 0 : 16;  // left shift that brings the wanted int16 of a pair to the top
        k_half = b * 256 + 128 * h;
    }

    template <int MT, bool XS, int SS>
    __device__ __forceinline__ void step(uint32_t slot, int i, int part, const XCtx &xc, float *acc) const
    {
        const uint32_t pa = slot + i * 1024 + a_off;
        const uint4 ua = lds128(pa), ub = lds128(pa + 32), uh = lds128(slot + SS * 1024 + i * 512 + h_off);
        const uint2 usc = lds64(slot + SS * 1536 + i * 128 + sc_off);
        const float d = smc_h2f((uint16_t)lds16u(slot + SS * 1664 + i * 16 + d_off));
        const uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x30303030u;
        const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wb[4] = {ub.x, ub.y, ub.z, ub.w}, wh[4] = {uh.x, uh.y, uh.z, uh.w};
        uint32_t q[4][4];  // [column c][word j]: six-bit codes of elements 32c + l0 + 4j .. +3
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            q[0][j] = (wa[j] & M4) | ((wh[j] << 4) & M2);
            q[1][j] = (wb[j] & M4) | ((wh[j] << 2) & M2);
            q[2][j] = ((wa[j] >> 4) & M4) | (wh[j] & M2);
            q[3][j] = ((wb[j] >> 4) & M4) | ((wh[j] >> 2) & M2);
        }
        // int8 scales is + {0, 2, 4, 6} with is = l0 / 16: bytes odd, odd+2, odd+4, odd+6 of the half's eight
        const uint32_t sw0 = odd ? (usc.x >> 8) : usc.x, sw1 = odd ? (usc.y >> 8) : usc.y;
        const int scl[4] = {(int)(int8_t)(sw0 & 0xFF), (int)(int8_t)((sw0 >> 16) & 0xFF), (int)(int8_t)(sw1 & 0xFF),
                            (int)(int8_t)((sw1 >> 16) & 0xFF)};
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint4 x[4], dxu, sw;
            if (XS) {
                const uint32_t xb = xc.sx + part * 2048;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) x[cc] = lds128(xb + xo[cc]);
                dxu = lds128(xc.sx + xc.K + part * 256 + dx_off);
                sw = lds128(xc.sx + xc.K + (xc.K >> 2) + part * 256 + s16_off);
            } else {
                const int mm = min(xc.m0 + m, xc.M - 1);
                const int kb = part * 2048 + k_half;
                const int8_t *xq = xc.g.q + (size_t)mm * xc.K + kb + l0;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) x[cc] = __ldg(reinterpret_cast<const uint4 *>(xq + 32 * cc));
                dxu = __ldg(reinterpret_cast<const uint4 *>(xc.g.d + (size_t)mm * (xc.K / 32) + (kb >> 5)));
                sw = __ldg(reinterpret_cast<const uint4 *>(xc.g.s16 + (size_t)mm * (xc.K / 16) + (kb >> 4)));
            }
            const uint32_t sws[4] = {sw.x, sw.y, sw.z, sw.w};
            const float dxs[4] = {__uint_as_float(dxu.x), __uint_as_float(dxu.y), __uint_as_float(dxu.z),
                                  __uint_as_float(dxu.w)};
            float rsum = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int s = smc_dp4a(q[c][0], x[c].x, 0), s2 = smc_dp4a(q[c][1], x[c].y, 0);
                s = smc_dp4a(q[c][2], x[c].z, s), s2 = smc_dp4a(q[c][3], x[c].w, s2);
                const int sxq = ((int)(sws[c] << ssel)) >> 16;  // sum of the 16 activation quants
                s = s + s2 - 32 * sxq;                           // sum (q - 32) x = sum q x - 32 sum x
                rsum = fmaf((float)(scl[c] * s), dxs[c], rsum);
            }
            acc[m] = fmaf(d, rsum, acc[m]);
        }
    }
};

// ------------------------------------------------------------------------------------------------ Q8_0
struct MathQ8_0 {
    static constexpr int STEP_ELEMS = 1024;
    static constexpr int PIECES = 2;  // 32 blocks of quants, their 32 fp16 scales
    static constexpr uint32_t STEP_BYTES = 1088;
    static __host__ __device__ constexpr uint32_t piece_bytes(int i) { return i == 0 ? 1024 : 64; }
    static __host__ __device__ constexpr uint32_t piece_off(int i) { return i == 0 ? 0 : 1024; }
    static constexpr bool SD = false, S16 = false;
    // lane l reads the two 16-byte halves of block l; lanes 0-3 of a quarter warp take half 0 first and
    // lanes 4-7 half 1 first, which already spreads eight reads over eight bank groups
    static __host__ __device__ __forceinline__ int swz(int c) { return c; }

    uint32_t qa_off, qb_off, d_off, dx_off;
    int sel, k_lane;
    __device__ __forceinline__ void init(int lane)
    {
        sel = (lane >> 2) & 1;
        qa_off = 32 * lane + 16 * sel;
        qb_off = 32 * lane + 16 * (1 - sel);
        d_off = 2 * lane;
        dx_off = 4 * lane;
        k_lane = 32 * lane;
    }
    template <int MT, bool XS, int SS>
    __device__ __forceinline__ void step(uint32_t slot, int i, int part, const XCtx &xc, float *acc) const
    {
        const uint4 q0 = lds128(slot + i * 1024 + qa_off), q1 = lds128(slot + i * 1024 + qb_off);
        const float d = smc_h2f((uint16_t)lds16u(slot + SS * 1024 + i * 64 + d_off));
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint4 a0, a1;
            float dx;
            if (XS) {
                const uint32_t xb = xc.sx + part * 1024;
                a0 = lds128(xb + qa_off), a1 = lds128(xb + qb_off);
                dx = __uint_as_float(lds32(xc.sx + xc.K + part * 128 + dx_off));
            } else {
                const int mm = min(xc.m0 + m, xc.M - 1);
                const int k0 = part * 1024 + k_lane;
                const uint4 *xq = reinterpret_cast<const uint4 *>(xc.g.q + (size_t)mm * xc.K + k0);
                a0 = __ldg(xq + sel), a1 = __ldg(xq + 1 - sel);
                dx = __ldg(xc.g.d + (size_t)mm * (xc.K / 32) + (k0 >> 5));
            }
            int s = smc_dp4a(q0.x, a0.x, 0), s2 = smc_dp4a(q0.y, a0.y, 0);
            s = smc_dp4a(q0.z, a0.z, s), s2 = smc_dp4a(q0.w, a0.w, s2);
            s = smc_dp4a(q1.x, a1.x, s), s2 = smc_dp4a(q1.y, a1.y, s2);
            s = smc_dp4a(q1.z, a1.z, s), s2 = smc_dp4a(q1.w, a1.w, s2);
            acc[m] = fmaf(d * dx, (float)(s + s2), acc[m]);
        }
    }
};

// ------------------------------------------------------------------------------------------------
// Work is handed out in "groups" of whole rows so that a row's partial sums never leave its warp:
// a stage is SS consecutive steps; when a row is shorter than a stage (spr <= SS) a group is SS/spr
// rows = one stage, otherwise a group is one row = spr/SS stages.  Warp w of W takes groups
// w, w + W, w + 2W, ...: at any moment the grid reads one dense window that slides through the matrix.
template <class Math, int MT, int MINB, int SS, bool GATHER>
__global__ void __launch_bounds__(256, MINB) gemv_tma_kernel(StepSrc src, XPtrs xg, float *__restrict__ out, int N, int K,
                                                             int M, int slots, int *__restrict__ status,
                                                             const smc_gather_dev *gd)
{
    extern __shared__ __align__(128) uint8_t smem[];
    int sending = -1;      // whether packets go out, known after the first look at the peers' ready flags (warp uniform)
    unsigned gtag = 0;     // number of the running exchange
    constexpr bool XS = (MT == 1);
    constexpr uint32_t SLOT = (Math::STEP_BYTES * SS + 127u) & ~127u;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m0 = blockIdx.y * MT;

    // shared layout: [x row (M = 1)] [8 warps x slots x SLOT bytes] [8 warps x slots barriers]
    const uint32_t xb = XS ? (uint32_t)((x_bytes(K) + 127) & ~(size_t)127) : 0u;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + xb + (uint32_t)(warp * slots) * SLOT;
    const uint32_t bars = sbase + xb + (uint32_t)(WARPS * slots) * SLOT + (uint32_t)(warp * slots) * 8u;

    const int spr = K / Math::STEP_ELEMS;            // steps per row
    const int rg = SS >= spr ? SS / spr : 1;         // rows per group
    const int spg = SS >= spr ? 1 : spr / SS;        // stages per group
    const int W = gridDim.x * WARPS, w = blockIdx.x * WARPS + warp;
    const int ngroups = N / rg;
    const int mine = w < ngroups ? (ngroups - w + W - 1) / W : 0;
    const int nstages = mine * spg;

    if (lane == 0) {
        for (int s = 0; s < slots; ++s) mbar_init(bars + 8 * s, 1);
        fence_barrier_init();
    }
    __syncwarp();
    // producer cursor (lane 0): global index of the next stage to fetch
    long long pstage = (long long)w * spg;
    int pin = 0, issued = 0;
    auto fetch_next = [&](uint32_t saddr, uint32_t bar) {
        issue_stage<Math, SS>(src, pstage, saddr, bar);
        ++issued;
        ++pstage;
        if (++pin == spg) {
            pin = 0;
            pstage += (long long)(W - 1) * spg;
        }
    };
    if (lane == 0) {
        const int pre = nstages < slots ? nstages : slots;
        for (int t = 0; t < pre; ++t) fetch_next(ring + (uint32_t)t * SLOT, bars + 8 * t);
    }
    // The weight stages requested above do not depend on earlier launches; everything below does (activations,
    // the output buffer, the exchange counters), so this is where a dependent launch waits for its predecessor.
    smc_grid_dep_sync();
    // row-split across GPUs (one row only): tell the peers that this rank's readers of the previous exchange are done
    if (GATHER && blockIdx.x == 0 && threadIdx.x == 32) smc_gather_post_ready(gd);
    if (XS) {
        if (xg.nw) stage_x_addnorm_quant<Math>(xg.xf, xg.xadd, xg.nw, xg.eps, blockIdx.x == 0 ? xg.xsum : nullptr, K, smem);
        else if (xg.xf) stage_x_quant<Math>(xg.xf, xg.xu, K, smem);
        else stage_x<Math>(xg, m0, K, smem);
        __syncthreads();
    }

    Math math;
    math.init(lane);
    XCtx xc{sbase, K, m0, M, xg};
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;

    int slot = 0, part = 0, row = w * rg, cin = 0;
    uint32_t phase = 0;
    for (int t = 0; t < nstages; ++t) {
        const uint32_t bar = bars + 8 * slot;
        const uint32_t saddr = ring + (uint32_t)slot * SLOT;
        if (!mbar_wait(bar, phase)) {
            if (lane == 0) atomicExch(status, 1);
            break;
        }
#pragma unroll
        for (int i = 0; i < SS; ++i) {
            math.template step<MT, XS, SS>(saddr, i, part, xc, acc);
            if (++part == spr) {
                if (XS && GATHER && sending < 0) {  // first finished row of this warp: the peers' ready flags, one lane each
                    gtag = smc_gather_tag(gd);
                    sending = smc_gather_wait_ready_warp(gd, gtag) ? 1 : 0;
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const float v = warp_sum32(acc[m]);  // every lane holds the sum
                    if (lane == 0 && m0 + m < M) out[(size_t)(m0 + m) * N + row] = v;
                    // this rank's chunk starts at rank * N in every peer's buffer; lane p sends to peer p
                    if (XS && GATHER && sending) smc_gather_send_warp(gd, (size_t)N, (size_t)row, v, gtag);
                    acc[m] = 0.f;
                }
                part = 0;
                ++row;
            }
        }
        __syncwarp();  // every lane has read the slot: it may be refilled
        if (lane == 0 && issued < nstages) fetch_next(saddr, bar);
        if (++slot == slots) {
            slot = 0;
            phase ^= 1;
        }
        if (++cin == spg) {
            cin = 0;
            row += (W - 1) * rg;
        }
    }
    // rows done: unpack this CTA's stripe of the peers' slices as they arrive
    if (GATHER) {
        smc_gather_collect(gd, (size_t)N, blockIdx.x, gridDim.x, smc_gather_tag(gd));
        smc_gather_done(gd, gridDim.x);
    }
}

struct Tuning {
    int slots = 2;        // ring depth per warp, in stages (measured best: 2 x 2 steps, 3 CTAs per SM)
    int ctas_per_sm = 3;  // resident CTAs the grid is sized for (M = 1)
    int ss = 2;           // steps per stage (M = 1): 1, 2 or 4
};

Tuning tuning()
{
    static Tuning t = [] {
        Tuning v;
        if (const char *e = getenv("SMC_TMA_SLOTS")) v.slots = atoi(e) > 1 ? atoi(e) : v.slots;
        if (const char *e = getenv("SMC_TMA_CTAS")) v.ctas_per_sm = atoi(e) > 0 ? atoi(e) : v.ctas_per_sm;
        if (const char *e = getenv("SMC_TMA_SS")) v.ss = atoi(e) > 0 ? atoi(e) : v.ss;
        return v;
    }();
    return t;
}

template <class Math, int MT, int MINB, int SS>
void launch_one(smc_ctx *ctx, dim3 grid, size_t smem, cudaStream_t s, const StepSrc &src, const XPtrs &x, float *out, int N,
                int K, int M, int slots, const smc_gather_dev *gd)
{
    if (MT == 1 && gd) {
        cudaFuncSetAttribute(gemv_tma_kernel<Math, MT, MINB, SS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        smc_launch_dep(ctx->use_pdl, gemv_tma_kernel<Math, MT, MINB, SS, true>, grid, dim3(256), smem, s, src, x, out, N, K, M, slots,
                       ctx->d_status, gd);
        return;
    }
    cudaFuncSetAttribute(gemv_tma_kernel<Math, MT, MINB, SS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    smc_launch_dep(ctx->use_pdl, gemv_tma_kernel<Math, MT, MINB, SS, false>, grid, dim3(256), smem, s, src, x, out, N, K, M, slots,
                   ctx->d_status, (const smc_gather_dev *)nullptr);
}

template <class Math>
int launch_math(smc_ctx *ctx, const StepSrc &src, const XPtrs &x, float *out, int N, int K, int M, cudaStream_t s,
                const smc_gather_dev *gd)
{
    const Tuning tn = tuning();
    const int mt = M == 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
    const int spr = K / Math::STEP_ELEMS;
    // steps per stage: the largest of 4, 2, 1 allowed by the tuning that tiles rows exactly
    int ss = 1;
    if (mt == 1)
        for (int c = 4; c >= 2; c >>= 1) {
            if (c > tn.ss) continue;
            const bool tiles = (c >= spr) ? (c % spr == 0 && N % (c / spr) == 0) : (spr % c == 0);
            if (tiles) {
                ss = c;
                break;
            }
        }
    const size_t xb = mt == 1 ? ((x_bytes(K) + 127) & ~(size_t)127) : 0;
    const size_t slot_bytes = ((size_t)Math::STEP_BYTES * ss + 127) & ~(size_t)127;
    int per_sm = mt == 1 ? tn.ctas_per_sm : 2;
    int slots = tn.slots;
    // `per_sm` CTAs must fit in the 227 KB of an SM (1 KB per CTA is reserved by the system)
    auto need = [&](int sl) { return xb + (size_t)WARPS * sl * (slot_bytes + 8); };
    while (per_sm > 1 && (need(slots) + 1024) * per_sm > 227 * 1024) {
        if (slots > 3) --slots;
        else --per_sm;
    }
    const size_t smem = need(slots);
    if (smem > 226 * 1024) return smc_fail(ctx, SMC_E_UNSUPPORTED, "K = %d needs %zu bytes of shared memory", K, smem);
    const int rg = ss >= spr ? ss / spr : 1;
    const int ngroups = N / rg;
    int warps = ctx->sm_count * per_sm * WARPS;
    if (warps > ngroups) warps = ngroups;
    dim3 grid((warps + WARPS - 1) / WARPS, (M + mt - 1) / mt);
    if (mt == 1) {
        const bool three = per_sm >= 3;
        if (ss == 4) three ? launch_one<Math, 1, 3, 4>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd)
                           : launch_one<Math, 1, 2, 4>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd);
        else if (ss == 2) three ? launch_one<Math, 1, 3, 2>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd)
                                : launch_one<Math, 1, 2, 2>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd);
        else three ? launch_one<Math, 1, 3, 1>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd)
                   : launch_one<Math, 1, 2, 1>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd);
    } else if (mt == 2) {
        launch_one<Math, 2, 2, 1>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd);
    } else if (mt == 4) {
        launch_one<Math, 4, 2, 1>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd);
    } else {
        launch_one<Math, 8, 2, 1>(ctx, grid, smem, s, src, x, out, N, K, M, slots, gd);
    }
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

}  // namespace

bool smc_tma_supported(const smc_weight *w, int M)
{
    if (!w->fast || M < 1) return false;
    if (w->dtype == SMC_Q8_0) return w->K % 1024 == 0 && w->K <= 65536;
    return w->K % 2048 == 0 && w->K <= 65536;
}

// M = 1 with fp32 input: the row is quantised inside the kernel, no scratch buffer is involved.
int smc_launch_gemv_tma_f32in(smc_ctx *ctx, const float *x, const smc_weight *w, float *out, cudaStream_t s)
{
    smc_q8act one{};
    one.M = 1, one.K = w->K;
    return smc_launch_gemv_tma_x(ctx, &one, x, w, out, s);
}

int smc_launch_gemv_tma(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s)
{
    return smc_launch_gemv_tma_x(ctx, a, nullptr, w, out, s);
}

int smc_launch_gemv_tma_x(smc_ctx *ctx, const smc_q8act *a, const float *xf, const smc_weight *w, float *out,
                          cudaStream_t s)
{
    return smc_launch_gemv_tma_xg(ctx, a, xf, w, out, nullptr, s);
}

// One fp32 row, quantised in the kernel, whose output slice is exchanged with the peers in the kernel's tail.
int smc_launch_gemv_tma_gather(smc_ctx *ctx, const float *x, const smc_weight *w, float *out, const smc_gather_dev *gd,
                               cudaStream_t s)
{
    smc_q8act one{};
    one.M = 1, one.K = w->K;
    return smc_launch_gemv_tma_xg(ctx, &one, x, w, out, gd, s);
}

// One row whose activation is SiLU(gate) * up, formed and quantised while the row is staged.
int smc_launch_gemv_tma_swiglu(smc_ctx *ctx, const float *gate, const float *up, const smc_weight *w, float *out, cudaStream_t s)
{
    smc_q8act one{};
    one.M = 1, one.K = w->K;
    return smc_launch_gemv_tma_xgu(ctx, &one, gate, up, w, out, nullptr, s);
}

int smc_launch_gemv_tma_xg(smc_ctx *ctx, const smc_q8act *a, const float *xf, const smc_weight *w, float *out,
                           const smc_gather_dev *gd, cudaStream_t s)
{
    return smc_launch_gemv_tma_xgu(ctx, a, xf, nullptr, w, out, gd, s);
}

// One row that is RMSNorm(x + add) * w, formed and quantised while the row is staged; x + add goes to `sum`.
int smc_launch_gemv_tma_addnorm(smc_ctx *ctx, const float *x, const smc_norm_prologue *pro, const smc_weight *w, float *out,
                                cudaStream_t s)
{
    smc_q8act one{};
    one.M = 1, one.K = w->K;
    return smc_launch_gemv_tma_full(ctx, &one, x, nullptr, pro, w, out, nullptr, s);
}

int smc_launch_gemv_tma_xgu(smc_ctx *ctx, const smc_q8act *a, const float *xf, const float *xu, const smc_weight *w, float *out,
                            const smc_gather_dev *gd, cudaStream_t s)
{
    return smc_launch_gemv_tma_full(ctx, a, xf, xu, nullptr, w, out, gd, s);
}

int smc_launch_gemv_tma_full(smc_ctx *ctx, const smc_q8act *a, const float *xf, const float *xu, const smc_norm_prologue *pro,
                             const smc_weight *w, float *out, const smc_gather_dev *gd, cudaStream_t s)
{
    const int N = w->N, K = w->K, M = a->M;
    XPtrs x{a->q, a->d, a->sd, a->s16, xf, xu, nullptr, nullptr, nullptr, 0.f};
    if (pro) x.xadd = pro->add, x.nw = pro->w, x.xsum = pro->sum, x.eps = pro->eps;
    StepSrc src{};
    if (w->dtype == SMC_Q4_K) {
        src.base[0] = w->d_raw;
        return launch_math<MathQ4K>(ctx, src, x, out, N, K, M, s, gd);
    }
    if (w->dtype == SMC_Q6_K) {
        src.base[0] = w->q6_ql;
        src.base[1] = w->q6_qh;
        src.base[2] = reinterpret_cast<const uint8_t *>(w->q6_sc);
        src.base[3] = reinterpret_cast<const uint8_t *>(w->q6_d);
        return launch_math<MathQ6K>(ctx, src, x, out, N, K, M, s, gd);
    }
    src.base[0] = reinterpret_cast<const uint8_t *>(w->q8_qs);
    src.base[1] = reinterpret_cast<const uint8_t *>(w->q8_d);
    return launch_math<MathQ8_0>(ctx, src, x, out, N, K, M, s, gd);
}
