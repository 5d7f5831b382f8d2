// TMA-staged streaming GEMV for Q8_0-quantised activations, the decode hot kernel.
//
// Each warp owns a contiguous range of weight rows, i.e. one contiguous byte stream per weight
// array, and consumes it in "steps" of 32 lane-units (Q4_K / Q6_K: 8 blocks = 2048 elements,
// Q8_0: 32 blocks = 1024 elements).  The bytes of a step are brought into a warp-private ring of
// shared-memory slots by bulk asynchronous copies (cp.async.bulk global -> shared, completion on an
// mbarrier) issued by one lane, up to `slots` steps ahead of the math:
//   * memory-level parallelism is set by shared memory, not by registers (8 slots x 8 warps x
//     2 CTAs keeps more than 100 KB per SM in flight, against the ~45 KB Little's law asks for);
//   * HBM and L2 see whole contiguous ranges, never half-used sectors;
//   * the lanes read their unit with conflict-free 128-bit shared loads, and the activation row is
//     also in shared memory (XOR-swizzled in 16-byte chunks so that the strided reads of eight
//     lanes fall in eight different bank groups), so the inner loop issues no global loads at all.
// A slot is re-armed only after __syncwarp(): every lane has passed its wait and read its data, so
// no lane can be left waiting on a phase that has already been reused.  Every wait is bounded; on
// expiry the warp raises a flag in device memory (read back by smc_device_status) and stops.
//
// Arithmetic is identical to the other SMC_ACT_Q8 kernels: exact int32 block dots (dp4a), one fp32
// multiply-add per 32-element block.  Shapes: K % 2048 == 0 (K-quants) / K % 1024 == 0 (Q8_0).
// References as in smc_gemv.cu.
#include "smc_common.cuh"

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
};

// Shared layout of the staged activation row: q | d | sd | s16.  The quants are stored in 16-byte
// chunks permuted by Math::swz so that the 128-bit reads of a quarter warp (eight lanes, each format
// with its own stride pattern) fall in eight different bank groups.
template <class Math>
__device__ __forceinline__ void stage_x(const XPtrs &g, int m, int K, uint8_t *sx, bool want_sd, bool want_s16)
{
    uint4 *sq = reinterpret_cast<uint4 *>(sx);
    float *sdx = reinterpret_cast<float *>(sx + K);
    float *ssd = sdx + K / 32;
    int16_t *ss16 = reinterpret_cast<int16_t *>(ssd + K / 32);
    const uint4 *gq = reinterpret_cast<const uint4 *>(g.q + (size_t)m * K);
    for (int i = threadIdx.x; i < K / 16; i += blockDim.x) sq[Math::swz(i)] = __ldg(gq + i);
    for (int i = threadIdx.x; i < K / 32; i += blockDim.x) {
        sdx[i] = __ldg(g.d + (size_t)m * (K / 32) + i);
        if (want_sd) ssd[i] = __ldg(g.sd + (size_t)m * (K / 32) + i);
    }
    if (want_s16)
        for (int i = threadIdx.x; i < K / 16; i += blockDim.x) ss16[i] = __ldg(g.s16 + (size_t)m * (K / 16) + i);
}
__host__ __device__ inline size_t x_bytes(int K) { return (size_t)K + (size_t)(K / 32) * 8 + (size_t)(K / 16) * 2; }

__device__ __forceinline__ uint4 lds16(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }

__device__ __forceinline__ void warp_rows(int N, int &r0, int &r1)
{
    const long long W = (long long)gridDim.x * WARPS;
    const long long w = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
    r0 = (int)((long long)N * w / W);
    r1 = (int)((long long)N * (w + 1) / W);
}

// Description of how one step of a format is fetched: up to four contiguous pieces.
struct StepSrc {
    const uint8_t *base[4];  // address of this warp's first step in each weight array
    uint32_t bytes[4];       // bytes per step in each array (multiples of 16)
    uint32_t off[4];         // offset of each piece inside a slot
    int pieces;
    uint32_t total;
};

__device__ __forceinline__ void issue_step(const StepSrc &s, int t, uint32_t slot_addr, uint32_t bar)
{
    mbar_expect_tx(bar, s.total);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (i < s.pieces) bulk_g2s(slot_addr + s.off[i], s.base[i] + (size_t)t * s.bytes[i], s.bytes[i], bar);
}

// ------------------------------------------------------------------------------------------------
// Format-specific math on one unit held in a shared-memory slot.
// ------------------------------------------------------------------------------------------------
struct MathQ4K {
    static constexpr int STEP_ELEMS = 2048;
    static constexpr uint32_t SLOT = 1152;  // 8 blocks x 144 B
    static constexpr bool SD = true, S16 = false;
    // a quarter warp reads chunks 16*b + 4*p + j (two blocks b, four p, fixed j)
    static __device__ __forceinline__ int swz(int c) { return c ^ ((c >> 3) & 7); }
    int b, p, sh;
    bool low;
    __device__ __forceinline__ void init(int lane)
    {
        b = lane >> 2, p = lane & 3;
        sh = (p & 1) * 16;
        low = p < 2;
    }
    template <int MT, bool XS>
    __device__ __forceinline__ void step(const uint8_t *slot, int part, const XPtrs &xs, const uint8_t *sx, int K, int m0,
                                         int M, float *acc) const
    {
        const uint8_t *blk = slot + b * 144;
        const uint4 hdr = lds16(blk), q0 = lds16(blk + 16 + 32 * p), q1 = lds16(blk + 32 + 32 * p);
        // scales / mins of sub-blocks 2p (low byte) and 2p+1 (high byte): GetScaleMinK4_* on 16-bit pairs
        const uint32_t s0 = hdr.y, s1 = hdr.z, s2 = hdr.w;
        const uint32_t hp = ((low ? s0 : s1) >> sh) & 0xFFFFu;
        const uint32_t hp2 = ((low ? s1 : s2) >> sh) & 0xFFFFu;
        const uint32_t hm2 = (s0 >> sh) & 0xFFFFu;
        const uint32_t sc = low ? (hp & 0x3F3Fu) : ((hp2 & 0x0F0Fu) | ((hm2 >> 2) & 0x3030u));
        const uint32_t mn = low ? (hp2 & 0x3F3Fu) : (((hp2 >> 4) & 0x0F0Fu) | ((hp >> 2) & 0x3030u));
        const int sc_lo = sc & 0xFF, sc_hi = sc >> 8;
        const float mn_lo = (float)(mn & 0xFF), mn_hi = (float)(mn >> 8);
        const float d = smc_h2f((uint16_t)(hdr.x & 0xFFFF));
        const float dmin = smc_h2f((uint16_t)(hdr.x >> 16));
        const uint32_t M4 = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
        const int k0 = part * 2048 + b * 256 + 64 * p;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint4 a0, a1, c0, c1;
            float2 dx, sdx;
            if (XS) {
                const int c = k0 >> 4;
                a0 = lds16(sx + 16 * swz(c)), a1 = lds16(sx + 16 * swz(c + 1));
                c0 = lds16(sx + 16 * swz(c + 2)), c1 = lds16(sx + 16 * swz(c + 3));
                const float *fd = reinterpret_cast<const float *>(sx + K);
                dx = *reinterpret_cast<const float2 *>(fd + (k0 >> 5));
                sdx = *reinterpret_cast<const float2 *>(fd + K / 32 + (k0 >> 5));
            } else {
                const int mm = min(m0 + m, M - 1);
                const uint4 *xq = reinterpret_cast<const uint4 *>(xs.q + (size_t)mm * K + k0);
                a0 = __ldg(xq), a1 = __ldg(xq + 1), c0 = __ldg(xq + 2), c1 = __ldg(xq + 3);
                const size_t b32 = (size_t)mm * (K / 32) + (k0 >> 5);
                dx = __ldg(reinterpret_cast<const float2 *>(xs.d + b32));
                sdx = __ldg(reinterpret_cast<const float2 *>(xs.sd + b32));
            }
            int lo = smc_dp4a(q0.x & M4, a0.x, 0);
            lo = smc_dp4a(q0.y & M4, a0.y, lo);
            lo = smc_dp4a(q0.z & M4, a0.z, lo);
            lo = smc_dp4a(q0.w & M4, a0.w, lo);
            lo = smc_dp4a(q1.x & M4, a1.x, lo);
            lo = smc_dp4a(q1.y & M4, a1.y, lo);
            lo = smc_dp4a(q1.z & M4, a1.z, lo);
            lo = smc_dp4a(q1.w & M4, a1.w, lo);
            int hi = smc_dp4a_us(q0.x & MH, c0.x, 0);
            hi = smc_dp4a_us(q0.y & MH, c0.y, hi);
            hi = smc_dp4a_us(q0.z & MH, c0.z, hi);
            hi = smc_dp4a_us(q0.w & MH, c0.w, hi);
            hi = smc_dp4a_us(q1.x & MH, c1.x, hi);
            hi = smc_dp4a_us(q1.y & MH, c1.y, hi);
            hi = smc_dp4a_us(q1.z & MH, c1.z, hi);
            hi = smc_dp4a_us(q1.w & MH, c1.w, hi);
            hi >>= 4;  // every term carried a factor 16: exact
            const float tsum = fmaf((float)(sc_lo * lo), dx.x, (float)(sc_hi * hi) * dx.y);
            const float msum = fmaf(mn_lo, sdx.x, mn_hi * sdx.y);
            acc[m] = fmaf(d, tsum, acc[m]);
            acc[m] = fmaf(-dmin, msum, acc[m]);
        }
    }
};

struct MathQ6K {
    static constexpr int STEP_ELEMS = 2048;
    static constexpr uint32_t OFF_QH = 1024, OFF_SC = 1536, OFF_D = 1664, SLOT = 1792;
    static constexpr bool SD = false, S16 = true;
    // a quarter warp reads chunks 16*b + 8*h + e + 2*cc (two b, two h, two e, fixed cc)
    static __device__ __forceinline__ int swz(int c) { return c ^ (((c >> 3) & 3) << 1); }
    int b, r, h, l0, ssel;
    __device__ __forceinline__ void init(int lane)
    {
        b = lane >> 2, r = lane & 3, h = r >> 1, l0 = 16 * (r & 1);
        ssel = (r & 1) ? 0 : 16;
    }
    template <int MT, bool XS>
    __device__ __forceinline__ void step(const uint8_t *slot, int part, const XPtrs &xs, const uint8_t *sx, int K, int m0,
                                         int M, float *acc) const
    {
        const uint4 ua = lds16(slot + b * 128 + 64 * h + l0), ub = lds16(slot + b * 128 + 64 * h + 32 + l0);
        const uint4 uh = lds16(slot + OFF_QH + b * 64 + 32 * h + l0);
        const uint2 usc = *reinterpret_cast<const uint2 *>(slot + OFF_SC + b * 16 + 8 * h);
        const float d = smc_h2f(*reinterpret_cast<const uint16_t *>(slot + OFF_D + 2 * b));
        const uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x30303030u;
        const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wb[4] = {ub.x, ub.y, ub.z, ub.w}, wh[4] = {uh.x, uh.y, uh.z, uh.w};
        uint32_t q[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            q[0][j] = (wa[j] & M4) | ((wh[j] << 4) & M2);
            q[1][j] = (wb[j] & M4) | ((wh[j] << 2) & M2);
            q[2][j] = ((wa[j] >> 4) & M4) | (wh[j] & M2);
            q[3][j] = ((wb[j] >> 4) & M4) | ((wh[j] >> 2) & M2);
        }
        const uint32_t sw0 = (r & 1) ? (usc.x >> 8) : usc.x, sw1 = (r & 1) ? (usc.y >> 8) : usc.y;
        const int scl[4] = {(int)(int8_t)(sw0 & 0xFF), (int)(int8_t)((sw0 >> 16) & 0xFF), (int)(int8_t)(sw1 & 0xFF),
                            (int)(int8_t)((sw1 >> 16) & 0xFF)};
        const int kb = part * 2048 + b * 256 + 128 * h;  // start of the 128-half; this lane adds l0
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float4 dx;
            uint4 sw, x[4];
            if (XS) {
                const int c = (kb + l0) >> 4;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) x[cc] = lds16(sx + 16 * swz(c + 2 * cc));
                const float *fd = reinterpret_cast<const float *>(sx + K);
                dx = *reinterpret_cast<const float4 *>(fd + (kb >> 5));
                const int16_t *s16 = reinterpret_cast<const int16_t *>(fd + 2 * (K / 32));
                sw = *reinterpret_cast<const uint4 *>(s16 + (kb >> 4));
            } else {
                const int mm = min(m0 + m, M - 1);
                const int8_t *xq = xs.q + (size_t)mm * K + kb + l0;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) x[cc] = __ldg(reinterpret_cast<const uint4 *>(xq + 32 * cc));
                dx = __ldg(reinterpret_cast<const float4 *>(xs.d + (size_t)mm * (K / 32) + (kb >> 5)));
                sw = __ldg(reinterpret_cast<const uint4 *>(xs.s16 + (size_t)mm * (K / 16) + (kb >> 4)));
            }
            const uint32_t sws[4] = {sw.x, sw.y, sw.z, sw.w};
            const float dxs[4] = {dx.x, dx.y, dx.z, dx.w};
            float rsum = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int s = smc_dp4a(q[c][0], x[c].x, 0);
                s = smc_dp4a(q[c][1], x[c].y, s);
                s = smc_dp4a(q[c][2], x[c].z, s);
                s = smc_dp4a(q[c][3], x[c].w, s);
                const int sxq = ((int)(sws[c] << ssel)) >> 16;  // sum of the 16 activation quants
                s -= 32 * sxq;                                   // sum (q - 32) x = sum q x - 32 sum x
                rsum = fmaf((float)(scl[c] * s), dxs[c], rsum);
            }
            acc[m] = fmaf(d, rsum, acc[m]);
        }
    }
};

struct MathQ8_0 {
    static constexpr int STEP_ELEMS = 1024;
    static constexpr uint32_t OFF_D = 1024, SLOT = 1152;  // 1024 quants + 32 fp16 scales, padded
    static constexpr bool SD = false, S16 = false;
    // lane l reads the two 16-byte halves of block l; lanes 0-3 of a quarter warp take half 0 first and
    // lanes 4-7 half 1 first, which already spreads eight reads over eight bank groups
    static __device__ __forceinline__ int swz(int c) { return c; }
    int lane_, sel_;
    __device__ __forceinline__ void init(int lane) { lane_ = lane, sel_ = (lane >> 2) & 1; }
    template <int MT, bool XS>
    __device__ __forceinline__ void step(const uint8_t *slot, int part, const XPtrs &xs, const uint8_t *sx, int K, int m0,
                                         int M, float *acc) const
    {
        const int blk = lane_;
        const uint4 q0 = lds16(slot + 32 * blk + 16 * sel_), q1 = lds16(slot + 32 * blk + 16 * (1 - sel_));
        const float d = smc_h2f(*reinterpret_cast<const uint16_t *>(slot + OFF_D + 2 * blk));
        const int k0 = part * 1024 + 32 * blk;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            uint4 a0, a1;
            float dx;
            if (XS) {
                const int c = k0 >> 4;
                a0 = lds16(sx + 16 * (c + sel_)), a1 = lds16(sx + 16 * (c + 1 - sel_));
                dx = reinterpret_cast<const float *>(sx + K)[k0 >> 5];
            } else {
                const int mm = min(m0 + m, M - 1);
                const uint4 *xq = reinterpret_cast<const uint4 *>(xs.q + (size_t)mm * K + k0);
                a0 = __ldg(xq + sel_), a1 = __ldg(xq + 1 - sel_);
                dx = __ldg(xs.d + (size_t)mm * (K / 32) + (k0 >> 5));
            }
            int s = smc_dp4a(q0.x, a0.x, 0);
            s = smc_dp4a(q0.y, a0.y, s);
            s = smc_dp4a(q0.z, a0.z, s);
            s = smc_dp4a(q0.w, a0.w, s);
            s = smc_dp4a(q1.x, a1.x, s);
            s = smc_dp4a(q1.y, a1.y, s);
            s = smc_dp4a(q1.z, a1.z, s);
            s = smc_dp4a(q1.w, a1.w, s);
            acc[m] = fmaf(d * dx, (float)s, acc[m]);
        }
    }
};

// ------------------------------------------------------------------------------------------------
template <class Math, int MT>
__global__ void __launch_bounds__(256, 2) gemv_tma_kernel(StepSrc src_rows, size_t row_stride0, size_t row_stride1,
                                                          size_t row_stride2, size_t row_stride3, XPtrs xg,
                                                          float *__restrict__ out, int N, int K, int M, int slots,
                                                          int *__restrict__ status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr bool XS = (MT == 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m0 = blockIdx.y * MT;

    // shared layout: [x row (MT == 1)] [8 warps x slots x SLOT bytes] [8 warps x slots barriers]
    const size_t xb = XS ? ((x_bytes(K) + 127) & ~(size_t)127) : 0;
    uint8_t *ring = smem + xb + (size_t)warp * slots * Math::SLOT;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + xb + (size_t)WARPS * slots * Math::SLOT) + warp * slots;

    int r0, r1;
    warp_rows(N, r0, r1);
    const int spr = K / Math::STEP_ELEMS;
    const int nsteps = (r1 - r0) * spr;

    StepSrc src = src_rows;
    src.base[0] += (size_t)r0 * row_stride0;
    src.base[1] += (size_t)r0 * row_stride1;
    src.base[2] += (size_t)r0 * row_stride2;
    src.base[3] += (size_t)r0 * row_stride3;

    if (lane == 0) {
        for (int s = 0; s < slots; ++s) mbar_init(smem_u32(bars + s), 1);
        fence_barrier_init();
    }
    __syncwarp();
    if (lane == 0) {
        const int pre = nsteps < slots ? nsteps : slots;
        for (int t = 0; t < pre; ++t) issue_step(src, t, smem_u32(ring + (size_t)t * Math::SLOT), smem_u32(bars + t));
    }
    if (XS) {
        stage_x<Math>(xg, m0, K, smem, Math::SD, Math::S16);
        __syncthreads();
    }

    Math math;
    math.init(lane);
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;

    int slot = 0, part = 0, row = r0;
    uint32_t phase = 0;
    for (int t = 0; t < nsteps; ++t) {
        const uint32_t bar = smem_u32(bars + slot);
        if (!mbar_wait(bar, phase)) {
            if (lane == 0) atomicExch(status, 1);
            return;
        }
        math.template step<MT, XS>(ring + (size_t)slot * Math::SLOT, part, xg, smem, K, m0, M, acc);
        __syncwarp();  // every lane has read the slot: it may be refilled
        if (lane == 0 && t + slots < nsteps) issue_step(src, t + slots, smem_u32(ring + (size_t)slot * Math::SLOT), bar);
        if (++slot == slots) {
            slot = 0;
            phase ^= 1;
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

int tma_ctas(const smc_ctx *ctx, int N)
{
    const int wmax = ctx->sm_count * 2 * WARPS;
    int rpw = (N + wmax - 1) / wmax;
    if (rpw < 1) rpw = 1;
    int warps = (N + rpw - 1) / rpw;
    int ctas = (warps + WARPS - 1) / WARPS;
    return ctas < 1 ? 1 : ctas;
}

template <class Math>
int launch_math(smc_ctx *ctx, const StepSrc &src, const size_t *row_stride, const XPtrs &x, float *out, int N, int K,
                int M, cudaStream_t s)
{
    const int mt = M == 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
    const size_t xb = mt == 1 ? ((x_bytes(K) + 127) & ~(size_t)127) : 0;
    // two CTAs per SM must fit: ~113 KB each
    const size_t budget = 112 * 1024;
    int slots = 8;
    while (slots > 2 && xb + (size_t)WARPS * slots * (Math::SLOT + 8) > budget) --slots;
    const size_t smem = xb + (size_t)WARPS * slots * (Math::SLOT + 8);
    if (smem > 220 * 1024) return smc_fail(ctx, SMC_E_UNSUPPORTED, "K = %d needs %zu bytes of shared memory", K, smem);
    dim3 grid(tma_ctas(ctx, N), (M + mt - 1) / mt);
#define SMC_TMA_LAUNCH(MTV)                                                                                          \
    do {                                                                                                             \
        cudaFuncSetAttribute(gemv_tma_kernel<Math, MTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        gemv_tma_kernel<Math, MTV><<<grid, 256, smem, s>>>(src, row_stride[0], row_stride[1], row_stride[2],         \
                                                           row_stride[3], x, out, N, K, M, slots, ctx->d_status);    \
    } while (0)
    switch (mt) {
    case 1: SMC_TMA_LAUNCH(1); break;
    case 2: SMC_TMA_LAUNCH(2); break;
    case 4: SMC_TMA_LAUNCH(4); break;
    default: SMC_TMA_LAUNCH(8); break;
    }
#undef SMC_TMA_LAUNCH
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

int smc_launch_gemv_tma(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s)
{
    const int N = w->N, K = w->K, M = a->M;
    XPtrs x{a->q, a->d, a->sd, a->s16};
    StepSrc src{};
    size_t rs[4] = {0, 0, 0, 0};
    if (w->dtype == SMC_Q4_K) {
        src.pieces = 1;
        src.base[0] = w->d_raw, src.bytes[0] = 1152, src.off[0] = 0, src.total = 1152;
        rs[0] = (size_t)(K / 256) * 144;
        return launch_math<MathQ4K>(ctx, src, rs, x, out, N, K, M, s);
    }
    if (w->dtype == SMC_Q6_K) {
        src.pieces = 4;
        src.base[0] = w->q6_ql, src.bytes[0] = 1024, src.off[0] = 0;
        src.base[1] = w->q6_qh, src.bytes[1] = 512, src.off[1] = MathQ6K::OFF_QH;
        src.base[2] = reinterpret_cast<const uint8_t *>(w->q6_sc), src.bytes[2] = 128, src.off[2] = MathQ6K::OFF_SC;
        src.base[3] = reinterpret_cast<const uint8_t *>(w->q6_d), src.bytes[3] = 16, src.off[3] = MathQ6K::OFF_D;
        src.total = 1680;
        const size_t nb = K / 256;
        rs[0] = nb * 128, rs[1] = nb * 64, rs[2] = nb * 16, rs[3] = nb * 2;
        return launch_math<MathQ6K>(ctx, src, rs, x, out, N, K, M, s);
    }
    src.pieces = 2;
    src.base[0] = reinterpret_cast<const uint8_t *>(w->q8_qs), src.bytes[0] = 1024, src.off[0] = 0;
    src.base[1] = reinterpret_cast<const uint8_t *>(w->q8_d), src.bytes[1] = 64, src.off[1] = MathQ8_0::OFF_D;
    src.total = 1088;
    rs[0] = (size_t)K, rs[1] = (size_t)(K / 32) * 2;
    return launch_math<MathQ8_0>(ctx, src, rs, x, out, N, K, M, s);
}
