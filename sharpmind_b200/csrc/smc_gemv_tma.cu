// Bulk-copy (TMA) staged streaming GEMV for one activation row: the decode hot kernel.
//
// Work split.  The weight bytes of a matrix are a flat stream of "steps" of 32 lane-units (Q4_K / Q6_K: 8 blocks =
// 2048 elements, Q8_0: 32 blocks = 1024 elements; a row is K / STEP_ELEMS steps).  A CTA owns a contiguous range
// of whole rows (rows are dealt out evenly, the first N % grid CTAs take one more), and its warps cut the CTA's
// steps into equal contiguous pieces WITHOUT regard to row boundaries, so every warp of the grid streams the same
// number of bytes (+-1 step) whatever N and K are: a 4096 x 14336 matrix, 1.15 rows per resident warp, no longer
// runs a second, nearly empty round of rows.  A row that straddles two warps is continued, not re-added: the warp
// that holds its first steps hands its 32 lane accumulators to the next warp through shared memory (an mbarrier
// says when), and that warp goes on accumulating from them.  The sum of a row is therefore formed in one fixed
// order (per lane over the row's steps in order, then a butterfly over the lanes) however the rows are divided:
// the bits of an output do not depend on the grid, on N, or on a split of the matrix across GPUs.  To keep the
// hand-over off the critical path a warp works in the order [its unfinished last row][its whole rows][the
// continuation of its predecessor's row]: what it hands over is produced first, what it receives is needed last.
//
// Data movement.  The bytes of a warp's next stages (1, 2 or 4 consecutive steps) are brought into a warp-private
// ring of shared-memory slots by bulk asynchronous copies (cp.async.bulk global -> shared, completion on an
// mbarrier) issued by one lane, up to `slots` stages ahead of the math:
//   * memory-level parallelism is set by shared memory, not by registers;
//   * HBM and L2 see whole contiguous ranges, never half-used sectors;
//   * Q4_K streams the GGUF blocks as they are (144 B = 9 x 16 B) and Q6_K the 1680-byte units of smc_common.cuh,
//     one copy per stage; Q8_0 streams its two planes (quants, scales), two copies per stage;
//   * the lanes read their unit with conflict-free 128-bit shared loads, and the activation row is in shared
//     memory too (16-byte chunks permuted per format so that the strided reads of eight lanes fall in eight
//     different bank groups): the inner loop issues no global loads at all.
// The activation row is quantised to Q8_0 inside the kernel while it is staged (rules of
// QuantizedKVCache.QuantizeRowQ8_0, SharpMind.Model/QuantizedKVCache.cs:191-223), optionally after SiLU(gate) * up
// or a residual add + RMSNorm, so a matmul is one launch with no scratch buffer; rows quantised beforehand
// (smc_q8act) are staged as they are.
// A slot is re-armed only after __syncwarp(): every lane has passed its wait and read its data, so no lane can be
// left waiting on a phase that has already been reused.  Every wait is bounded; on expiry the warp raises a flag in
// device memory (read back by smc_device_status), drains the copies it still has in flight and stops.
//
// Arithmetic is that of the other SMC_ACT_Q8 kernels: exact int32 block dots (dp4a), one fp32 multiply-add per
// 16- or 32-element block.  Shapes: K % 2048 == 0 (K-quants) / K % 1024 == 0 (Q8_0).
// References: VecDotQ4K_* SharpMind.Core/Quantization/QuantizationKernels.Q4.cs:586-747, GetScaleMinK4_*
// QuantizationKernels.cs:177-189, VecDotQ6K_* QuantizationKernels.Q6.cs:12-235, VecDotQ8_0_*
// QuantizationKernels.Q8.cs:11-138.
#include <stdlib.h>

#include "smc_common.cuh"
#include "smc_gather.cuh"

namespace {

constexpr int WARPS = 24;  // warps per SM: one CTA of 24, or two of 12 (the CTA size is a launch parameter)
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
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

// explicit shared-space accesses on 32-bit addresses
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
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }

// stores into the staged activation row (sx = its shared::cta address)
__device__ __forceinline__ void xst64(uint32_t sx, uint32_t off, uint2 v)
{
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(sx + off), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void xst32(uint32_t sx, uint32_t off, uint32_t v)
{
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(sx + off), "r"(v) : "memory");
}
// Thread-block clusters: the CTAs of a pair each quantise half of the activation row and store it into both shared
// memories (sx2 = the partner's row as a shared::cluster address; 0 = no partner).
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t v;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(v));
    return v;
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t cta_addr, uint32_t rank)
{
    uint32_t v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(v) : "r"(cta_addr), "r"(rank));
    return v;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void xst64r(uint32_t sx2, uint32_t off, uint2 v)
{
    asm volatile("st.shared::cluster.v2.u32 [%0], {%1,%2};" ::"r"(sx2 + off), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void xst32r(uint32_t sx2, uint32_t off, uint32_t v)
{
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(sx2 + off), "r"(v) : "memory");
}

__device__ __forceinline__ float warp_sum32(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct XPtrs {
    const int8_t *q;    // rows quantised beforehand (smc_q8act), used when xf is null
    const float *d;
    const float *sd;
    const int16_t *s16;
    const float *xf;  // when set: fp32 activations, quantised to Q8_0 while they are staged
    const float *xu;  // when set too: the staged row is SiLU(xf[i]) * xu[i] (FfnKernels.Gated's activation)
    // when nw is set: the staged row is RMSNorm(xf + xadd) * nw (xadd may be null), and CTA 0 writes xf + xadd to
    // xsum: the residual add and the norm of a decoder block folded into the matmul that consumes them
    const float *xadd, *nw;
    float *xsum;
    float eps;
};

// Shared layout of the staged activation row: q [K] int8 | d [K/32] float | aux.  The quants are stored in 16-byte
// chunks permuted by Math::swz so that the 128-bit reads of a quarter warp (eight lanes, each format with its own
// stride pattern) fall in eight different bank groups.  aux is, per format,
//   Q4_K (Math::SD):  sd [K/32] float = d * sum(q) of the block (the min term's factor);
//   Q6_K (Math::S16): m32 [K/16] int32 = -32 * sum(q) of each sixteen (the codes' offset), eight per 128 elements in
//                     the order [sixteen o of a column][column c], so that a lane reads its four with one 16-byte load.
template <class Math>
__host__ __device__ inline size_t x_bytes(int K)
{
    return (size_t)K + (size_t)(K / 32) * 4 + (Math::SD ? (size_t)(K / 32) * 4 : 0) + (Math::S16 ? (size_t)(K / 16) * 4 : 0);
}
__device__ __forceinline__ int m32_pos(int g16) { return (g16 >> 3) * 8 + (g16 & 1) * 4 + ((g16 >> 1) & 3); }

// `mid` is called once, after the first round of loads has been issued and before anything waits for it: the kernel
// uses it to request the rest of its weight stages BEHIND the activation loads.  Requested the other way round, the
// activation loads would queue behind every byte the rings have in flight, and the whole CTA would wait for them.
template <class Math, class Mid>
__device__ __forceinline__ void stage_x(const XPtrs &g, int K, uint8_t *sx, Mid mid)
{
    uint4 *sq = reinterpret_cast<uint4 *>(sx);
    float *sdx = reinterpret_cast<float *>(sx + K);
    float *ssd = sdx + K / 32;
    int *sm32 = reinterpret_cast<int *>(sdx + K / 32);
    const uint4 *gq = reinterpret_cast<const uint4 *>(g.q);
    constexpr int R = 4;  // 16-byte chunks per thread and round
    const int nq = K / 16;
    bool first = true;
    for (int i0 = threadIdx.x; i0 < nq || first; i0 += R * blockDim.x) {
        uint4 v[R];
        int16_t hs[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int i = i0 + j * blockDim.x;
            if (i < nq) {
                v[j] = __ldg(gq + i);
                if (Math::S16) hs[j] = __ldg(g.s16 + i);
            }
        }
        if (first) mid();
        first = false;
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int i = i0 + j * blockDim.x;
            if (i < nq) {
                sq[Math::swz(i)] = v[j];
                if (Math::S16) sm32[m32_pos(i)] = -32 * (int)hs[j];
            }
        }
    }
    for (int i = threadIdx.x; i < K / 32; i += blockDim.x) {
        sdx[i] = __ldg(g.d + i);
        if (Math::SD) ssd[i] = __ldg(g.sd + i);
    }
}
// round-half-even(x / scale), the quotient correctly rounded first (what QuantizeRowQ8_0's MathF.Round(x / d) does), at
// the price of a multiplication in all but rare cases: x * (1/scale) with an approximate reciprocal is within 1e-4 of
// the exact quotient for |quotient| <= 128, so both round to the same integer unless the product lies that close to a
// half; only then (or when the product is not finite) the IEEE division decides.
__device__ __forceinline__ int quant_div_rn(float x, float scale, float rcp)
{
    const float t = x * rcp;
    const float f = fabsf(t - rintf(t));
    if (!(fabsf(f - 0.5f) > 1e-3f) || !(fabsf(t) < 200.0f)) return __float2int_rn(__fdiv_rn(x, scale));
    return __float2int_rn(t);
}

// Quantises the eight values of chunk c (lanes 4b .. 4b+3 hold the four chunks of block b) and stores them, their
// block scale and sums in the staged layout: the rules of QuantizedKVCache.QuantizeRowQ8_0 (d = amax/127, 1 for a
// zero block, stored through fp16; q = round-half-even(x/d)).
template <class Math>
__device__ __forceinline__ void quant_chunk(const float (&v)[8], int c, int K, uint32_t dst, uint32_t dst2 = 0)
{
    const uint32_t o_d = (uint32_t)K, o_aux = (uint32_t)K + (uint32_t)(K / 32) * 4u;
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float scale = __fdiv_rn(amax, 127.0f);
    if (amax == 0.0f) scale = 1.0f;
    float rcp;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"(scale));
    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[i] = max(-128, min(127, quant_div_rn(v[i], scale, rcp)));
        s += q[i];
    }
    uint2 packed;
    packed.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
    packed.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
    const uint32_t o_q = 16u * (uint32_t)Math::swz(c >> 1) + 8u * (c & 1);
    xst64(dst, o_q, packed);
    if (dst2) xst64r(dst2, o_q, packed);
    const int s16v = s + __shfl_xor_sync(0xffffffffu, s, 1);
    const int total = s16v + __shfl_xor_sync(0xffffffffu, s16v, 2);
    const int blk = c >> 2;
    if (Math::S16 && (c & 1) == 0) {
        xst32(dst, o_aux + 4u * (uint32_t)m32_pos(c >> 1), (uint32_t)(-32 * s16v));
        if (dst2) xst32r(dst2, o_aux + 4u * (uint32_t)m32_pos(c >> 1), (uint32_t)(-32 * s16v));
    }
    if ((c & 3) == 0) {
        const float df = __half2float(__float2half_rn(scale));
        xst32(dst, o_d + 4u * blk, __float_as_uint(df));
        if (Math::SD) xst32(dst, o_aux + 4u * blk, __float_as_uint(df * (float)total));
        if (dst2) {
            xst32r(dst2, o_d + 4u * blk, __float_as_uint(df));
            if (Math::SD) xst32r(dst2, o_aux + 4u * blk, __float_as_uint(df * (float)total));
        }
    }
}

// Same layout, filled by quantising an fp32 row on the fly.  Four consecutive lanes share a 32-element block,
// eight elements each; all loads of a round (R chunks per thread) are issued before any arithmetic so a round costs
// one memory latency, not one per block.  With `up` the row is SiLU(x) * up in the arithmetic of the stand-alone
// kernel.  `mid` as for stage_x: called once, after the first round's loads are on their way.
// In a cluster of two, CTA `part` of `parts` quantises that share of the row and stores it into both shared memories
// (dst2 = the partner's copy); the caller then meets the partner at a cluster barrier.
template <class Math, int R, bool GATE, class Mid>
__device__ __forceinline__ void stage_x_quant(const float *x, const float *up, int K, uint32_t dst, Mid mid, int part = 0, int parts = 1,
                                              uint32_t dst2 = 0)
{
    // K is a multiple of 1024, so whole warps stay converged, also in a half of the row
    const int cbeg = (K / 8 / parts) * part, cend = cbeg + K / 8 / parts;
    bool called = false;
    for (int c0 = cbeg + threadIdx.x; c0 < cend; c0 += R * blockDim.x) {
        float4 va[R], vb[R], ua[GATE ? R : 1], ub[GATE ? R : 1];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int c = c0 + j * blockDim.x;
            if (c < cend) {
                va[j] = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c);
                vb[j] = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c + 1);
                if (GATE) {
                    ua[j] = __ldg(reinterpret_cast<const float4 *>(up) + 2 * c);
                    ub[j] = __ldg(reinterpret_cast<const float4 *>(up) + 2 * c + 1);
                }
            }
        }
        if (!called) mid(), called = true;
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int c = c0 + j * blockDim.x;
            if (c < cend) {  // uniform per warp: the row is a multiple of 128 chunks
                float v[8] = {va[j].x, va[j].y, va[j].z, va[j].w, vb[j].x, vb[j].y, vb[j].z, vb[j].w};
                if (GATE) {  // g / (1 + exp(-g)) * u
                    const float u[8] = {ua[j].x, ua[j].y, ua[j].z, ua[j].w, ub[j].x, ub[j].y, ub[j].z, ub[j].w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = __fdiv_rn(v[i], 1.0f + expf(-v[i])) * u[i];
                }
                quant_chunk<Math>(v, c, K, dst, dst2);
            }
        }
    }
    if (!called) mid();
}

// The residual add and the RMSNorm that precede a matmul in a decoder block, done while its activation row is
// staged: v = x + add (add may be null), xsum = v (written by the CTA that is given a pointer), row = v * rsqrt(mean
// v^2 + eps) * w, quantised as above.  K <= 9216: a thread keeps its (at most three) chunks in registers between the
// sum of squares and the scaling.  The sum of squares is taken in a fixed order (thread chunks in order, warp
// butterfly, warps in order), which is not the order of the stand-alone norm kernel: results agree to rounding.
template <class Math, class Mid>
__device__ __forceinline__ void stage_x_addnorm_quant(const float *x, const float *add, const float *w, float eps, float *xsum,
                                                      int K, uint32_t dst, Mid mid)
{
    __shared__ float red[32];
    const int nchunks = K / 8;
    constexpr int UB = 3;  // chunks per thread: K <= 8 * 3 * 384 with CTAs of twelve warps
    float v[UB][8];
    float ss = 0.f;
    float4 pa[UB], pb[UB];
#pragma unroll
    for (int j = 0; j < UB; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nchunks) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c), b = __ldg(reinterpret_cast<const float4 *>(x) + 2 * c + 1);
            v[j][0] = a.x, v[j][1] = a.y, v[j][2] = a.z, v[j][3] = a.w, v[j][4] = b.x, v[j][5] = b.y, v[j][6] = b.z, v[j][7] = b.w;
            if (add) pa[j] = __ldg(reinterpret_cast<const float4 *>(add) + 2 * c), pb[j] = __ldg(reinterpret_cast<const float4 *>(add) + 2 * c + 1);
        }
    }
    mid();
#pragma unroll
    for (int j = 0; j < UB; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < nchunks) {
            if (add) {
                const float4 p = pa[j], q = pb[j];
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
            quant_chunk<Math>(r, c, K, dst);
        }
    }
}

// Where the weight arrays of a format start (piece sizes and slot offsets are Math constants).
struct StepSrc {
    const uint8_t *base[2];  // step 0 of the tensor in each weight array
};

// Fetches `n` consecutive steps starting at global step `g` (contiguous in every weight array) into a slot sized
// for SS steps.  PIECES and the per-piece sizes are compile-time so that the elected lane spends a handful of
// instructions here.
template <class Math, int SS>
__device__ __forceinline__ void issue_stage(const StepSrc &s, long long g, int n, uint32_t slot_addr, uint32_t bar)
{
    mbar_expect_tx(bar, Math::STEP_BYTES * (uint32_t)n);
#pragma unroll
    for (int i = 0; i < Math::PIECES; ++i)
        bulk_g2s(slot_addr + Math::piece_off(i) * SS, s.base[i] + (size_t)g * Math::piece_bytes(i), Math::piece_bytes(i) * (uint32_t)n,
                 bar);
}

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

    uint32_t blk_off, q_off;   // lane's block and qs bytes inside a step
    uint32_t xo[4];            // swizzled byte offsets of the lane's four activation chunks inside a step
    uint32_t dx_off;           // byte offset of the lane's two block scales inside a step
    uint32_t selR, selT;       // PRMT selectors of the scale unpack
    bool low;

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
    }

    // step i of the slot against part `part` of the staged row (sx = shared address of the row, K its length)
    template <int SS>
    __device__ __forceinline__ void step(uint32_t slot, int i, int part, uint32_t sx, int K, float &acc) const
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
        const uint32_t xb = sx + part * 2048;
        const uint4 a0 = lds128(xb + xo[0]), a1 = lds128(xb + xo[1]), c0 = lds128(xb + xo[2]), c1 = lds128(xb + xo[3]);
        const uint32_t db = sx + K + part * 256 + dx_off;
        const uint2 t0 = lds64(db), t1 = lds64(db + (K >> 3));
        const float2 dx = make_float2(__uint_as_float(t0.x), __uint_as_float(t0.y));
        const float2 sdx = make_float2(__uint_as_float(t1.x), __uint_as_float(t1.y));
        int lo = smc_dp4a(q0.x & M4, a0.x, 0), lo2 = smc_dp4a(q0.y & M4, a0.y, 0);
        lo = smc_dp4a(q0.z & M4, a0.z, lo), lo2 = smc_dp4a(q0.w & M4, a0.w, lo2);
        lo = smc_dp4a(q1.x & M4, a1.x, lo), lo2 = smc_dp4a(q1.y & M4, a1.y, lo2);
        lo = smc_dp4a(q1.z & M4, a1.z, lo), lo2 = smc_dp4a(q1.w & M4, a1.w, lo2);
        // high nibbles are dotted in place: every term carries a factor 16, taken out exactly afterwards
        int hi = smc_dp4a_us(q0.x & MH, c0.x, 0), hi2 = smc_dp4a_us(q0.y & MH, c0.y, 0);
        hi = smc_dp4a_us(q0.z & MH, c0.z, hi), hi2 = smc_dp4a_us(q0.w & MH, c0.w, hi2);
        hi = smc_dp4a_us(q1.x & MH, c1.x, hi), hi2 = smc_dp4a_us(q1.y & MH, c1.y, hi2);
        hi = smc_dp4a_us(q1.z & MH, c1.z, hi), hi2 = smc_dp4a_us(q1.w & MH, c1.w, hi2);
        lo += lo2;
        hi = (hi + hi2) >> 4;
        const float tsum = fmaf((float)(sc_lo * lo), dx.x, (float)(sc_hi * hi) * dx.y);
        const float msum = fmaf(mn_lo, sdx.x, mn_hi * sdx.y);
        acc = fmaf(d, tsum, acc);
        acc = fmaf(-dmin, msum, acc);
    }
};

// ------------------------------------------------------------------------------------------------ Q6_K
struct MathQ6K {
    static constexpr int STEP_ELEMS = 2048;
    static constexpr int PIECES = 1;  // one unit of the layout in smc_common.cuh
    static constexpr uint32_t STEP_BYTES = SMC_Q6U_BYTES;
    static __host__ __device__ constexpr uint32_t piece_bytes(int) { return SMC_Q6U_BYTES; }
    static __host__ __device__ constexpr uint32_t piece_off(int) { return 0; }
    static constexpr bool SD = false, S16 = true;
    // a quarter warp reads chunks 16*b + 8*h + o + 2*c (two b, two h, two o, fixed c)
    static __host__ __device__ __forceinline__ int swz(int c) { return c ^ (((c >> 3) & 3) << 1); }

    uint32_t w_off, sc_off, d_off;
    uint32_t xo[4], dx_off, m32_off;
    int odd;

    __device__ __forceinline__ void init(int lane)
    {
        const int b = lane >> 2, r = lane & 3, h = r >> 1;
        odd = r & 1;
        w_off = 16 * lane;  // lane slot 4b + 2h + o is the lane itself
        sc_off = SMC_Q6U_SC + b * 16 + 8 * h;
        d_off = SMC_Q6U_D + 2 * b;
        const int c = 16 * b + 8 * h + odd;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) xo[cc] = 16 * swz(c + 2 * cc);
        dx_off = (8 * b + 4 * h) * 4;
        m32_off = (2 * b + h) * 32 + odd * 16;
    }

    template <int SS>
    __device__ __forceinline__ void step(uint32_t slot, int i, int part, uint32_t sx, int K, float &acc) const
    {
        slot += i * SMC_Q6U_BYTES;
        const uint4 X = lds128(slot + w_off), Y = lds128(slot + SMC_Q6U_Y + w_off), Z = lds128(slot + SMC_Q6U_Z + w_off);
        const uint2 usc = lds64(slot + sc_off);
        const float d = smc_h2f((uint16_t)lds16u(slot + d_off));
        const uint32_t wx[4] = {X.x, X.y, X.z, X.w}, wy[4] = {Y.x, Y.y, Y.z, Y.w}, wz[4] = {Z.x, Z.y, Z.z, Z.w};
        uint32_t q[4][4];  // [word j][column c]
#pragma unroll
        for (int j = 0; j < 4; ++j) smc_q6u_codes(wx[j], wy[j], wz[j], q[j]);
        const uint32_t xb = sx + part * 2048;
        // sum (q - 32) x = sum q x - 32 sum x: the second term is the chain's starting value
        const uint4 mu = lds128(sx + K + (K >> 3) + part * 512 + m32_off);
        int s[4] = {(int)mu.x, (int)mu.y, (int)mu.z, (int)mu.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 x = lds128(xb + xo[c]);
            s[c] = smc_dp4a(q[0][c], x.x, s[c]);
            s[c] = smc_dp4a(q[1][c], x.y, s[c]);
            s[c] = smc_dp4a(q[2][c], x.z, s[c]);
            s[c] = smc_dp4a(q[3][c], x.w, s[c]);
        }
        const uint4 dxu = lds128(sx + K + part * 256 + dx_off);
        // int8 scales is + {0, 2, 4, 6} with is = o: bytes o, o+2, o+4, o+6 of the half's eight
        const uint32_t sw0 = odd ? (usc.x >> 8) : usc.x, sw1 = odd ? (usc.y >> 8) : usc.y;
        const int scl[4] = {(int)(int8_t)(sw0 & 0xFF), (int)(int8_t)((sw0 >> 16) & 0xFF), (int)(int8_t)(sw1 & 0xFF),
                            (int)(int8_t)((sw1 >> 16) & 0xFF)};
        const float dxs[4] = {__uint_as_float(dxu.x), __uint_as_float(dxu.y), __uint_as_float(dxu.z), __uint_as_float(dxu.w)};
        float rsum = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) rsum = fmaf((float)(scl[c] * s[c]), dxs[c], rsum);
        acc = fmaf(d, rsum, acc);
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
    __device__ __forceinline__ void init(int lane)
    {
        const int sel = (lane >> 2) & 1;
        qa_off = 32 * lane + 16 * sel;
        qb_off = 32 * lane + 16 * (1 - sel);
        d_off = 2 * lane;
        dx_off = 4 * lane;
    }
    template <int SS>
    __device__ __forceinline__ void step(uint32_t slot, int i, int part, uint32_t sx, int K, float &acc) const
    {
        const uint4 q0 = lds128(slot + i * 1024 + qa_off), q1 = lds128(slot + i * 1024 + qb_off);
        const float d = smc_h2f((uint16_t)lds16u(slot + SS * 1024 + i * 64 + d_off));
        const uint32_t xb = sx + part * 1024;
        const uint4 a0 = lds128(xb + qa_off), a1 = lds128(xb + qb_off);
        const float dx = __uint_as_float(lds32(sx + K + part * 128 + dx_off));
        int s = smc_dp4a(q0.x, a0.x, 0), s2 = smc_dp4a(q0.y, a0.y, 0);
        s = smc_dp4a(q0.z, a0.z, s), s2 = smc_dp4a(q0.w, a0.w, s2);
        s = smc_dp4a(q1.x, a1.x, s), s2 = smc_dp4a(q1.y, a1.y, s2);
        s = smc_dp4a(q1.z, a1.z, s), s2 = smc_dp4a(q1.w, a1.w, s2);
        acc = fmaf(d * dx, (float)(s + s2), acc);
    }
};

// ------------------------------------------------------------------------------------------------
// MODE 0: out[row] = sum.  MODE 1: the same, and the slice is exchanged with the peers (gather, or partial sums added in
// rank order).  MODE 2: the matrix holds gate and up rows interleaved (row 2i = gate i, row 2i + 1 = up i) and the
// kernel writes out[i] = SiLU(sum(2i)) * sum(2i + 1) (FfnKernels.Gated's activation, Layers/Ffn/FfnKernels.cs:35-59):
// a CTA owns whole pairs, parks its row sums in shared memory and forms the products when its rows are done, so the
// down projection stages a plain row instead of every SM recomputing SiLU over the whole row.
template <class Math, int SS, int MODE, bool PAIR = false>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_tma_kernel(StepSrc src, XPtrs xg, float *__restrict__ out, int N, int K,
                                                                    int slots, int tune, int *__restrict__ status,
                                                                    const smc_gather_dev *gd)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t SLOT = (Math::STEP_BYTES * SS + 127u) & ~127u;
    constexpr bool GATHER = MODE == 1, PAIRS = MODE == 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nw = blockDim.x >> 5;  // warps of this CTA

    // shared layout: [x row] [WARPS x slots x SLOT bytes] [WARPS x slots ring barriers] [WARPS x 32 floats handed
    // from warp w-1 to warp w] [WARPS hand-over barriers]
    const uint32_t xb = (uint32_t)((x_bytes<Math>(K) + 127) & ~(size_t)127);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + xb + (uint32_t)(warp * slots) * SLOT;
    const uint32_t bars = sbase + xb + (uint32_t)(nw * slots) * SLOT + (uint32_t)(warp * slots) * 8u;
    const uint32_t hand = sbase + xb + (uint32_t)(nw * slots) * (SLOT + 8u);  // + 128 * warp
    const uint32_t hbar = hand + nw * 128u;                                     // + 8 * warp

    // this CTA's rows, and this warp's piece [s0, s1) of their steps
    const int spr = K / Math::STEP_ELEMS;  // steps per row
    const int G = gridDim.x, cta = blockIdx.x;
    constexpr int RU = PAIRS ? 2 : 1;  // rows are dealt out in units of one row, or of one (gate, up) pair
    const int rbase = (N / RU) / G, rrem = N / RU - rbase * G;
    const int R0 = RU * (cta * rbase + min(cta, rrem)), nrows = RU * (rbase + (cta < rrem ? 1 : 0));
    const uint32_t srow = hbar + nw * 8u;  // PAIRS: this CTA's row sums, RU * (rbase + 1) floats
    const int T = nrows * spr;
    const int Wa = T < nw ? T : nw;  // warps that get work
    int s0 = 0, s1 = 0;
    if (warp < Wa) {
        s0 = (int)((long long)T * warp / Wa);
        s1 = (int)((long long)T * (warp + 1) / Wa);
    }
    // processing order: [tb, s1) the start of a row the next warp finishes, [hb, tb) whole rows, [s0, hb) the end of a
    // row the previous warp started.  A piece that lies inside one row is all "end of row" and is handed on.
    const int hb = (s0 % spr == 0) ? s0 : min(s1, (s0 / spr + 1) * spr);
    const int tb = (s1 % spr == 0) ? s1 : max(hb, (s1 / spr) * spr);
    const int segb[3] = {tb, hb, s0}, sege[3] = {s1, tb, hb};
    const long long gstep0 = (long long)R0 * spr;

    if (lane == 0) {
        for (int s = 0; s < slots; ++s) mbar_init(bars + 8 * s, 1);
        mbar_init(hbar + 8 * warp, 1);
        fence_barrier_init();
    }
    __syncwarp();
    // producer cursor (used by lane 0): segment and step of the next stage to fetch
    int pseg = 0, ps = segb[0], issued = 0;
    auto fetch_next = [&](uint32_t saddr, uint32_t bar) -> bool {
        while (pseg < 3 && ps >= sege[pseg]) {
            ++pseg;
            if (pseg < 3) ps = segb[pseg];
        }
        if (pseg >= 3) return false;
        const int n = min(SS, sege[pseg] - ps);
        issue_stage<Math, SS>(src, gstep0 + ps, n, saddr, bar);
        ps += n;
        ++issued;
        return true;
    };
    // One stage per warp is requested at once: weights depend on no earlier launch, so this part of the stream runs
    // under the predecessor's tail.  The other slots are filled from `fill_rest`, behind the activation loads.
    const int pre = tune & 0xFF;
    if (lane == 0)
        for (int t = 0; t < pre && t < slots; ++t)
            if (!fetch_next(ring + (uint32_t)t * SLOT, bars + 8 * t)) break;
    auto fill_rest = [&]() {
        if (lane == 0)
            for (int t = pre; t < slots; ++t)
                if (!fetch_next(ring + (uint32_t)t * SLOT, bars + 8 * t)) break;
    };
    // Everything below depends on earlier launches (activations, the output buffer, the exchange counters), so this
    // is where a dependent launch waits for its predecessor.
    smc_grid_dep_sync();
    // split across GPUs: the number of this exchange (the counter is advanced by the previous exchange's last CTA, which
    // the dependency wait above has seen complete)
    const unsigned gtag = GATHER ? smc_gather_tag(gd) : 0u;
    const bool greduce = GATHER && (tune & 0x100);  // partial sums of a K-split: every rank gets every output, summed
    // PAIR: launched as clusters of two (long fp32 rows), each CTA of a pair quantises half of the row for both.  A
    // template parameter, so that the kernels of short rows (a decode step's) carry none of this code.
    constexpr uint32_t cn = PAIR ? 2u : 1u;
    const int cpart = PAIR ? (int)cluster_cta_rank() : 0;
    const uint32_t peer_x = PAIR ? cluster_map(sbase, (uint32_t)cpart ^ 1u) : 0u;
    if (xg.xf) {
        if (xg.nw) stage_x_addnorm_quant<Math>(xg.xf, xg.xadd, xg.nw, xg.eps, blockIdx.x == 0 ? xg.xsum : nullptr, K, sbase, fill_rest);
        else if (xg.xu) stage_x_quant<Math, 2, true>(xg.xf, xg.xu, K, sbase, fill_rest, cpart, (int)cn, peer_x);
        else stage_x_quant<Math, 4, false>(xg.xf, nullptr, K, sbase, fill_rest, cpart, (int)cn, peer_x);
    } else {
        stage_x<Math>(xg, K, smem, fill_rest);  // rows quantised beforehand
    }
    // the row is staged, and every warp's hand-over barrier is initialised; nothing touches the partner's shared
    // memory after this barrier, so either CTA of a pair may finish first
    if (PAIR) cluster_sync_all();
    else __syncthreads();
    Math math;
    math.init(lane);
    float acc = 0.f;
    int slot = 0, consumed = 0;
    uint32_t phase = 0;
    bool dead = false;
    for (int sg = 0; sg < 3 && !dead; ++sg) {
        int s = segb[sg];
        const int e = sege[sg];
        if (s >= e) continue;
        int part = s % spr, row = R0 + s / spr;
        if (sg == 2) {  // the lane sums of the row's first steps, left by the previous warp
            if (!__all_sync(0xffffffffu, mbar_wait(hbar + 8 * warp, 0))) {
                if (lane == 0) atomicExch(status, 1);
                dead = true;
                break;
            }
            acc = __uint_as_float(lds32(hand + 128 * warp + 4 * lane));
        }
        while (s < e) {
            const int n = min(SS, e - s);
            const uint32_t bar = bars + 8 * slot;
            const uint32_t saddr = ring + (uint32_t)slot * SLOT;
            if (!__all_sync(0xffffffffu, mbar_wait(bar, phase))) {  // one decision for the warp
                if (lane == 0) atomicExch(status, 1);
                dead = true;
                break;
            }
            ++consumed;
#pragma unroll
            for (int i = 0; i < SS; ++i) {
                if (i < n) {
                    math.template step<SS>(saddr, i, part, sbase, K, acc);
                    if (++part == spr) {
                        const float v = warp_sum32(acc);  // every lane holds the sum
                        if (lane == 0) {
                            if (PAIRS) sts32(srow + 4u * (uint32_t)(row - R0), __float_as_uint(v));
                            else if (!greduce) out[row] = v;
                        }
                        // this rank's chunk starts at rank * N in every peer's packet area; lane p sends to peer p
                        if (GATHER) smc_gather_send_warp(gd, (size_t)N, (size_t)row, v, gtag, greduce);
                        acc = 0.f;
                        part = 0;
                        ++row;
                    }
                }
            }
            __syncwarp();  // every lane has read the slot: it may be refilled
            if (lane == 0) fetch_next(saddr, bar);
            if (++slot == slots) {
                slot = 0;
                phase ^= 1;
            }
            s += n;
        }
        if (!dead && part != 0) {  // an unfinished row: the next warp continues from these sums
            sts32(hand + 128 * (warp + 1) + 4 * lane, __float_as_uint(acc));
            __syncwarp();
            if (lane == 0) mbar_arrive(hbar + 8 * (warp + 1));
            acc = 0.f;
        }
    }
    if (dead) {
        // copies already requested still target this CTA's shared memory: wait for them (bounded) before leaving
        const int pending = __shfl_sync(0xffffffffu, issued, 0) - consumed;
        for (int t = 0; t < pending; ++t) {
            mbar_wait(bars + 8 * slot, phase);
            if (++slot == slots) {
                slot = 0;
                phase ^= 1;
            }
        }
    }
    if (PAIRS) {  // every row sum of this CTA is in shared memory: out[i] = SiLU(gate i) * up i, the stand-alone kernel's arithmetic
        __syncthreads();
        for (int i = threadIdx.x; i < nrows / 2; i += blockDim.x) {
            const float g = __uint_as_float(lds32(srow + 8u * i)), u = __uint_as_float(lds32(srow + 8u * i + 4u));
            out[R0 / 2 + i] = __fdiv_rn(g, 1.0f + expf(-g)) * u;
        }
    }
    // rows done: unpack this CTA's stripe of the peers' slices as they arrive
    if (GATHER) {
        if (greduce) smc_gather_collect_reduce(gd, (size_t)N, blockIdx.x, gridDim.x, gtag);
        else smc_gather_collect(gd, (size_t)N, blockIdx.x, gridDim.x, gtag);
        smc_gather_done(gd, gridDim.x);
    }
}

template <class Math, int SS>
void launch_one(smc_ctx *ctx, dim3 grid, int nw, size_t smem, cudaStream_t s, const StepSrc &src, const XPtrs &x, float *out, int N,
                int K, int slots, const smc_gather_dev *gd, bool reduce, bool pairs)
{
    const int tune = (ctx->tma_pre & 0xFF) | (reduce ? 0x100 : 0);
    // A long fp32 row (quantised, perhaps SiLU-gated, by every CTA while HBM waits) is shared by the two SMs of a pair:
    // each quantises half.  Only the plain and the gated staging split (K % 1024 == 0 keeps whole warps in each half).
    const int pair_min_k = ctx->tma_cluster > 1 ? ctx->tma_cluster : (x.xu ? 6144 : 8192);  // an option value above 1 is the row length to pair from
    const bool pair_sms = ctx->tma_cluster && x.xf && !x.nw && K >= pair_min_k && grid.x % 2 == 0 && (nw == WARPS || ctx->tma_cluster > 1);
    if (gd) {
        cudaFuncSetAttribute(gemv_tma_kernel<Math, SS, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (pair_sms) {
            cudaFuncSetAttribute(gemv_tma_kernel<Math, SS, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            smc_launch_dep_cluster(ctx->use_pdl, 2, gemv_tma_kernel<Math, SS, 1, true>, grid, dim3(nw * 32), smem, s, src, x, out, N, K, slots,
                                   tune, ctx->d_status, gd);
        } else
            smc_launch_dep(ctx->use_pdl, gemv_tma_kernel<Math, SS, 1>, grid, dim3(nw * 32), smem, s, src, x, out, N, K, slots,
                           tune, ctx->d_status, gd);
        return;
    }
    if (pairs) {
        cudaFuncSetAttribute(gemv_tma_kernel<Math, SS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        smc_launch_dep(ctx->use_pdl, gemv_tma_kernel<Math, SS, 2>, grid, dim3(nw * 32), smem, s, src, x, out, N, K, slots,
                       tune, ctx->d_status, (const smc_gather_dev *)nullptr);
        return;
    }
    cudaFuncSetAttribute(gemv_tma_kernel<Math, SS, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (pair_sms) {
        cudaFuncSetAttribute(gemv_tma_kernel<Math, SS, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        smc_launch_dep_cluster(ctx->use_pdl, 2, gemv_tma_kernel<Math, SS, 0, true>, grid, dim3(nw * 32), smem, s, src, x, out, N, K, slots,
                               tune, ctx->d_status, (const smc_gather_dev *)nullptr);
        return;
    }
    smc_launch_dep(ctx->use_pdl, gemv_tma_kernel<Math, SS, 0>, grid, dim3(nw * 32), smem, s, src, x, out, N, K, slots,
                   tune, ctx->d_status, (const smc_gather_dev *)nullptr);
}

template <class Math>
int launch_math(smc_ctx *ctx, const StepSrc &src, const XPtrs &x, float *out, int N, int K, cudaStream_t s,
                const smc_gather_dev *gd, bool reduce, bool pairs)
{
    // One CTA of 24 warps per SM: the activation row is fetched and quantised once per SM (with three CTAs of eight
    // warps each, 444 copies of a 14336-element fp32 row were half as many bytes into the SMs as the matrix itself).
    // Ring geometry: `slots` stages of `ss` steps per warp.
    int slots = ctx->tma_slots ? ctx->tma_slots : 2;
    int ss = ctx->tma_ss ? ctx->tma_ss : 2;
    // short rows (little to stage per CTA) run a little faster as two CTAs of twelve warps per SM (measured: 28672 x 4096
    // Q4_K 15.2 -> 14.7 us, 3072 x 1024 Q8_0 4.5 -> 4.0 us); long rows as one CTA of 24, which stages the row once per SM
    const int nw = ctx->tma_warps ? ctx->tma_warps : (K <= 4096 ? 12 : WARPS), per_sm = WARPS / nw;
    const size_t xb = (x_bytes<Math>(K) + 127) & ~(size_t)127;
    auto need = [&](int sl, int st) {
        const size_t slot_bytes = ((size_t)Math::STEP_BYTES * st + 127) & ~(size_t)127;
        return xb + (size_t)nw * sl * (slot_bytes + 8) + (size_t)nw * 136;
    };
    // a long activation row first costs ring depth, then stage length
    while ((need(slots, ss) + 1024) * per_sm > 227 * 1024) {
        if (slots > 2) --slots;
        else if (ss > 1) ss >>= 1;
        else break;
    }
    int ctas = ctx->tma_ctas ? ctx->tma_ctas : ctx->sm_count * per_sm;
    const int units = pairs ? N / 2 : N;  // what is dealt out to the CTAs: rows, or (gate, up) pairs
    if (ctas > units) ctas = units;
    // the pair form parks a CTA's row sums in shared memory behind the hand-over barriers
    const size_t smem = need(slots, ss) + (pairs ? (size_t)8 * (units / ctas + 1) + 16 : 0);
    if ((smem + 1024) * per_sm > 227 * 1024) return smc_fail(ctx, SMC_E_UNSUPPORTED, "K = %d needs %zu bytes of shared memory", K, smem);
    const dim3 grid(ctas);
    if (ss == 4) launch_one<Math, 4>(ctx, grid, nw, smem, s, src, x, out, N, K, slots, gd, reduce, pairs);
    else if (ss == 2) launch_one<Math, 2>(ctx, grid, nw, smem, s, src, x, out, N, K, slots, gd, reduce, pairs);
    else launch_one<Math, 1>(ctx, grid, nw, smem, s, src, x, out, N, K, slots, gd, reduce, pairs);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

}  // namespace

bool smc_tma_supported(const smc_weight *w, int M)
{
    if (!w->fast || M != 1) return false;
    if (w->dtype == SMC_Q8_0) return w->K % 1024 == 0 && w->K <= 65536 && w->q8_qs != nullptr;
    if (w->dtype == SMC_Q6_K) return w->K % 2048 == 0 && w->K <= 65536 && w->q6u != nullptr;
    return w->K % 2048 == 0 && w->K <= 65536 && w->d_raw != nullptr;
}

// fp32 input: the row is quantised inside the kernel, no scratch buffer is involved.
int smc_launch_gemv_tma_f32in(smc_ctx *ctx, const float *x, const smc_weight *w, float *out, cudaStream_t s)
{
    return smc_launch_gemv_tma_full(ctx, nullptr, x, nullptr, nullptr, w, out, nullptr, s);
}

// Row 0 of `a`, quantised beforehand.
int smc_launch_gemv_tma(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s)
{
    return smc_launch_gemv_tma_full(ctx, a, nullptr, nullptr, nullptr, w, out, nullptr, s);
}

// One fp32 row, quantised in the kernel, whose output slice is exchanged with the peers in the kernel's tail.
int smc_launch_gemv_tma_gather(smc_ctx *ctx, const float *x, const smc_weight *w, float *out, const smc_gather_dev *gd,
                               cudaStream_t s)
{
    return smc_launch_gemv_tma_full(ctx, nullptr, x, nullptr, nullptr, w, out, gd, s);
}

// The same exchange for a row quantised beforehand.
int smc_launch_gemv_tma_xg(smc_ctx *ctx, const smc_q8act *a, const float *xf, const smc_weight *w, float *out,
                           const smc_gather_dev *gd, cudaStream_t s)
{
    return smc_launch_gemv_tma_full(ctx, a, xf, nullptr, nullptr, w, out, gd, s);
}

// One row whose activation is SiLU(gate) * up, formed and quantised while the row is staged.
int smc_launch_gemv_tma_swiglu(smc_ctx *ctx, const float *gate, const float *up, const smc_weight *w, float *out, cudaStream_t s)
{
    return smc_launch_gemv_tma_full(ctx, nullptr, gate, up, nullptr, w, out, nullptr, s);
}

// One row that is RMSNorm(x + add) * w, formed and quantised while the row is staged; x + add goes to `sum`.
int smc_launch_gemv_tma_addnorm(smc_ctx *ctx, const float *x, const smc_norm_prologue *pro, const smc_weight *w, float *out,
                                cudaStream_t s)
{
    return smc_launch_gemv_tma_full(ctx, nullptr, x, nullptr, pro, w, out, nullptr, s);
}

int smc_launch_gemv_tma_full(smc_ctx *ctx, const smc_q8act *a, const float *xf, const float *xu, const smc_norm_prologue *pro,
                             const smc_weight *w, float *out, const smc_gather_dev *gd, cudaStream_t s)
{
    return smc_launch_gemv_tma_any(ctx, a, xf, xu, pro, w, out, gd, false, false, s);
}

// `reduce`: the matrix is a K-slice; the partial sums of all ranks are exchanged and added in rank order into the
// dense buffer of `gd` (out is not written).
// `pairs`: the matrix is gate / up rows interleaved and out [N / 2] receives SiLU(gate) * up (no exchange in this form).
int smc_launch_gemv_tma_any(smc_ctx *ctx, const smc_q8act *a, const float *xf, const float *xu, const smc_norm_prologue *pro,
                            const smc_weight *w, float *out, const smc_gather_dev *gd, bool reduce, bool pairs, cudaStream_t s)
{
    if (pairs && (gd || (w->N & 1))) return smc_fail(ctx, SMC_E_INVALID, "one-row matmul: the pair form takes an even row count and no exchange");
    const int N = w->N, K = w->K;
    if (!xf && (!a || a->M != 1 || a->K != K)) return smc_fail(ctx, SMC_E_INVALID, "one-row matmul: the activation buffer must hold one row of %d", K);
    XPtrs x{};
    if (a) x.q = a->q, x.d = a->d, x.sd = a->sd, x.s16 = a->s16;
    x.xf = xf, x.xu = xu;
    if (pro) x.xadd = pro->add, x.nw = pro->w, x.xsum = pro->sum, x.eps = pro->eps;
    StepSrc src{};
    if (w->dtype == SMC_Q4_K) {
        src.base[0] = w->d_raw;
        return launch_math<MathQ4K>(ctx, src, x, out, N, K, s, gd, reduce, pairs);
    }
    if (w->dtype == SMC_Q6_K) {
        src.base[0] = w->q6u;
        return launch_math<MathQ6K>(ctx, src, x, out, N, K, s, gd, reduce, pairs);
    }
    src.base[0] = reinterpret_cast<const uint8_t *>(w->q8_qs);
    src.base[1] = reinterpret_cast<const uint8_t *>(w->q8_d);
    return launch_math<MathQ8_0>(ctx, src, x, out, N, K, s, gd, reduce, pairs);
}
