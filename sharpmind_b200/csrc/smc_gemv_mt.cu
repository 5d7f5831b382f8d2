// Small-batch (2..32 activation rows) quantised-activation matmul with the weights streamed through a bulk-copy ring:
// the arithmetic of SMC_ACT_Q8 on the int8 tensor-core path (exact int32 block sums by mma.sync, fp32 scaling on the
// CUDA cores), fed the way the one-row kernel is fed.
//
// Why.  The first small-batch kernel (smc_gemv_mma.cu) fetched its MMA fragments from global memory just in time as
// 4- and 8-byte loads and ran at a quarter of the HBM bandwidth with the L1 request path saturated.  Here
//   * a CTA (one per SM) works on TILES of 16 weight rows; the bytes of a tile arrive in STAGES of one step per row
//     (2048 elements for the K-quants, 1024 for Q8_0: the same unit the one-row kernel streams), one bulk copy per
//     row and stage issued by a producer warp into a ring of shared-memory slots with full / empty mbarriers;
//   * rows lie in a slot at a stride that is an odd multiple of 16 bytes modulo 128 (Q4_K 1152 + 16, the Q6_K unit's
//     own 1680, Q8_0 1024 + 16), so one `ldmatrix` delivers the A fragment of 16 rows x 32 bytes without a bank conflict;
//   * the activations of the current SLAB of 4096 columns are staged once per CTA in fragment order (a lane's B
//     fragment is one 8-byte shared load), with their block scales (and d * sum(q) for Q4_K's min term) as pairs in
//     the accumulator's column order.
// Sixteen compute warps share a stage: it has 16 pieces (block b = 0..7 of the step, half hf = 0, 1 of the block; for
// Q8_0 four consecutive 32-element blocks count as a "block").  With up to 8 rows a warp takes one piece; with more it
// takes both halves of a block for half of the token tiles.
//
// Summation order (what makes a result independent of the batch size, of the grid and of a row split across GPUs):
// for every output, per slab, each piece (b, hf) accumulates its blocks' scaled sums over the slab's stages in k
// order; the slab's value is ((P[0,0] + P[0,1]) + (P[1,0] + P[1,1]) + ...) in b order; slabs are added in order.  The CTA
// that owns a tile does all of this itself (slab after slab, adding into the output it wrote before), so nothing
// depends on timing.
//
// Every wait is bounded; on expiry the CTA raises the context's status word, stops consuming, waits (bounded) for
// the copies it still has in flight and ends.
// References: QuantizedMatMul* SharpMind.Core/Quantization/QuantizationKernels.cs:24-42 (weights re-streamed per
// row there), block formats QuantizationKernels.Q4.cs:586-623, Q6.cs:12-65, Q8.cs:11-40.
#include <type_traits>

#include "smc_async.cuh"
#include "smc_common.cuh"

namespace {

constexpr int CW = 16;                     // compute warps
constexpr int THREADS = (CW + 2) * 32;     // + the producer warp and the warp that adds the partial tiles
template <int NT>
__host__ __device__ constexpr int red_buffers() { return NT == 4 ? 1 : 2; }  // buffers the partial tiles of consecutive tiles alternate between (shared memory is short at 32 rows)
constexpr int TILE = 16;                   // weight rows per tile
constexpr int SLAB = 4096;                 // columns whose activations are resident at a time
constexpr int RED_PAD = 1;

__device__ __forceinline__ void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t &r0, uint32_t &r1)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// int -> float of a block sum.  The kernel is bound by instruction issue, not by the conversion pipe: one conversion
// (quarter rate, its own pipe) costs one issue slot where the add-a-magic-number form costs two.
__device__ __forceinline__ float i2f(int c) { return (float)c; }
__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory"); }

// Activations of one slab in shared memory, `sbs` 32-element blocks x NT token tiles:
//   xq  uint2  [sbs][NT][32 lanes]   lane (g, tg): bytes 4tg..4tg+3 and 16+4tg..16+4tg+3 of token 8t+g's block
//   xd  float2 [sbs][NT][4]          block scales of tokens 8t+2tg and 8t+2tg+1
//   xs  float2 [sbs][NT][4]          the same tokens' d * sum(q) (formats with a min term)
// Plain pointers, not inline-asm loads: the compiler may then request all of a piece's operands before the first MMA
// (a warp issues in order, so a load written behind a dependent chain would wait for that chain); the mbarrier waits
// are volatile asm with a memory clobber, which keeps these loads behind them.
struct XAddr {
    const uint2 *xq;
    const float2 *xd, *xs;
    uint32_t xq_s, xd_s, xs_s;  // the same as shared-space addresses, for the staging stores
};

// ---- per-format geometry and the work on one piece (b, hf) of a stage ----------------------------------------
// SPS = steps of a row that one bulk copy brings (a stage is 16 rows x SPS steps).  The copy engine of an SM takes
// roughly one request per 50 ns whatever its size (measured: sixteen 1152-byte requests per stage capped the kernel
// at 25 GB/s per SM), so a request has to carry 2 KB or more for the SM's 44 GB/s share of HBM.
// STRIDE / 16 is odd for every format and SPS: eight consecutive rows then start in eight different 16-byte bank groups.
template <int SPS>
struct FQ4K {
    static constexpr int STEP = 2048, ROW_BYTES = 1152, STRIDE = SPS * ROW_BYTES + 16, SLOT_BYTES = TILE * STRIDE, SB = 64;
    static constexpr bool HAS_MIN = true;
    const uint8_t *raw;
    size_t row_pitch;  // bytes between rows
    __device__ void issue(uint32_t slot, uint32_t bar, int row, int step, int ns, int lane) const
    {
        if (lane < TILE)
            smc_bulk_g2s(slot + lane * STRIDE, raw + (size_t)(row + lane) * row_pitch + (size_t)step * ROW_BYTES, (uint32_t)ns * ROW_BYTES, bar);
    }
    static __device__ uint32_t tx(int ns) { return (uint32_t)(TILE * ROW_BYTES) * (uint32_t)ns; }
    template <int NT, int TW, int hf>
    __device__ __forceinline__ void piece(uint32_t slot, const uint8_t *sp, int u, int b, int jj0, int t0, const XAddr &x, float (&acc)[TW][4], int lane) const
    {
        slot += u * ROW_BYTES, sp += u * ROW_BYTES;
        const int g = lane >> 2, tg = lane & 3;
        const int e0 = (jj0 + 8 * b + 4 * hf) * NT + t0;  // operand index of this piece's first block and token tile
        const uint2 *xqp = x.xq + e0 * 32 + lane;
        const float2 *xdp = x.xd + e0 * 4 + tg, *xsp = x.xs + e0 * 4 + tg;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(sp + (lane & 15) * STRIDE + b * 144);
        const float d = smc_h2f((uint16_t)(hdr.x & 0xFFFFu)), dmin = smc_h2f((uint16_t)(hdr.x >> 16));
        float dsc[4], dmn[4];
#pragma unroll
        for (int jl = 0; jl < 4; ++jl) {
            int sc, mn;
            smc_k4_scale_min(hdr.y, hdr.z, hdr.w, 4 * hf + jl, sc, mn);
            dsc[jl] = d * (float)sc;
            dmn[jl] = dmin * (float)mn;
        }
        const uint32_t rowsel = ((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + 16 * (lane >> 4);
#pragma unroll
        for (int gl = 0; gl < 2; ++gl) {
            uint32_t a[4];
            ldsm_x4(slot + rowsel + b * 144 + 16 + 32 * (2 * hf + gl), a[0], a[1], a[2], a[3]);
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {
                const int jl = 2 * gl + hi;
                uint32_t an[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) an[k] = (hi ? (a[k] >> 4) : a[k]) & 0x0F0F0F0Fu;
                const float ws0 = __shfl_sync(0xffffffffu, dsc[jl], g), ws1 = __shfl_sync(0xffffffffu, dsc[jl], g + 8);
                const float wm0 = __shfl_sync(0xffffffffu, dmn[jl], g), wm1 = __shfl_sync(0xffffffffu, dmn[jl], g + 8);
#pragma unroll
                for (int tw = 0; tw < TW; ++tw) {
                    const int e = jl * NT + tw;
                    const uint2 bq = xqp[e * 32];
                    const float2 dx = xdp[e * 4], sx = xsp[e * 4];
                    int c[4];
                    mma_k32(c, an[0], an[1], an[2], an[3], bq.x, bq.y);
                    acc[tw][0] = fmaf(-wm0, sx.x, fmaf(i2f(c[0]), ws0 * dx.x, acc[tw][0]));
                    acc[tw][1] = fmaf(-wm0, sx.y, fmaf(i2f(c[1]), ws0 * dx.y, acc[tw][1]));
                    acc[tw][2] = fmaf(-wm1, sx.x, fmaf(i2f(c[2]), ws1 * dx.x, acc[tw][2]));
                    acc[tw][3] = fmaf(-wm1, sx.y, fmaf(i2f(c[3]), ws1 * dx.y, acc[tw][3]));
                }
            }
        }
    }
};

template <int C>
__device__ __forceinline__ uint32_t q6_col(uint32_t wx, uint32_t wy, uint32_t wz)
{
    const uint32_t M6 = 0x3F3F3F3Fu;
    uint32_t q;
    if (C == 0) q = wx & M6;
    else if (C == 1) q = wy & M6;
    else if (C == 2) q = wz & M6;
    else q = ((wx >> 6) & 0x03030303u) | ((wy >> 4) & 0x0C0C0C0Cu) | ((wz >> 2) & 0x30303030u);
    return __vsub4(q, 0x20202020u);  // codes 0..63 -> -32..31
}

template <int SPS>
struct FQ6K {
    static constexpr int STEP = 2048, ROW_BYTES = SMC_Q6U_BYTES, STRIDE = SPS * ROW_BYTES + (SPS % 2 ? 0 : 16), SLOT_BYTES = TILE * STRIDE, SB = 64;
    static constexpr bool HAS_MIN = false;
    const uint8_t *raw;  // unit layout
    size_t row_pitch;
    __device__ void issue(uint32_t slot, uint32_t bar, int row, int step, int ns, int lane) const
    {
        if (lane < TILE)
            smc_bulk_g2s(slot + lane * STRIDE, raw + (size_t)(row + lane) * row_pitch + (size_t)step * ROW_BYTES, (uint32_t)ns * ROW_BYTES, bar);
    }
    static __device__ uint32_t tx(int ns) { return (uint32_t)(TILE * ROW_BYTES) * (uint32_t)ns; }
    // piece (b, hf): half hf of block b: per sixteen o the X / Y / Z entries of lane slot (b, hf, o) give the codes of the
    // four 32-element columns; a scale covers 16 elements, so the unit is mma.m16n8k16
    template <int NT, int TW, int hf>
    __device__ __forceinline__ void piece(uint32_t slot, const uint8_t *sp, int u, int b, int jj0, int t0, const XAddr &x, float (&acc)[TW][4], int lane) const
    {
        slot += u * ROW_BYTES, sp += u * ROW_BYTES;
        const int g = lane >> 2, tg = lane & 3;
        const int e0 = (jj0 + 8 * b + 4 * hf) * NT + t0;
        const uint2 *xqp = x.xq + e0 * 32 + lane;
        const float2 *xdp = x.xd + e0 * 4 + tg;
        const uint8_t *mine = sp + (lane & 15) * STRIDE;
        const uint4 scw = *reinterpret_cast<const uint4 *>(mine + SMC_Q6U_SC + 16 * b);
        const float d = smc_h2f(*reinterpret_cast<const uint16_t *>(mine + SMC_Q6U_D + 2 * b));
        const uint32_t scws[2] = {hf ? scw.z : scw.x, hf ? scw.w : scw.y};
        const uint32_t rowsel = ((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE;
#pragma unroll
        for (int o = 0; o < 2; ++o) {
            const uint32_t ent = 16 * (4 * b + 2 * hf + o);
            uint32_t wx[2], wy[2], wz[2];
            ldsm_x4(slot + rowsel + ent + SMC_Q6U_Y * (lane >> 4), wx[0], wx[1], wy[0], wy[1]);
            ldsm_x2(slot + rowsel + ent + SMC_Q6U_Z, wz[0], wz[1]);
            auto column = [&](auto cc) {
                constexpr int c = decltype(cc)::value;
                const int si = o + 2 * c;
                const uint32_t a0 = q6_col<c>(wx[0], wy[0], wz[0]), a1 = q6_col<c>(wx[1], wy[1], wz[1]);
                const float dsc = d * (float)(int)(int8_t)((scws[si >> 2] >> (8 * (si & 3))) & 0xFF);
                const float ws0 = __shfl_sync(0xffffffffu, dsc, g), ws1 = __shfl_sync(0xffffffffu, dsc, g + 8);
#pragma unroll
                for (int tw = 0; tw < TW; ++tw) {
                    const int e = c * NT + tw;
                    const uint2 bq = xqp[e * 32];
                    const float2 dx = xdp[e * 4];
                    int c4[4];
                    mma_k16(c4, a0, a1, o ? bq.y : bq.x);
                    acc[tw][0] = fmaf(i2f(c4[0]), ws0 * dx.x, acc[tw][0]);
                    acc[tw][1] = fmaf(i2f(c4[1]), ws0 * dx.y, acc[tw][1]);
                    acc[tw][2] = fmaf(i2f(c4[2]), ws1 * dx.x, acc[tw][2]);
                    acc[tw][3] = fmaf(i2f(c4[3]), ws1 * dx.y, acc[tw][3]);
                }
            };
            column(std::integral_constant<int, 0>{});
            column(std::integral_constant<int, 1>{});
            column(std::integral_constant<int, 2>{});
            column(std::integral_constant<int, 3>{});
        }
    }
};

template <int SPS>
struct FQ8_0 {
    static constexpr int STEP = 1024, ROW_BYTES = 1024, STRIDE = SPS * 1024 + 16, SCALES = TILE * STRIDE, SLOT_BYTES = TILE * STRIDE + TILE * 64 * SPS, SB = 32;
    static constexpr bool HAS_MIN = false;
    const uint8_t *qs;    // [N][K] int8
    const uint8_t *ds;    // [N][K/32] fp16
    size_t row_pitch;     // K
    __device__ void issue(uint32_t slot, uint32_t bar, int row, int step, int ns, int lane) const
    {
        if (lane < TILE) smc_bulk_g2s(slot + lane * STRIDE, qs + (size_t)(row + lane) * row_pitch + (size_t)step * 1024, (uint32_t)ns * 1024, bar);
        else smc_bulk_g2s(slot + SCALES + (lane - TILE) * 64 * SPS, ds + ((size_t)(row + lane - TILE) * (row_pitch / 32) + (size_t)step * 32) * 2, (uint32_t)ns * 64, bar);
    }
    static __device__ uint32_t tx(int ns) { return (uint32_t)(TILE * (1024 + 64)) * (uint32_t)ns; }
    // piece (b, hf): blocks 4b + 2hf and 4b + 2hf + 1 of the step's 32
    template <int NT, int TW, int hf>
    __device__ __forceinline__ void piece(uint32_t slot, const uint8_t *sp, int u, int b, int jj0, int t0, const XAddr &x, float (&acc)[TW][4], int lane) const
    {
        const int g = lane >> 2, tg = lane & 3;
        const int e0 = (jj0 + 4 * b + 2 * hf) * NT + t0;
        const uint2 *xqp = x.xq + e0 * 32 + lane;
        const float2 *xdp = x.xd + e0 * 4 + tg;
        const uint32_t rowsel = ((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + 16 * (lane >> 4) + u * 1024;
        const uint32_t dpair = *reinterpret_cast<const uint32_t *>(sp + SCALES + (lane & 15) * 64 * SPS + u * 64 + 2 * (4 * b + 2 * hf));  // this lane's row: both blocks' scales
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
            const int s = 4 * b + 2 * hf + sl;
            uint32_t a[4];
            ldsm_x4(slot + rowsel + 32 * s, a[0], a[1], a[2], a[3]);
            const float dw = smc_h2f((uint16_t)(sl ? (dpair >> 16) : (dpair & 0xFFFFu)));
            const float ws0 = __shfl_sync(0xffffffffu, dw, g), ws1 = __shfl_sync(0xffffffffu, dw, g + 8);
#pragma unroll
            for (int tw = 0; tw < TW; ++tw) {
                const int e = sl * NT + tw;
                const uint2 bq = xqp[e * 32];
                const float2 dx = xdp[e * 4];
                int c[4];
                mma_k32(c, a[0], a[1], a[2], a[3], bq.x, bq.y);
                acc[tw][0] = fmaf(i2f(c[0]), ws0 * dx.x, acc[tw][0]);
                acc[tw][1] = fmaf(i2f(c[1]), ws0 * dx.y, acc[tw][1]);
                acc[tw][2] = fmaf(i2f(c[2]), ws1 * dx.x, acc[tw][2]);
                acc[tw][3] = fmaf(i2f(c[3]), ws1 * dx.y, acc[tw][3]);
            }
        }
    }
};

template <class F, int NT>
__host__ __device__ constexpr size_t x_region_bytes()
{
    return (size_t)(SLAB / 32) * NT * (256 + 32 + (F::HAS_MIN ? 32 : 0));
}
template <int NT>
__host__ __device__ constexpr size_t red_bytes()
{
    return (size_t)(NT == 1 ? 16 : 8) * TILE * (8 * NT + RED_PAD) * 4;  // one buffer
}

// Shared memory: [x region][red buffers][ring slots][barriers: full[slots], empty[slots], redfull[RB], redfree[RB]]
template <class F, int NT, int SPS>
__global__ void __launch_bounds__(THREADS, 1)
gemv_mt_kernel(F fmt, const int8_t *__restrict__ xq, const float *__restrict__ xd, const float *__restrict__ xsd,
               float *__restrict__ out, int N, int K, int M, int slots, int *status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int s_abort;
    constexpr int TW = NT == 4 ? 2 : 1;          // token tiles per warp
    constexpr int NPART = NT == 1 ? 16 : 8;      // partial tiles that meet in the reduction
    constexpr int RSTRIDE = 8 * NT + RED_PAD;    // floats per row of a partial tile
    constexpr int RB = red_buffers<NT>();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t sbase = smc_smem_u32(smem);
    const uint32_t xr = sbase, redr = xr + (uint32_t)x_region_bytes<F, NT>();
    const uint32_t ring = (redr + (uint32_t)(RB * red_bytes<NT>()) + 127u) & ~127u;
    const uint32_t slot_bytes = (F::SLOT_BYTES + 127u) & ~127u;
    const uint32_t bars = ring + (uint32_t)slots * slot_bytes;
    const uint32_t rbars = bars + 16 * (uint32_t)slots;  // redfull[RB], redfree[RB]
    XAddr xa;
    xa.xq_s = xr, xa.xd_s = xr + (SLAB / 32) * NT * 256, xa.xs_s = xa.xd_s + (SLAB / 32) * NT * 32;
    xa.xq = reinterpret_cast<const uint2 *>(smem), xa.xd = reinterpret_cast<const float2 *>(smem + (SLAB / 32) * NT * 256);
    xa.xs = xa.xd + (SLAB / 32) * NT * 4;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < slots; ++s) {
            smc_mbar_init(bars + 8 * s, 1);
            smc_mbar_init(bars + 8 * (slots + s), CW);
        }
        for (int r = 0; r < RB; ++r) {
            smc_mbar_init(rbars + 8 * r, CW);
            smc_mbar_init(rbars + 8 * (RB + r), 1);
        }
        smc_fence_barrier_init();
    }
    __syncthreads();
    // tiles of this CTA: a contiguous range
    const int tiles = N / TILE;
    const int tile0 = (int)((long long)blockIdx.x * tiles / gridDim.x), tile1 = (int)((long long)(blockIdx.x + 1) * tiles / gridDim.x);
    const int nslab = (K + SLAB - 1) / SLAB;
    volatile int *abortp = &s_abort;
    auto give_up = [&]() {
        if (lane == 0 && !*abortp) atomicExch(status, 1), *abortp = 1;
    };

    if (warp == CW) {
        // ---- producer: the same (slab, tile, stage) sequence as the consumers, `slots` stages ahead at most.
        // Weights depend on no earlier launch, so this runs ahead of the dependency wait of the other warps.
        int slot = 0, issued = 0;
        uint32_t phase = 0;
        bool dead = false;
        for (int sl = 0; sl < nslab && !dead; ++sl) {
            const int st0 = sl * (SLAB / F::STEP), st1 = min(K / F::STEP, st0 + SLAB / F::STEP);
            for (int t = tile0; t < tile1 && !dead; ++t)
                for (int st = st0; st < st1; st += SPS) {
                    const int ns = min(SPS, st1 - st);
                    if (issued >= slots) {  // the slot's previous stage must have been consumed by all compute warps
                        bool ok = true;
                        if (lane == 0) ok = smc_mbar_wait(bars + 8 * (slots + slot), phase ^ 1);
                        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) && !*abortp;
                        if (!ok) {
                            give_up();
                            dead = true;
                            break;
                        }
                    }
                    if (lane == 0) smc_mbar_expect_tx(bars + 8 * slot, F::tx(ns));
                    __syncwarp();
                    fmt.issue(ring + (uint32_t)slot * slot_bytes, bars + 8 * slot, t * TILE, st, ns, lane);
                    ++issued;
                    if (++slot == slots) slot = 0, phase ^= 1;
                }
        }
        // nothing may still be in flight towards this CTA's shared memory when it ends
        __syncwarp();
        if (lane == 0) {
            const int pend = issued < slots ? issued : slots;
            for (int i = 0; i < pend; ++i) {
                const int k = issued - 1 - i;  // stage number; its slot and the parity of its completion
                smc_mbar_wait(bars + 8 * (k % slots), (uint32_t)(k / slots) & 1u);
            }
        }
        return;
    }

    smc_grid_dep_sync();  // activations (and the output an earlier slab wrote) come from earlier launches

    if (warp == CW + 1) {
        // ---- the warp that adds the partial tiles of a (slab, tile) and stores (slab 0) or adds to (later slabs) the
        // output: the compute warps only post their tile and go on
        int n = 0;
        bool dead = false;
        for (int sl = 0; sl < nslab; ++sl)
            for (int t = tile0; t < tile1; ++t, ++n) {
                const int buf = n % RB;
                const uint32_t use = (uint32_t)(n / RB);
                if (!dead && (!__all_sync(0xffffffffu, smc_mbar_wait(rbars + 8 * buf, use & 1u)) || *abortp)) {
                    give_up();
                    dead = true;
                }
                if (dead) continue;
                const uint32_t rb = redr + (uint32_t)buf * (uint32_t)red_bytes<NT>();
#pragma unroll
                for (int q = 0; q < 4 * NT; ++q) {
                    const int o = lane + 32 * q, row = o & 15, tok = o >> 4;
                    auto rd = [&](int p) { return __uint_as_float(smc_lds32(rb + (uint32_t)((p * TILE + row) * RSTRIDE + tok) * 4)); };
                    float s;
                    if (NT == 1) {
                        s = rd(0) + rd(1);
#pragma unroll
                        for (int p = 1; p < 8; ++p) s += rd(2 * p) + rd(2 * p + 1);
                    } else {
                        s = rd(0);
#pragma unroll
                        for (int p = 1; p < NPART; ++p) s += rd(p);
                    }
                    if (tok < M) {
                        float *dst = out + (size_t)tok * N + (size_t)t * TILE + row;
                        *dst = sl == 0 ? s : *dst + s;
                    }
                }
                __syncwarp();
                if (lane == 0) smc_mbar_arrive(rbars + 8 * (RB + buf));
            }
        return;
    }

    // ---- compute warps
    const int g = lane >> 2, tg = lane & 3;
    const int nb = K / 32;
    int slot = 0, n = 0;
    uint32_t phase = 0;
    bool dead = false;
    const int b = NT == 1 ? (warp >> 1) : (warp & 7);
    const int t0w = NT == 1 ? 0 : (NT == 2 ? (warp >> 3) : 2 * (warp >> 3));
    for (int sl = 0; sl < nslab; ++sl) {
        const int col0 = sl * SLAB, cols = min(SLAB, K - col0), sbs = cols / 32;
        const int st0 = col0 / F::STEP, st1 = st0 + cols / F::STEP;
        // ---- stage this slab's activations in fragment order
        bar_compute();  // everybody is done with the previous slab's
        {
            // one 16-byte load per (block, token, half of the block): its four words go to the four lanes (token, tg);
            // all of a thread's loads are requested before the first one is used
            constexpr int UN = 4;  // loads in flight per thread and round; a full slab is 4 * NT items per thread
            const int items = sbs * NT * 16;
            for (int base = 0; base < items; base += UN * CW * 32) {
                uint4 v[UN];
#pragma unroll
                for (int u = 0; u < UN; ++u) {
                    const int i = base + threadIdx.x + u * CW * 32;
                    if (i < items) {
                        const int h = i & 1, gq = (i >> 1) & 7, t = (i >> 4) % NT, jj = i / (16 * NT);
                        const int tok = min(8 * t + gq, M - 1);
                        v[u] = __ldg(reinterpret_cast<const uint4 *>(xq + (size_t)tok * K + col0 + 32 * jj + 16 * h));
                    }
                }
#pragma unroll
                for (int u = 0; u < UN; ++u) {
                    const int i = base + threadIdx.x + u * CW * 32;
                    if (i < items) {
                        const int h = i & 1, gq = (i >> 1) & 7, t = (i >> 4) % NT, jj = i / (16 * NT);
                        const uint32_t dst = xa.xq_s + (uint32_t)(((jj * NT + t) * 32 + 4 * gq) * 8 + 4 * h);
                        smc_sts32(dst, v[u].x), smc_sts32(dst + 8, v[u].y), smc_sts32(dst + 16, v[u].z), smc_sts32(dst + 24, v[u].w);
                    }
                }
            }
        }
        for (int i = threadIdx.x; i < sbs * NT * 4; i += CW * 32) {
            const int q = i & 3, t = (i >> 2) % NT, jj = i / (4 * NT);
            const int tk0 = min(8 * t + 2 * q, M - 1), tk1 = min(8 * t + 2 * q + 1, M - 1);
            const size_t o0 = (size_t)tk0 * nb + col0 / 32 + jj, o1 = (size_t)tk1 * nb + col0 / 32 + jj;
            smc_sts64(xa.xd_s + (uint32_t)i * 8, make_uint2(__float_as_uint(xd[o0]), __float_as_uint(xd[o1])));
            if (F::HAS_MIN) smc_sts64(xa.xs_s + (uint32_t)i * 8, make_uint2(__float_as_uint(xsd[o0]), __float_as_uint(xsd[o1])));
        }
        bar_compute();
        for (int t = tile0; t < tile1; ++t, ++n) {
            float acc[2][TW][4];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int tw = 0; tw < TW; ++tw)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[h][tw][i] = 0.f;
            for (int st = st0; st < st1; st += SPS) {
                const int ns = min(SPS, st1 - st);
                if (!dead && (!__all_sync(0xffffffffu, smc_mbar_wait(bars + 8 * slot, phase)) || *abortp)) {
                    give_up();
                    dead = true;
                }
                if (!dead) {
                    const uint32_t sa = ring + (uint32_t)slot * slot_bytes;
                    const uint8_t *sp = smem + (sa - sbase);
#pragma unroll
                    for (int u = 0; u < SPS; ++u) {
                        if (u < ns) {
                            const int jj0 = (st + u - st0) * F::SB;
                            if (NT == 1) {  // warp-uniform: the half is a property of the warp
                                if (warp & 1) fmt.template piece<NT, TW, 1>(sa, sp, u, b, jj0, 0, xa, acc[0], lane);
                                else fmt.template piece<NT, TW, 0>(sa, sp, u, b, jj0, 0, xa, acc[0], lane);
                            } else {
                                fmt.template piece<NT, TW, 0>(sa, sp, u, b, jj0, t0w, xa, acc[0], lane);
                                fmt.template piece<NT, TW, 1>(sa, sp, u, b, jj0, t0w, xa, acc[1], lane);
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) smc_mbar_arrive(bars + 8 * (slots + slot));
                }
                if (++slot == slots) slot = 0, phase ^= 1;
            }
            // ---- post this warp's partial tile: red[buf][part][row][token]
            const int buf = n % RB;
            const uint32_t use = (uint32_t)(n / RB);
            if (!dead && use > 0 && (!__all_sync(0xffffffffu, smc_mbar_wait(rbars + 8 * (RB + buf), (use - 1) & 1u)) || *abortp)) {
                give_up();
                dead = true;
            }
            if (dead) continue;
            const uint32_t rb = redr + (uint32_t)buf * (uint32_t)red_bytes<NT>();
            const int part = NT == 1 ? warp : b;
#pragma unroll
            for (int tw = 0; tw < TW; ++tw)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float v = NT == 1 ? acc[0][tw][i] : acc[0][tw][i] + acc[1][tw][i];
                    const int row = g + ((i >> 1) << 3), tok = 8 * (t0w + tw) + 2 * tg + (i & 1);
                    smc_sts32(rb + (uint32_t)((part * TILE + row) * RSTRIDE + tok) * 4, __float_as_uint(v));
                }
            __syncwarp();
            if (lane == 0) smc_mbar_arrive(rbars + 8 * buf);
        }
    }
}

template <class F, int NT, int SPS>
int launch_nt(smc_ctx *ctx, const F &fmt, const smc_q8act *a, float *out, int N, int K, cudaStream_t s)
{
    constexpr int RB = red_buffers<NT>();
    const size_t fixed = x_region_bytes<F, NT>() + RB * red_bytes<NT>() + 128;
    const size_t slot_bytes = (F::SLOT_BYTES + 127u) & ~127u;
    const size_t room = 227 * 1024 - 1024 - fixed - 256;
    int slots = room / slot_bytes > 4 ? 4 : (int)(room / slot_bytes);
    if (slots < 2) return smc_fail(ctx, SMC_E_UNSUPPORTED, "small-batch kernel: no room for a ring of two stages");
    const size_t smem = fixed + (size_t)slots * slot_bytes + 16 * slots + 16 * RB + 128;
    int ctas = ctx->tma_ctas ? ctx->tma_ctas : ctx->sm_count;  // one per SM; the option exists for the partition tests
    if (ctas > N / TILE) ctas = N / TILE;
    auto kernel = gemv_mt_kernel<F, NT, SPS>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    smc_launch_dep(ctx->use_pdl, kernel, dim3(ctas), dim3(THREADS), smem, s, fmt, (const int8_t *)a->q, (const float *)a->d,
                   (const float *)a->sd, out, N, K, a->M, slots, ctx->d_status);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// Steps per bulk copy: as many as leave room for a ring next to the activations of a slab (which grow with the rows).
// The choice moves bytes only: every (row, step) is added in the same place of the same sum whatever it is.
template <template <int> class FT, int S_SMALL, int S_MID, int S_BIG, class... Init>
int launch_fmt(smc_ctx *ctx, const smc_q8act *a, float *out, int N, int K, cudaStream_t s, Init... init)
{
    if (a->M <= 8) return launch_nt<FT<S_SMALL>, 1, S_SMALL>(ctx, FT<S_SMALL>{init...}, a, out, N, K, s);
    if (a->M <= 16) return launch_nt<FT<S_MID>, 2, S_MID>(ctx, FT<S_MID>{init...}, a, out, N, K, s);
    return launch_nt<FT<S_BIG>, 4, S_BIG>(ctx, FT<S_BIG>{init...}, a, out, N, K, s);
}

}  // namespace

bool smc_mt_supported(const smc_weight *w, int M)
{
    if (!w->fast || M < 2 || M > 32 || w->N % TILE) return false;
    if (w->dtype == SMC_Q8_0) return w->K % 1024 == 0 && w->q8_qs != nullptr;
    if (w->dtype == SMC_Q4_K) return w->K % 2048 == 0 && w->d_raw != nullptr;
    if (w->dtype == SMC_Q6_K) return w->K % 2048 == 0 && w->q6u != nullptr;
    return false;
}

int smc_launch_gemv_mt(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s)
{
    const int N = w->N, K = w->K;
    if (w->dtype == SMC_Q4_K) return launch_fmt<FQ4K, 2, 2, 1>(ctx, a, out, N, K, s, (const uint8_t *)w->d_raw, (size_t)(K / 256) * 144);
    if (w->dtype == SMC_Q6_K) return launch_fmt<FQ6K, 2, 2, 1>(ctx, a, out, N, K, s, (const uint8_t *)w->q6u, (size_t)(K / 2048) * SMC_Q6U_BYTES);
    return launch_fmt<FQ8_0, 4, 4, 1>(ctx, a, out, N, K, s, reinterpret_cast<const uint8_t *>(w->q8_qs), reinterpret_cast<const uint8_t *>(w->q8_d), (size_t)K);
}
