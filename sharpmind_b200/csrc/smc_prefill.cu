// Prefill-sized quantised matmul on the 5th-generation tensor cores (tcgen05 + TMEM), Q4_K weights.
//
//   out[t, r] = sum_k x[t, k] * w[r, k],   w[r, k] = d_b * (sc_j * q_k) - dmin_b * m_j
//
// (block b = k / 256 of row r, sub-block j = (k % 256) / 32; VecDotQ4K, QuantizationKernels.Q4.cs:586-747).
// The integer part sc_j * q_k <= 63 * 15 is exact in fp16, so the tensor cores multiply exact weights:
//   acc_d[r, t] = sum_{k in b} (sc_j q_k) * x~[t, k]        16 MMAs of K = 16 per block and activation half
//   acc_m[r, t] = sum_b sum_{j < 8} (dmin_b m_j) * sx~[t, b, j]   two MMAs of K = 16 per block, one accumulator
//   out[t, r]   = s_t * (sum_b d_b * acc_d(b) - acc_m)      CUDA cores: one FMA per block, one subtraction at the end
// x~ = x / s_t with s_t a power of two that brings the row's largest magnitude to about 2^10, carried as an
// fp16 pair (hi, lo) so that hi + lo holds 22 significant bits of x~: the result stays inside the fp32 parity
// bound of the fp32-activation mode.  sx~ is the fp32 sum of x~ over a 32-element sub-block and dmin_b m_j the
// exact fp32 product (17 significant bits), both also carried as fp16 pairs.
//
// One CTA computes 128 weight rows x 128 tokens.  Warp roles:
//   warp 0        lane 0 streams the activation tiles with bulk copies (global -> shared, mbarrier tx count)
//   warp 1        lane 0 issues tcgen05.mma / tcgen05.commit
//   warps 2..5    one thread per weight row: reads its 144-byte block, expands the nibbles to fp16 sc*q and
//                 stores them with tcgen05.st into its own lane of tensor memory: the A operand never touches
//                 shared memory (a first version that wrote A tiles to shared memory was bound by shared-memory
//                 bandwidth: 64 KB of stores and 256 KB of MMA operand reads per block and CTA)
//   warps 6..13   drain: tcgen05.ld of acc_d, scaling by d_b, fp32 running sums in registers (64 tokens per
//                 thread), final store
// Shared memory: 6 stages of {B_hi 16 KB, B_lo 16 KB} (64 k each) + 2 x {A'' 4 KB, B'' 8 KB} for the min term.
// TMEM (512 columns): acc_d x 2 buffers (the drain of one block overlaps the MMAs of the next), acc_m, and four
// A stages of 32 columns.  Every mbarrier wait is bounded; a wait that runs out raises the context's status
// word and a CTA-wide abort flag that makes every later wait return at once, so the kernel still ends and
// frees its TMEM.
#include <cuda_fp16.h>
#include <stdio.h>
#include <stdlib.h>

#include "smc_common.cuh"

namespace {

constexpr int TM = 128;    // weight rows per CTA (MMA M)
constexpr int TN = 128;    // tokens per CTA (MMA N)
constexpr int KS = 64;     // k per stage
constexpr int NA = 4;      // A stages in tensor memory = stages per 256-element block
constexpr int NB = 4;      // B stages in shared memory
constexpr int NW = 4;      // blocks of raw weight bytes in shared memory
constexpr uint32_t B_BYTES = TN * KS * 2;      // one of hi / lo
constexpr uint32_t SLOT_BYTES = 2 * B_BYTES;
constexpr uint32_t W_BYTES = TM * 144;          // one 256-element block of every row of the tile
constexpr uint32_t AM_BYTES = TM * 16 * 2;
constexpr uint32_t BM_BYTES = 2 * TN * 16 * 2;  // two tiles: [sx_hi | sx_hi] and [sx_lo | sx_lo]
constexpr uint32_t AUX_BYTES = AM_BYTES + BM_BYTES;
constexpr uint32_t OFF_W = NB * SLOT_BYTES;
constexpr uint32_t OFF_AUX = OFF_W + NW * W_BYTES;
constexpr uint32_t OFF_BAR = OFF_AUX + 2 * AUX_BYTES;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 256;
constexpr int EXPAND_WARPS = 8, DRAIN_WARPS = 8;
constexpr int WARP_EXPAND0 = 2, WARP_DRAIN0 = WARP_EXPAND0 + EXPAND_WARPS;
constexpr int THREADS = (WARP_DRAIN0 + DRAIN_WARPS) * 32;
constexpr unsigned WAIT_LIMIT = 1u << 22;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
// tensor-memory columns
constexpr uint32_t COL_ACC_D = 0;    // 2 x 128
constexpr uint32_t COL_ACC_M = 256;  // 128
constexpr uint32_t COL_A = 384;      // NA x 32

// barrier slots (8 bytes each) inside the last 256 bytes
enum {
    BAR_FULL_B = 0,
    BAR_EMPTY_B = BAR_FULL_B + NB,
    BAR_FULL_A = BAR_EMPTY_B + NB,
    BAR_EMPTY_A = BAR_FULL_A + NA,
    BAR_FULL_W = BAR_EMPTY_A + NA,
    BAR_EMPTY_W = BAR_FULL_W + NW,
    BAR_ACC_FULL = BAR_EMPTY_W + NW,
    BAR_ACC_EMPTY = BAR_ACC_FULL + 2,
    BAR_COUNT = BAR_ACC_EMPTY + 2
};
static_assert(BAR_COUNT * 8 + 8 <= 256, "barrier area");
constexpr uint32_t OFF_TMEM_PTR = OFF_BAR + BAR_COUNT * 8;
constexpr uint32_t OFF_ABORT = OFF_TMEM_PTR + 4;

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
// Bounded wait.  When the limit runs out, or another thread of the CTA already gave up, raises the flags and
// returns: the caller carries on with whatever is in memory so that the kernel ends in bounded time.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, int *status)
{
    for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 255u) == 255u && *abort_flag) return;
    }
    *abort_flag = 1;
    atomicExch(status, 3);
}
// One lane polls, the warp follows: 128 or 256 threads polling (and arriving on) one barrier word made the
// handshakes themselves the slowest part of the pipeline.
__device__ __forceinline__ void warp_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag, int *status)
{
    if ((threadIdx.x & 31) == 0) mbar_wait(bar, parity, abort_flag, status);
    __syncwarp();
}
__device__ __forceinline__ void warp_arrive(uint32_t bar)
{
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], M = 128, N = 128, K = 16, fp16 operands, fp32 accumulate; one thread issues.
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the A operand taken from tensor memory (128 lanes x 8 columns of packed fp16 pairs).
__device__ __forceinline__ void tc_mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane, written from registers.
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t *r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float *v)
{
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices of 128 contiguous
// bytes; `lbo` = bytes between the two core matrices along K of one MMA, `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// Instruction descriptor: fp32 accumulator, fp16 A and B, both K-major, N = 128, M = 128.
constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);

// ------------------------------------------------------------------------------ activation image
// Global layout read by the GEMM kernel with plain bulk copies (already in the shared-memory order):
//   img  [token tile][stage = k / 64][hi | lo][token / 8][k chunk = (k % 64) / 8][token % 8][k % 8]   fp16
//   mimg [token tile][block = k / 256][hi | lo][token / 8][2][token % 8][8]                          fp16
//        (tile hi: sx~ hi of sub-blocks 0..7, twice; tile lo: sx~ lo, twice)
//   scale[token]  fp32 power of two
__global__ void __launch_bounds__(256) prefill_scale_kernel(const float *__restrict__ x, int M, int K, float *__restrict__ scale)
{
    __shared__ float red[8];
    const int t = blockIdx.x;
    float amax = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) amax = fmaxf(amax, fabsf(x[(size_t)t * K + k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
        float s = 1.0f;
        if (amax > 0.f && amax < INFINITY) {
            int e;
            frexpf(amax, &e);          // amax = f * 2^e, f in [0.5, 1)
            s = ldexpf(1.0f, e - 10);  // amax / s in [512, 1024)
        }
        scale[t] = s;
    }
}

__global__ void __launch_bounds__(256) prefill_image_kernel(const float *__restrict__ x, int M, int K,
                                                            const float *__restrict__ scale, __half *__restrict__ img,
                                                            __half *__restrict__ mimg)
{
    // one CTA per (token tile, 256-element block): 128 tokens x 32 chunks of 8
    const int nsb = K / 256;
    const int tt = blockIdx.x / nsb, sb = blockIdx.x % nsb;
    for (int it = threadIdx.x; it < TN * 32; it += blockDim.x) {
        const int tl = it >> 5, c = it & 31;  // token in tile, chunk in block
        const int t = tt * TN + tl;
        float v[8];
        float inv = 0.f;
        if (t < M) {
            inv = 1.0f / scale[t];  // exact: a power of two
            const float4 a = *reinterpret_cast<const float4 *>(x + (size_t)t * K + sb * 256 + c * 8);
            const float4 b = *reinterpret_cast<const float4 *>(x + (size_t)t * K + sb * 256 + c * 8 + 4);
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        __align__(16) __half hi[8], lo[8];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float xs = v[i] * inv;
            hi[i] = __float2half_rn(xs);
            lo[i] = __float2half_rn(xs - __half2float(hi[i]));
            sum += xs;
        }
        const int stage = sb * 4 + (c >> 3);
        const size_t base = ((size_t)(tt * (K / KS) + stage) * 2) * (TN * KS) + (size_t)(tl >> 3) * (KS / 8 * 64) +
                            (size_t)(c & 7) * 64 + (size_t)(tl & 7) * 8;
        *reinterpret_cast<uint4 *>(img + base) = *reinterpret_cast<const uint4 *>(hi);
        *reinterpret_cast<uint4 *>(img + base + TN * KS) = *reinterpret_cast<const uint4 *>(lo);
        // sub-block sums: chunks 4j .. 4j+3 are adjacent lanes
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((c & 3) == 0) {
            const int j = c >> 2;
            const __half sh = __float2half_rn(sum);
            const __half sl = __float2half_rn(sum - __half2float(sh));
            const size_t mb = (size_t)(tt * nsb + sb) * (2 * TN * 16) + (size_t)(tl >> 3) * 128 + (size_t)(tl & 7) * 8 + j;
            mimg[mb] = sh;
            mimg[mb + 64] = sh;
            mimg[mb + TN * 16] = sl;
            mimg[mb + TN * 16 + 64] = sl;
        }
    }
}

// ------------------------------------------------------------------------------ nibble expansion
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
// One nibble plane of bytes bA bB of `w`: {mul * (1024 + nibble << shift) + off} as an fp16 pair.
__device__ __forceinline__ uint32_t expand_half(uint32_t w, uint32_t sel, uint32_t mask, __half2 mul, __half2 off)
{
    const uint32_t p = (__byte_perm(w, 0u, sel) & mask) | 0x64006400u;
    const __half2 r = __hfma2(*reinterpret_cast<const __half2 *>(&p), mul, off);
    return *reinterpret_cast<const uint32_t *>(&r);
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ------------------------------------------------------------------------------ the GEMM
__global__ void __launch_bounds__(THREADS, 1)
prefill_q4k_kernel(const uint8_t *__restrict__ raw, const __half *__restrict__ img, const __half *__restrict__ mimg,
                   const float *__restrict__ scale, float *__restrict__ out, int N, int K, int M, int ntt, int *status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rt = blockIdx.x / ntt, tt = blockIdx.x % ntt;
    const int row0 = rt * TM;
    const int nsb = K / 256;
    const size_t row_bytes = (size_t)nsb * 144;
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + OFF_ABORT);
    auto bar = [&](int i) { return sbase + OFF_BAR + 8u * (uint32_t)i; };

    if (threadIdx.x == 0) {
        for (int i = 0; i < NB; ++i) {
            mbar_init(bar(BAR_FULL_B + i), 1);
            mbar_init(bar(BAR_EMPTY_B + i), 1);
        }
        for (int i = 0; i < NA; ++i) {
            mbar_init(bar(BAR_FULL_A + i), EXPAND_WARPS);  // one arrival per expansion warp
            mbar_init(bar(BAR_EMPTY_A + i), 1);
        }
        for (int i = 0; i < NW; ++i) {
            mbar_init(bar(BAR_FULL_W + i), 1);             // the expect_tx arrival; the 128 row copies add bytes
            mbar_init(bar(BAR_EMPTY_W + i), EXPAND_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(BAR_ACC_FULL + i), 1);
            mbar_init(bar(BAR_ACC_EMPTY + i), DRAIN_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    if (warp == 0) {
        const uint32_t dst = sbase + OFF_TMEM_PTR;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem + OFF_TMEM_PTR);

    if (warp == 0) {
        // ---------------- activation tiles: one bulk copy of hi|lo per stage (+ the min-term tiles per block)
        if (lane == 0) {
            const __half *src = img + (size_t)tt * (K / KS) * 2 * (TN * KS);
            const __half *msrc = mimg + (size_t)tt * nsb * (2 * TN * 16);
            int slot = 0;
            uint32_t phase = 1;  // a fresh barrier passes a wait on the phase before its first
            for (int sb = 0; sb < nsb; ++sb) {
#pragma unroll
                for (int g = 0; g < NA; ++g) {
                    mbar_wait(bar(BAR_EMPTY_B + slot), phase, abort_flag, status);
                    const uint32_t fb = bar(BAR_FULL_B + slot);
                    mbar_expect_tx(fb, 2 * B_BYTES + (g == 0 ? BM_BYTES : 0u));
                    bulk_g2s(sbase + (uint32_t)slot * SLOT_BYTES, src + (size_t)(sb * NA + g) * 2 * (TN * KS), 2 * B_BYTES, fb);
                    // the aux buffer sb & 1 was last read by the MMAs of block sb - 2, which completed before the
                    // MMAs whose commit released this B slot (a stage of block sb - 1) were even issued
                    if (g == 0)
                        bulk_g2s(sbase + OFF_AUX + (uint32_t)(sb & 1) * AUX_BYTES + AM_BYTES, msrc + (size_t)sb * (2 * TN * 16),
                                 BM_BYTES, fb);
                    if (++slot == NB) slot = 0, phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue.  One thread feeds the tensor cores: an MMA of this shape lasts 64 clocks, so
        // the instructions between two MMAs must stay well below that.  Descriptors are therefore built once and
        // advanced by adding the 16-byte-unit offset to their low word.
        if (lane == 0) {
            const uint32_t acc_m = tmem_base + COL_ACC_M;
            const uint64_t b_desc0 = smem_desc(sbase, 128, 1024);            // stage 0, hi tile, k step 0
            const uint64_t aux_desc0 = smem_desc(sbase + OFF_AUX, 128, 256);  // aux buffer 0, A''
            constexpr uint64_t U_SLOT = SLOT_BYTES >> 4, U_LO = B_BYTES >> 4, U_KK = 256 >> 4;
            constexpr uint64_t U_AUX = AUX_BYTES >> 4, U_BM = AM_BYTES >> 4, U_BM2 = (AM_BYTES + TN * 16 * 2) >> 4;
            int slot = 0;
            uint32_t b_phase = 0;
            for (int sb = 0; sb < nsb; ++sb) {
                const int buf = sb & 1;
                mbar_wait(bar(BAR_ACC_EMPTY + buf), (uint32_t)(((sb >> 1) & 1) ^ 1), abort_flag, status);
                tc_fence_after();
                const uint32_t acc_d = tmem_base + COL_ACC_D + (uint32_t)buf * 128u;
#pragma unroll
                for (int g = 0; g < NA; ++g) {
                    mbar_wait(bar(BAR_FULL_B + slot), b_phase, abort_flag, status);
                    mbar_wait(bar(BAR_FULL_A + g), (uint32_t)(sb & 1), abort_flag, status);
                    tc_fence_after();
                    const uint64_t bh = b_desc0 + (uint64_t)slot * U_SLOT;
                    const uint32_t a0 = tmem_base + COL_A + (uint32_t)g * 32u;
                    if (g == 0) {
                        const uint64_t am = aux_desc0 + (uint64_t)buf * U_AUX;
                        tc_mma_f16(acc_m, am, am + U_BM, IDESC, sb != 0 ? 1u : 0u);
                        tc_mma_f16(acc_m, am, am + U_BM2, IDESC, 1u);
                    }
#pragma unroll
                    for (int kk = 0; kk < KS / 16; ++kk)
                        tc_mma_f16_ta(acc_d, a0 + kk * 8, bh + kk * U_KK, IDESC, (g | kk) != 0 ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < KS / 16; ++kk) tc_mma_f16_ta(acc_d, a0 + kk * 8, bh + U_LO + kk * U_KK, IDESC, 1u);
                    // both arrive when the MMAs above have read their operands
                    tc_commit(bar(BAR_EMPTY_B + slot));
                    tc_commit(bar(BAR_EMPTY_A + g));
                    if (++slot == NB) slot = 0, b_phase ^= 1;
                }
                tc_commit(bar(BAR_ACC_FULL + buf));
            }
        }
    } else if (warp < WARP_DRAIN0) {
        // ---------------- weight expansion.  A warp may only touch the TMEM lanes of its quarter (warp % 4); the
        // two warps of a quarter split a stage: plane 0 expands the low nibbles (sub-block 2g, columns 0..15),
        // plane 1 the high nibbles (sub-block 2g + 1, columns 16..31).  The raw 144-byte blocks arrive through a
        // ring of bulk copies, one copy per row and block, issued NW - 1 blocks ahead by the plane-0 thread of
        // the row: register prefetch of one block was not enough to cover the latency of these scattered reads.
        const int quarter = warp & 3, plane = (warp - WARP_EXPAND0) >> 2;
        const int r = quarter * 32 + lane;
        const uint8_t *rowp = raw + (size_t)(row0 + r) * row_bytes;
        const uint32_t am_row = (uint32_t)(r >> 3) * 256u + (uint32_t)(r & 7) * 16u;
        const uint32_t a_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + COL_A + (uint32_t)plane * 16u;
        const uint32_t w_row = sbase + OFF_W + (uint32_t)r * 144u;
        auto fetch_block = [&](int p) {  // plane-0 threads: request block p of this thread's row
            const int ws = p % NW;
            warp_wait(bar(BAR_EMPTY_W + ws), (uint32_t)(((p / NW) & 1) ^ 1), abort_flag, status);
            const uint32_t fw = bar(BAR_FULL_W + ws);
            if (warp == WARP_EXPAND0 && lane == 0) mbar_expect_tx(fw, W_BYTES);
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the four plane-0 warps: bytes are expected before any copy lands
            bulk_g2s(w_row + (uint32_t)ws * W_BYTES, rowp + (size_t)p * 144, 144u, fw);
        };
        if (plane == 0)
            for (int p = 0; p < NW - 1 && p < nsb; ++p) fetch_block(p);
        for (int sb = 0; sb < nsb; ++sb) {
            const int ws = sb % NW;
            if (plane == 0 && sb + NW - 1 < nsb) fetch_block(sb + NW - 1);
            warp_wait(bar(BAR_FULL_W + ws), (uint32_t)((sb / NW) & 1), abort_flag, status);
            uint4 cur[9];
#pragma unroll
            for (int i = 0; i < 9; ++i) cur[i] = lds128(w_row + (uint32_t)ws * W_BYTES + 16u * i);
            warp_arrive(bar(BAR_EMPTY_W + ws));  // the bytes are in registers: the slot may be refilled
            const uint32_t s0 = cur[0].y, s1 = cur[0].z, s2 = cur[0].w;  // the 12 packed scale / min bytes
#pragma unroll
            for (int g = 0; g < NA; ++g) {
                warp_wait(bar(BAR_EMPTY_A + g), (uint32_t)((sb & 1) ^ 1), abort_flag, status);
                tc_fence_after();
                if (g == 0 && plane == 1) {
                    // A'' of the min term: dmin * m_j as fp16 pairs, hi in columns 0..7, lo in 8..15
                    const float dmin = smc_h2f((uint16_t)(cur[0].x >> 16));
                    uint32_t mh[4], ml[4];
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        int sc, ma, mb;
                        smc_k4_scale_min(s0, s1, s2, j, sc, ma);
                        smc_k4_scale_min(s0, s1, s2, j + 1, sc, mb);
                        const float pa = dmin * (float)ma, pb = dmin * (float)mb;
                        const __half ha = __float2half_rn(pa), hb = __float2half_rn(pb);
                        const __half2 hh = __halves2half2(ha, hb);
                        const __half2 ll = __halves2half2(__float2half_rn(pa - __half2float(ha)), __float2half_rn(pb - __half2float(hb)));
                        mh[j >> 1] = *reinterpret_cast<const uint32_t *>(&hh);
                        ml[j >> 1] = *reinterpret_cast<const uint32_t *>(&ll);
                    }
                    const uint32_t am = sbase + OFF_AUX + (uint32_t)(sb & 1) * AUX_BYTES + am_row;
                    sts128(am, mh[0], mh[1], mh[2], mh[3]);
                    sts128(am + 128u, ml[0], ml[1], ml[2], ml[3]);
                    fence_proxy_async();  // the tensor cores read this tile through the async proxy
                }
                int sc, mn;
                smc_k4_scale_min(s0, s1, s2, 2 * g + plane, sc, mn);
                // low nibble: (1024 + q) * sc - 1024 sc; high nibble: (1024 + 16 q) * sc / 16 - 64 sc; both exact
                const __half2 mul = plane ? __half2half2(__float2half_rn((float)sc * 0.0625f)) : __half2half2(__int2half_rn(sc));
                const __half2 off = __half2half2(__int2half_rn((plane ? -64 : -1024) * sc));
                const uint32_t mask = plane ? 0x00F000F0u : 0x000F000Fu;
                const uint32_t wq[8] = {cur[1 + 2 * g].x, cur[1 + 2 * g].y, cur[1 + 2 * g].z, cur[1 + 2 * g].w,
                                        cur[2 + 2 * g].x, cur[2 + 2 * g].y, cur[2 + 2 * g].z, cur[2 + 2 * g].w};
                // column c of the plane holds elements 2c, 2c + 1 of the sub-block = bytes 2c, 2c + 1 of the group
                uint32_t col[16];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    col[2 * c] = expand_half(wq[c], 0x4140u, mask, mul, off);
                    col[2 * c + 1] = expand_half(wq[c], 0x4342u, mask, mul, off);
                }
                tc_st16(a_lane + (uint32_t)g * 32u, col);
                tc_wait_st();
                tc_fence_before();
                warp_arrive(bar(BAR_FULL_A + g));
            }
        }
    } else {
        // ---------------- drain: thread = (TMEM lane = weight row, 64 of the 128 token columns)
        const int quarter = warp & 3, half = (warp - WARP_DRAIN0) >> 2;
        const int rl = quarter * 32 + lane;
        const uint8_t *rowp = raw + (size_t)(row0 + rl) * row_bytes;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)half * 64u;
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.f;
        for (int sb = 0; sb < nsb; ++sb) {
            const int buf = sb & 1;
            const float d = smc_h2f(smc_ldg_stream2(rowp + (size_t)sb * 144));
            warp_wait(bar(BAR_ACC_FULL + buf), (uint32_t)((sb >> 1) & 1), abort_flag, status);
            tc_fence_after();
            const uint32_t td = lane_base + COL_ACC_D + (uint32_t)buf * 128u;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float va[16];
                tc_ld16(td + (uint32_t)c * 16u, va);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[c * 16 + i] = fmaf(d, va[i], acc[c * 16 + i]);
            }
            tc_fence_before();
            warp_arrive(bar(BAR_ACC_EMPTY + buf));
        }
        // the commit that completed the last block also covers every min-term MMA
        const int t0 = tt * TN + half * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float vm[16];
            tc_ld16(lane_base + COL_ACC_M + (uint32_t)c * 16u, vm);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int t = t0 + c * 16 + i;
                if (t < M) out[(size_t)t * N + row0 + rl] = (acc[c * 16 + i] - vm[i]) * scale[t];
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace

bool smc_prefill_supported(const smc_weight *w, int M)
{
    return w->dtype == SMC_Q4_K && w->N % TM == 0 && w->K % 256 == 0 && M >= 1 && w->d_raw != nullptr;
}

// Scratch for the activation image, owned by the context and grown on demand (the first call of a larger
// shape allocates: make it outside stream capture).
static int ensure_scratch(smc_ctx *ctx, size_t bytes)
{
    if (ctx->prefill_cap >= bytes) return SMC_OK;
    if (ctx->d_prefill) {
        cudaDeviceSynchronize();
        cudaFree(ctx->d_prefill);
        ctx->d_prefill = nullptr, ctx->prefill_cap = 0;
    }
    SMC_CUDA(ctx, cudaMalloc(&ctx->d_prefill, bytes));
    ctx->prefill_cap = bytes;
    return SMC_OK;
}

// Q8_0 activation rows back to fp32 (x^ = d * q, exact: an 11-bit scale times an 8-bit code), four values per thread.
__global__ void __launch_bounds__(256) dequant_q8_rows_kernel(const int8_t *__restrict__ q, const float *__restrict__ d,
                                                              float *__restrict__ out, long long nquads)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= nquads) return;
    const char4 c = reinterpret_cast<const char4 *>(q)[t];
    const float dd = d[t >> 3];
    reinterpret_cast<float4 *>(out)[t] = make_float4(dd * (float)c.x, dd * (float)c.y, dd * (float)c.z, dd * (float)c.w);
}

// x: fp32 activations [M, K]; or, when `a` is given, the rows it holds: they are expanded to fp32 in the scratch first
// (their values d * q are exact in the fp16 pairs of the activation image, so the contraction sees exactly the
// quantised activations).
static int launch_prefill(smc_ctx *ctx, const float *x, const smc_q8act *a, const smc_weight *w, float *out, int M, cudaStream_t s,
                          bool scratch_locked = false)
{
    if (!smc_prefill_supported(w, M)) return smc_fail(ctx, SMC_E_UNSUPPORTED, "tensor-core matmul needs Q4_K, N %% 128 == 0, K %% 256 == 0");
    if (reinterpret_cast<uintptr_t>(x) & 15) return smc_fail(ctx, SMC_E_INVALID, "tensor-core matmul needs 16-byte aligned activations");
    const int N = w->N, K = w->K, ntt = (M + TN - 1) / TN, nsb = K / 256;
    const size_t img_halves = (size_t)ntt * TN * K * 2, mimg_halves = (size_t)ntt * nsb * 2 * TN * 16;
    const size_t scale_off = (img_halves + mimg_halves) * sizeof(__half);
    const size_t x_off = (scale_off + (size_t)ntt * TN * sizeof(float) + 255) & ~(size_t)255;
    const size_t bytes = x_off + (a ? (size_t)M * K * sizeof(float) : 0);
    if (scratch_locked) {  // the caller holds mu_scratch (its own scratch rows are the input)
        int rc = ensure_scratch(ctx, bytes);
        if (rc) return rc;
    } else {
        std::lock_guard<std::mutex> lock(ctx->mu_scratch);
        int rc = ensure_scratch(ctx, bytes);
        if (rc) return rc;
    }
    __half *img = reinterpret_cast<__half *>(ctx->d_prefill);
    __half *mimg = img + img_halves;
    float *scale = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ctx->d_prefill) + scale_off);
    if (a) {
        float *xd = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ctx->d_prefill) + x_off);
        const long long nquads = (long long)M * K / 4;
        dequant_q8_rows_kernel<<<(unsigned)((nquads + 255) / 256), 256, 0, s>>>(a->q, a->d, xd, nquads);
        x = xd;
    }
    prefill_scale_kernel<<<M, 256, 0, s>>>(x, M, K, scale);
    prefill_image_kernel<<<ntt * nsb, 256, 0, s>>>(x, M, K, scale, img, mimg);
    static bool attr_set = false;
    if (!attr_set) {
        SMC_CUDA(ctx, cudaFuncSetAttribute(prefill_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
        attr_set = true;
    }
    prefill_q4k_kernel<<<(N / TM) * ntt, THREADS, SMEM_BYTES, s>>>(w->d_raw, img, mimg, scale, out, N, K, M, ntt, ctx->d_status);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_launch_prefill_q4k(smc_ctx *ctx, const float *x, const smc_weight *w, float *out, int M, cudaStream_t s)
{
    return launch_prefill(ctx, x, nullptr, w, out, M, s);
}

// The same contraction over quantised activation rows (SMC_ACT_Q8 at prefill sizes): out = W . (d * q).
int smc_launch_prefill_q4k_q8(smc_ctx *ctx, const smc_q8act *a, const smc_weight *w, float *out, cudaStream_t s, bool scratch_locked)
{
    if (a->K != w->K) return smc_fail(ctx, SMC_E_INVALID, "tensor-core matmul: activations have K=%d, weight has K=%d", a->K, w->K);
    return launch_prefill(ctx, nullptr, a, w, out, a->M, s, scratch_locked);
}
