// Quantisers and layout kernels:
//   * run-time Q8_0 activation quantiser (QuantizedKVCache.QuantizeRowQ8_0,
//     SharpMind.Model/QuantizedKVCache.cs:191-223) writing the structure-of-arrays form the
//     integer GEMV kernels read;
//   * weight quantisers, bit-exact device forms of TensorQuantizer.WriteBlock (Q8_0,
//     SharpMind.Core/Quantization/TensorQuantizer.cs:80-144), WriteKQ4 and WriteKQ6
//     (TensorQuantizer.KQuant.cs:173-225, 303-376) -- they make the synthetic weights;
//   * the upload-time repack of Q8_0 tensors into 16-byte-aligned planes and of Q6_K tensors into 1680-byte units.
// All arithmetic that decides a code or a scale uses explicit round-to-nearest intrinsics.
#include "smc_common.cuh"

namespace {

// ---------------------------------------------------------------------------- activations -> Q8_0
// One warp per 32-element block; x [M][K], K % 32 == 0.
// With `up` the quantised value is SiLU(x) * up (x / (1 + exp(-x)) * up in the arithmetic of the stand-alone gate
// kernel), x and up being rows of `ld` floats of which the first K are used: the FFN's gate step and the
// quantisation of the down projection's input in one pass, without the fp32 product going through memory.
__global__ void __launch_bounds__(256) quantize_q8_kernel(const float *__restrict__ x, const float *__restrict__ up, int K, int ld,
                                                          int8_t *__restrict__ q,
                                                          float *__restrict__ d, uint16_t *__restrict__ dbits,
                                                          float *__restrict__ sd, int16_t *__restrict__ s16,
                                                          long long nblocks)
{
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31;
    long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    const int bpr = K / 32;  // blocks per row
    for (; blk < nblocks; blk += stride) {
        float v;
        if (up) {
            const long long at = (blk / bpr) * ld + (blk % bpr) * 32 + lane;
            const float g = x[at];
            v = __fdiv_rn(g, 1.0f + expf(-g)) * up[at];
        } else {
            v = x[blk * 32 + lane];
        }
        float amax = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        float scale = __fdiv_rn(amax, 127.0f);
        if (amax == 0.0f) scale = 1.0f;
        int qi = __float2int_rn(__fdiv_rn(v, scale));  // round half to even, like MathF.Round(x)
        qi = max(-128, min(127, qi));
        q[blk * 32 + lane] = (int8_t)qi;
        int s = qi;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        int total = s + __shfl_xor_sync(0xffffffffu, s, 16);
        if ((lane & 15) == 0) s16[blk * 2 + (lane >> 4)] = (int16_t)s;
        if (lane == 0) {
            __half h = __float2half_rn(scale);
            float df = __half2float(h);
            d[blk] = df;
            dbits[blk] = __half_as_ushort(h);
            sd[blk] = df * (float)total;
        }
    }
}

// The same with 16-byte accesses: eight consecutive threads hold one block (four values each), a warp four blocks.
// Same arithmetic per value, block and half block, hence the same bytes; rows and `ld` must be multiples of four floats
// on 16-byte aligned pointers.  (One lane per value made a 2048 x 2048 batch a 32 us launch for 16 MB.)
__global__ void __launch_bounds__(256) quantize_q8_vec_kernel(const float *__restrict__ x, const float *__restrict__ up, int K, int ld,
                                                              int8_t *__restrict__ q, float *__restrict__ d,
                                                              uint16_t *__restrict__ dbits, float *__restrict__ sd,
                                                              int16_t *__restrict__ s16, long long nquads)
{
    smc_grid_dep_sync();
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int qpr = K / 4;  // quads per row
    // whole warps stay in the loop (the shuffles name all lanes); a group of eight threads is live or not as one
    for (long long base = (long long)blockIdx.x * blockDim.x; base < nquads; base += stride) {
        const long long t = base + threadIdx.x;
        const bool live = t < nquads;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            const long long at = up ? (t / qpr) * ld + (t % qpr) * 4 : t * 4;
            v = *reinterpret_cast<const float4 *>(x + at);
            if (up) {
                const float4 u = *reinterpret_cast<const float4 *>(up + at);
                v.x = __fdiv_rn(v.x, 1.0f + expf(-v.x)) * u.x, v.y = __fdiv_rn(v.y, 1.0f + expf(-v.y)) * u.y;
                v.z = __fdiv_rn(v.z, 1.0f + expf(-v.z)) * u.z, v.w = __fdiv_rn(v.w, 1.0f + expf(-v.w)) * u.w;
            }
        }
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        float scale = __fdiv_rn(amax, 127.0f);
        if (amax == 0.0f) scale = 1.0f;
        const int q0 = max(-128, min(127, __float2int_rn(__fdiv_rn(v.x, scale))));
        const int q1 = max(-128, min(127, __float2int_rn(__fdiv_rn(v.y, scale))));
        const int q2 = max(-128, min(127, __float2int_rn(__fdiv_rn(v.z, scale))));
        const int q3 = max(-128, min(127, __float2int_rn(__fdiv_rn(v.w, scale))));
        int sum = q0 + q1 + q2 + q3;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // half block
        const int total = sum + __shfl_xor_sync(0xffffffffu, sum, 4);
        if (live) {
            const long long blk = t >> 3;
            reinterpret_cast<uint32_t *>(q)[t] =
                (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
            if ((t & 3) == 0) s16[blk * 2 + ((t >> 2) & 1)] = (int16_t)sum;
            if ((t & 7) == 0) {
                const __half h = __float2half_rn(scale);
                const float df = __half2float(h);
                d[blk] = df;
                dbits[blk] = __half_as_ushort(h);
                sd[blk] = df * (float)total;
            }
        }
    }
}

// fp32 rows as three Q8_0-shaped "digit" planes: per 32-element block x = d1 q1 + d2 q2 + d3 q3 + r with d1 = amax / 127,
// d2 = d1 / 254, d3 = d2 / 254 and |r| <= d3 / 2 = amax / 1.6e7, i.e. the activations to fp32 accuracy as int8 operands.
// The integer kernels run once per plane and the three results add up to the fp32-activation product (SMC_ACT_F32 at
// prefill sizes over formats without a tcgen05 kernel).  Eight threads per block, four values each.
struct DigitPlane {
    int8_t *q;
    float *d, *sd;
    int16_t *s16;
};
__global__ void __launch_bounds__(256) quantize_q8_digits_kernel(const float *__restrict__ x, DigitPlane p0, DigitPlane p1, DigitPlane p2,
                                                                 long long nquads)
{
    smc_grid_dep_sync();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long base = (long long)blockIdx.x * blockDim.x; base < nquads; base += stride) {
        const long long t = base + threadIdx.x;
        const bool live = t < nquads;  // uniform over each group of eight threads
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            const float4 f = *reinterpret_cast<const float4 *>(x + t * 4);
            v[0] = f.x, v[1] = f.y, v[2] = f.z, v[3] = f.w;
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        float d = __fdiv_rn(amax, 127.0f);
        if (!(amax > 0.0f) || !(amax < INFINITY)) d = 1.0f;
        const DigitPlane planes[3] = {p0, p1, p2};
#pragma unroll
        for (int pl = 0; pl < 3; ++pl) {
            int q[4], sum = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q[i] = max(-127, min(127, __float2int_rn(__fdiv_rn(v[i], d))));
                v[i] = fmaf(-d, (float)q[i], v[i]);  // what this digit leaves
                sum += q[i];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // half block
            const int total = sum + __shfl_xor_sync(0xffffffffu, sum, 4);
            if (live) {
                const long long blk = t >> 3;
                reinterpret_cast<uint32_t *>(planes[pl].q)[t] =
                    (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
                if ((t & 3) == 0) planes[pl].s16[blk * 2 + ((t >> 2) & 1)] = (int16_t)sum;
                if ((t & 7) == 0) {
                    planes[pl].d[blk] = d;
                    planes[pl].sd[blk] = d * (float)total;
                }
            }
            d = __fdiv_rn(d, 254.0f);
        }
    }
}

// ---------------------------------------------------------------------------- weights -> Q8_0
__global__ void __launch_bounds__(256) wq_q8_0_kernel(const float *__restrict__ v, uint8_t *__restrict__ out,
                                                      long long nblocks)
{
    const int lane = threadIdx.x & 31;
    long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (; blk < nblocks; blk += stride) {
        float x = v[blk * 32 + lane];
        float amax = fabsf(x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        uint8_t *o = out + blk * 34;
        if (amax == 0.0f) {
            if (lane == 0) o[0] = 0, o[1] = 0;
            o[2 + lane] = 0;
            continue;
        }
        float d = __fdiv_rn(amax, 127.0f);
        int qi = (int)roundf(__fdiv_rn(x, d));  // MidpointRounding.AwayFromZero
        qi = max(-128, min(127, qi));
        o[2 + lane] = (uint8_t)(int8_t)qi;
        if (lane == 0) {
            // block offsets are even, so the scale goes out as one 16-bit store
            *reinterpret_cast<uint16_t *>(o) = __half_as_ushort(__float2half_rn(d));
        }
    }
}

// ---------------------------------------------------------------------------- weights -> Q4_K
// One warp per 256-element block.  Lane l owns elements 64g + l and 64g + 32 + l (g = 0..3), i.e.
// both nibbles of byte qs[32g + l]; sub-block 2g holds the first, 2g + 1 the second.
__global__ void __launch_bounds__(256) wq_q4_K_kernel(const float *__restrict__ v, uint8_t *__restrict__ out,
                                                      long long nblocks)
{
    const int lane = threadIdx.x & 31;
    long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (; blk < nblocks; blk += stride) {
        const float *p = v + blk * 256;
        uint8_t *o = out + blk * 144;
        float e[8];  // e[2g] = element 64g + l (sub-block 2g), e[2g+1] = 64g + 32 + l (sub-block 2g+1)
        float amax = 0.f;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            e[2 * g] = p[64 * g + lane];
            e[2 * g + 1] = p[64 * g + 32 + lane];
            amax = fmaxf(amax, fmaxf(fabsf(e[2 * g]), fabsf(e[2 * g + 1])));
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
        if (amax == 0.0f) {
            // all-zero block encodes as 144 zero bytes
            for (int i = lane; i < 144; i += 32) o[i] = 0;
            continue;
        }
        float step = __fdiv_rn(amax, 63.0f);
        int sc[8], mn[8];
        uint32_t code[8];
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
            float gmn = e[sb], gmx = e[sb];
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) {
                gmn = fminf(gmn, __shfl_xor_sync(0xffffffffu, gmn, s));
                gmx = fmaxf(gmx, __shfl_xor_sync(0xffffffffu, gmx, s));
            }
            float range = __fsub_rn(gmx, gmn);
            mn[sb] = max(0, min(63, (int)roundf(__fdiv_rn(-gmn, step))));
            if (range <= 0.0f) {
                sc[sb] = 0;
                code[sb] = 0;
                continue;
            }
            sc[sb] = max(1, min(63, (int)roundf(__fdiv_rn(range, __fmul_rn(15.0f, step)))));
            float scF = __fmul_rn((float)sc[sb], step);
            float num = __fadd_rn(e[sb], __fmul_rn((float)mn[sb], step));
            code[sb] = (uint32_t)max(0, min(15, (int)roundf(__fdiv_rn(num, scF))));
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) o[16 + 32 * g + lane] = (uint8_t)(code[2 * g] | (code[2 * g + 1] << 4));
        if (lane == 0) {
            uint16_t hb = __half_as_ushort(__float2half_rn(step));
            reinterpret_cast<uint16_t *>(o)[0] = hb;  // d
            reinterpret_cast<uint16_t *>(o)[1] = hb;  // dmin
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o[4 + j] = (uint8_t)((sc[j] & 0x3F) | ((sc[4 + j] >> 4) << 6));
                o[8 + j] = (uint8_t)((mn[j] & 0x3F) | ((mn[4 + j] >> 4) << 6));
                o[12 + j] = (uint8_t)((sc[4 + j] & 0x0F) | ((mn[4 + j] & 0x0F) << 4));
            }
        }
    }
}

// ---------------------------------------------------------------------------- weights -> Q6_K
// One warp per block.  Lane l owns elements 128h + 32c + l (h = 0..1, c = 0..3): bytes ql[64h + l]
// (c = 0 low, c = 2 high nibble), ql[64h + 32 + l] (c = 1 low, c = 3 high) and qh[32h + l].
__global__ void __launch_bounds__(256) wq_q6_K_kernel(const float *__restrict__ v, uint8_t *__restrict__ out,
                                                      long long nblocks)
{
    const int lane = threadIdx.x & 31;
    long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (; blk < nblocks; blk += stride) {
        const float *p = v + blk * 256;
        uint8_t *o = out + blk * 210;
        float e[8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            e[i] = p[32 * i + lane];  // i = 4h + c
            amax = fmaxf(amax, fabsf(e[i]));
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
        if (amax == 0.0f) {
            for (int i = lane; i < 210; i += 32) o[i] = 0;
            continue;
        }
        float d = __fdiv_rn(amax, 4064.0f);
        int code[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // group = 16 consecutive elements = lanes (l & 16) .. +15 of column i
            float gmx = fabsf(e[i]);
#pragma unroll
            for (int s = 8; s > 0; s >>= 1) gmx = fmaxf(gmx, __shfl_xor_sync(0xffffffffu, gmx, s));
            int scale = gmx == 0.0f ? 0 : max(1, min(127, (int)roundf(__fdiv_rn(gmx, __fmul_rn(32.0f, d)))));
            if ((lane & 15) == 0) o[192 + 2 * i + (lane >> 4)] = (uint8_t)(int8_t)scale;
            float scf = __fmul_rn(d, (float)scale);
            code[i] = gmx == 0.0f ? 32 : max(0, min(63, (int)roundf(__fdiv_rn(e[i], scf)) + 32));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int *c = code + 4 * h;
            o[64 * h + lane] = (uint8_t)((c[0] & 0x0F) | ((c[2] & 0x0F) << 4));
            o[64 * h + 32 + lane] = (uint8_t)((c[1] & 0x0F) | ((c[3] & 0x0F) << 4));
            o[128 + 32 * h + lane] =
                (uint8_t)(((c[0] >> 4) & 3) | (((c[1] >> 4) & 3) << 2) | (((c[2] >> 4) & 3) << 4) | (((c[3] >> 4) & 3) << 6));
        }
        if (lane == 0) {
            *reinterpret_cast<uint16_t *>(o + 208) = __half_as_ushort(__float2half_rn(d));
        }
    }
}

// ---------------------------------------------------------------------------- repack
__global__ void repack_q8_0_kernel(const uint8_t *__restrict__ raw, int8_t *__restrict__ qs, __half *__restrict__ d,
                                   long long nblocks)
{
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; t < nblocks * 32; t += stride) {
        long long blk = t >> 5;
        int i = (int)(t & 31);
        const uint8_t *b = raw + blk * 34;
        qs[t] = (int8_t)b[2 + i];
        if (i == 0) d[blk] = __ushort_as_half((uint16_t)(b[0] | (b[1] << 8)));
    }
}

// GGUF Q6_K blocks -> the unit layout of smc_common.cuh.  One thread per (block, half h, byte l of the 32-element
// columns): it forms the four six-bit codes of elements 128h + 32c + l (c = 0..3, as VecDotQ6K_Scalar reads them,
// QuantizationKernels.Q6.cs:28-41) and stores the X, Y, Z bytes of its lane slot; the first threads of a block also
// move its scales and d.
__global__ void repack_q6_K_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ units, long long nblocks)
{
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; t < nblocks * 64; t += stride) {
        const long long blk = t >> 6;
        const int h = (int)(t >> 5) & 1, l = (int)(t & 31);
        const uint8_t *b = raw + blk * 210;
        const uint32_t la = b[64 * h + l], lb = b[64 * h + 32 + l], hh = b[128 + 32 * h + l];
        const uint32_t c0 = (la & 0x0F) | ((hh & 3) << 4), c1 = (lb & 0x0F) | (((hh >> 2) & 3) << 4);
        const uint32_t c2 = (la >> 4) | (((hh >> 4) & 3) << 4), c3 = (lb >> 4) | (((hh >> 6) & 3) << 4);
        uint8_t *slot = units + smc_q6u_slot((size_t)blk, h, l >> 4) + (l & 15);
        slot[0] = (uint8_t)(c0 | ((c3 & 3) << 6));
        slot[SMC_Q6U_Y] = (uint8_t)(c1 | (((c3 >> 2) & 3) << 6));
        slot[SMC_Q6U_Z] = (uint8_t)(c2 | (((c3 >> 4) & 3) << 6));
        const int i = (int)(t & 63);
        if (i < 16) units[smc_q6u_scales((size_t)blk) + i] = b[192 + i];
        if (i == 16) *reinterpret_cast<uint16_t *>(units + smc_q6u_d((size_t)blk)) = (uint16_t)(b[208] | (b[209] << 8));
    }
}

int grid_for(long long work_items, int per_cta, int cap)
{
    long long g = (work_items + per_cta - 1) / per_cta;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

int smc_q8act_alloc(smc_ctx *ctx, int max_rows, int max_k, smc_q8act **out)
{
    if (max_rows <= 0 || max_k <= 0 || max_k % 32) return smc_fail(ctx, SMC_E_INVALID, "q8act: bad capacity %d x %d", max_rows, max_k);
    smc_q8act *a = new smc_q8act();
    a->max_rows = max_rows;
    a->max_k = max_k;
    size_t n = (size_t)max_rows * max_k, nb = n / 32;
    cudaError_t e = cudaMalloc(&a->q, n);
    if (e == cudaSuccess) e = cudaMalloc(&a->d, nb * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&a->dbits, nb * sizeof(uint16_t));
    if (e == cudaSuccess) e = cudaMalloc(&a->sd, nb * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&a->s16, nb * 2 * sizeof(int16_t));
    if (e != cudaSuccess) {
        smc_q8act_free(a);
        return smc_fail(ctx, SMC_E_CUDA, "q8act allocation failed: %s", cudaGetErrorString(e));
    }
    *out = a;
    return SMC_OK;
}

void smc_q8act_free(smc_q8act *a)
{
    if (!a) return;
    cudaFree(a->q);
    cudaFree(a->d);
    cudaFree(a->dbits);
    cudaFree(a->sd);
    cudaFree(a->s16);
    delete a;
}

int smc_launch_quantize_q8(smc_ctx *ctx, const float *x, int M, int K, smc_q8act *a, cudaStream_t s)
{
    if (K % 32) return smc_fail(ctx, SMC_E_UNSUPPORTED, "Q8 activations need K %% 32 == 0 (K = %d)", K);
    if (M > a->max_rows || K > a->max_k || (size_t)M * K > (size_t)a->max_rows * a->max_k)
        return smc_fail(ctx, SMC_E_INVALID, "q8act buffer %d x %d too small for %d x %d", a->max_rows, a->max_k, M, K);
    a->M = M;
    a->K = K;
    long long nblocks = (long long)M * K / 32;
    if (nblocks >= 64 && (reinterpret_cast<uintptr_t>(x) & 15) == 0)  // batches: 16-byte accesses (one block is a single warp's work either way)
        smc_launch_dep(ctx->use_pdl, quantize_q8_vec_kernel, dim3(grid_for(nblocks * 8, 256, ctx->sm_count * 8)), dim3(256), 0, s, x,
                       (const float *)nullptr, K, K, a->q, a->d, a->dbits, a->sd, a->s16, nblocks * 8);
    else
        smc_launch_dep(ctx->use_pdl, quantize_q8_kernel, dim3(grid_for(nblocks, 8, ctx->sm_count * 8)), dim3(256), 0, s, x,
                       (const float *)nullptr, K, K, a->q, a->d, a->dbits, a->sd, a->s16, nblocks);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// x [M, K] fp32 -> three digit planes stacked as 3 M rows of `a` (plane p in rows p M .. p M + M - 1), so that one
// several-row matmul over `a` reads the weights once for all three; their fp16 scale bits are not written (the
// integer kernels read the fp32 scales).
int smc_launch_quantize_q8_digits(smc_ctx *ctx, const float *x, int M, int K, smc_q8act *a, cudaStream_t s)
{
    if (K % 32) return smc_fail(ctx, SMC_E_UNSUPPORTED, "Q8 activations need K %% 32 == 0 (K = %d)", K);
    if ((size_t)3 * M * K > (size_t)a->max_rows * a->max_k)
        return smc_fail(ctx, SMC_E_INVALID, "q8act buffer %d x %d too small for %d x %d", a->max_rows, a->max_k, 3 * M, K);
    a->M = 3 * M, a->K = K;
    const size_t n = (size_t)M * K, nb = n / 32;
    DigitPlane p[3];
    for (size_t i = 0; i < 3; ++i) p[i] = DigitPlane{a->q + i * n, a->d + i * nb, a->sd + i * nb, a->s16 + i * nb * 2};
    const long long nquads = (long long)n / 4;
    smc_launch_dep(ctx->use_pdl, quantize_q8_digits_kernel, dim3(grid_for(nquads, 256, ctx->sm_count * 8)), dim3(256), 0, s, x, p[0], p[1],
                   p[2], nquads);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// out = (y[0] + y[1]) + y[2] over three stacked [n] results
__global__ void __launch_bounds__(256) sum3_kernel(const float *__restrict__ y, float *__restrict__ out, long long n)
{
    smc_grid_dep_sync();
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = (y[i] + y[n + i]) + y[2 * n + i];
}
int smc_launch_sum3(smc_ctx *ctx, const float *y, float *out, long long n, cudaStream_t s)
{
    smc_launch_dep(ctx->use_pdl, sum3_kernel, dim3(grid_for(n, 256, ctx->sm_count * 8)), dim3(256), 0, s, y, out, n);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// Rows of SiLU(gate) * up, quantised: gate and up are [M] rows of `ld` floats, K of them used.
int smc_launch_swiglu_quantize_q8(smc_ctx *ctx, const float *gate, const float *up, int M, int K, int ld, smc_q8act *a,
                                  cudaStream_t s)
{
    if (K % 32) return smc_fail(ctx, SMC_E_UNSUPPORTED, "Q8 activations need K %% 32 == 0 (K = %d)", K);
    if (M > a->max_rows || K > a->max_k || (size_t)M * K > (size_t)a->max_rows * a->max_k)
        return smc_fail(ctx, SMC_E_INVALID, "q8act buffer %d x %d too small for %d x %d", a->max_rows, a->max_k, M, K);
    a->M = M;
    a->K = K;
    long long nblocks = (long long)M * K / 32;
    if (nblocks >= 64 && ld % 4 == 0 && ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) & 15) == 0)
        smc_launch_dep(ctx->use_pdl, quantize_q8_vec_kernel, dim3(grid_for(nblocks * 8, 256, ctx->sm_count * 8)), dim3(256), 0, s, gate, up, K,
                       ld, a->q, a->d, a->dbits, a->sd, a->s16, nblocks * 8);
    else
        smc_launch_dep(ctx->use_pdl, quantize_q8_kernel, dim3(grid_for(nblocks, 8, ctx->sm_count * 8)), dim3(256), 0, s, gate, up, K, ld,
                       a->q, a->d, a->dbits, a->sd, a->s16, nblocks);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_launch_quantize_weights(smc_ctx *ctx, int dtype, const float *v, int64_t n, void *raw, cudaStream_t s)
{
    const int be = dtype == SMC_Q8_0 ? 32 : 256;
    if (dtype != SMC_Q8_0 && dtype != SMC_Q4_K && dtype != SMC_Q6_K)
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "no quantiser for dtype %d", dtype);
    if (n < 0 || n % be)
        return smc_fail(ctx, SMC_E_INVALID, "cannot quantise %lld values: length must be a multiple of %d", (long long)n, be);
    if (n == 0) return SMC_OK;
    long long nblocks = n / be;
    int grid = grid_for(nblocks, 8, ctx->sm_count * 16);
    uint8_t *o = static_cast<uint8_t *>(raw);
    if (dtype == SMC_Q8_0) wq_q8_0_kernel<<<grid, 256, 0, s>>>(v, o, nblocks);
    else if (dtype == SMC_Q4_K) wq_q4_K_kernel<<<grid, 256, 0, s>>>(v, o, nblocks);
    else wq_q6_K_kernel<<<grid, 256, 0, s>>>(v, o, nblocks);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// Builds the planes of `w` from w->d_raw.  Planes are allocated here; d_raw is left to the caller.
int smc_launch_repack(smc_ctx *ctx, smc_weight *w, cudaStream_t s)
{
    if (w->dtype == SMC_Q8_0) {
        long long nblocks = (long long)w->N * (w->K / 32);
        SMC_CUDA(ctx, cudaMalloc(&w->q8_qs, (size_t)nblocks * 32));
        SMC_CUDA(ctx, cudaMalloc(&w->q8_d, (size_t)nblocks * sizeof(__half)));
        repack_q8_0_kernel<<<grid_for(nblocks * 32, 256, ctx->sm_count * 16), 256, 0, s>>>(w->d_raw, w->q8_qs, w->q8_d,
                                                                                          nblocks);
        SMC_LAUNCH_CHECK(ctx);
    } else if (w->dtype == SMC_Q6_K) {
        long long nblocks = (long long)w->N * w->K / 256;
        SMC_CUDA(ctx, cudaMalloc(&w->q6u, smc_q6u_bytes((size_t)nblocks)));
        if (nblocks % 8)  // the blocks missing from the last unit read as zero weights
            SMC_CUDA(ctx, cudaMemsetAsync(w->q6u + smc_q6u_bytes((size_t)nblocks) - SMC_Q6U_BYTES, 0, SMC_Q6U_BYTES, s));
        repack_q6_K_kernel<<<grid_for(nblocks * 64, 256, ctx->sm_count * 16), 256, 0, s>>>(w->d_raw, w->q6u, nblocks);
        SMC_LAUNCH_CHECK(ctx);
    }
    return SMC_OK;
}
