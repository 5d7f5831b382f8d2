// fp32 elementwise / reduction ops the decoder runs around the quantized matmuls.  All are bound
// by one read and one write of their operands; rows are mapped to a warp (short rows) or a CTA
// (long rows), reductions use warp shuffles plus one shared-memory hop, loads are 128-bit where
// the row length allows.
//
// References (SharpMind repository paths):
//   RMSNorm   SharpMind.Model/Layers/NormKernels.cs:13-60, NormLayer.cs:42-70
//   SwiGLU    SharpMind.Core/Activations/ActivationKernels.cs:194-201 (scalar form: g/(1+exp(-g))*u)
//   SiLU      ActivationKernels.cs:161-168
//   softmax   ActivationKernels.cs:316-348 (max, exp(x-max), normalise)
//   RoPE      SharpMind.Core/Embeddings/RoPE.cs:168-259
//   add       SharpMind.Core/Tensors/Tensor.cs:328-332
//   argmax    SharpMind.Inference/Sampler.cs:50-58
//   embedding SharpMind.Core/Embeddings/EmbeddingTable.cs:87-116 over ReadQ8_0_Scalar
#include <math.h>

#include <vector>

#include "smc_common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum, result broadcast to every thread. `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float *red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // protect `red` against a previous use
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : 0.f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float *red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = lane < nw ? red[lane] : -INFINITY;
    return warp_max(t);
}

__device__ __forceinline__ float silu_ref(float g)
{
    // x / (1 + exp(-x)), division and addition rounded like the scalar reference
    return __fdiv_rn(g, 1.0f + expf(-g));
}

// ---------------------------------------------------------------------------- RMSNorm
// A warp per row for short rows, a CTA per row for long ones.  `out` may alias `x` (in-place
// final norm), so neither is declared restrict.
__global__ void __launch_bounds__(256) rmsnorm_warp_kernel(const float *x, const float *__restrict__ w, float *out,
                                                           int rows, int n, float eps)
{
    smc_grid_dep_sync();
    const int lane = threadIdx.x & 31;
    int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float *p = x + (size_t)row * n;
    float *o = out + (size_t)row * n;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    float inv = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(ss, (float)n) + eps));
    for (int i = lane; i < n; i += 32) o[i] = (p[i] * inv) * w[i];
}

__global__ void __launch_bounds__(256) rmsnorm_cta_kernel(const float *x, const float *__restrict__ w, float *out, int n,
                                                          float eps, int vec)
{
    __shared__ float red[32];
    smc_grid_dep_sync();
    const float *p = x + (size_t)blockIdx.x * n;
    float *o = out + (size_t)blockIdx.x * n;
    float ss = 0.f;
    if (vec) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            float4 v = p4[i];
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(p[i], p[i], ss);
    }
    ss = block_sum(ss, red);
    float inv = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(ss, (float)n) + eps));
    if (vec) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p);
        const float4 *w4 = reinterpret_cast<const float4 *>(w);
        float4 *o4 = reinterpret_cast<float4 *>(o);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            float4 v = p4[i], g = __ldg(w4 + i);
            o4[i] = make_float4((v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = (p[i] * inv) * w[i];
    }
}

// x[row] += y[row] (Tensor.AddInPlace), then out[row] = RMSNorm(x[row]) * w: the residual add and the norm that
// follows it in a decoder block as one pass.  Arithmetic and summation order are those of add_kernel followed by
// rmsnorm_cta_kernel, so the fused and the separate forms give the same bits.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(float *x, const float *__restrict__ y, const float *__restrict__ w,
                                                          float *out, int n, float eps, int vec)
{
    __shared__ float red[32];
    smc_grid_dep_sync();
    float *p = x + (size_t)blockIdx.x * n;
    const float *q = y + (size_t)blockIdx.x * n;
    float *o = out + (size_t)blockIdx.x * n;
    float ss = 0.f;
    if (vec) {
        float4 *p4 = reinterpret_cast<float4 *>(p);
        const float4 *q4 = reinterpret_cast<const float4 *>(q);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            const float4 a = p4[i], b = q4[i];
            const float4 v = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
            p4[i] = v;
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = p[i] + q[i];
            p[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(ss, (float)n) + eps));
    // each thread re-reads exactly the elements it wrote above
    if (vec) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p);
        const float4 *w4 = reinterpret_cast<const float4 *>(w);
        float4 *o4 = reinterpret_cast<float4 *>(o);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            const float4 v = p4[i], g = __ldg(w4 + i);
            o4[i] = make_float4((v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = (p[i] * inv) * w[i];
    }
}

// The same pass with the normalised row leaving as Q8_0 activations (QuantizeRowQ8_0's rules, the structure-of-arrays
// form the integer matmuls read) instead of, or besides, fp32: in a block of several rows with quantised activations
// the norm's output is only ever read by the quantiser, so the fp32 row need not go through memory.  n % 32 == 0 and
// 16-byte aligned rows; eight consecutive threads hold one 32-element block (four values each).  Values, scales and
// sums are bit for bit those of add_rmsnorm_kernel followed by the row quantiser.
__global__ void __launch_bounds__(256) add_rmsnorm_q8_kernel(float *x, const float *__restrict__ y, const float *__restrict__ w,
                                                             float *out, int n, float eps, int8_t *__restrict__ q,
                                                             float *__restrict__ d, uint16_t *__restrict__ dbits,
                                                             float *__restrict__ sd, int16_t *__restrict__ s16)
{
    __shared__ float red[32];
    smc_grid_dep_sync();
    float4 *p4 = reinterpret_cast<float4 *>(x + (size_t)blockIdx.x * n);
    const int n4 = n / 4;
    float ss = 0.f;
    if (y) {
        const float4 *q4 = reinterpret_cast<const float4 *>(y + (size_t)blockIdx.x * n);
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 a = p4[i], b = q4[i];
            const float4 v = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
            p4[i] = v;
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 v = p4[i];
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(ss, (float)n) + eps));
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    const size_t blk0 = (size_t)blockIdx.x * (n / 32);
    for (int i0 = 0; i0 < n4; i0 += blockDim.x) {  // whole warps stay in the loop: the shuffles below name all lanes
        const int i = i0 + threadIdx.x;
        const bool live = i < n4;                   // uniform over each group of eight threads (n4 % 8 == 0)
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            const float4 a = p4[i], g = __ldg(w4 + i);
            v = make_float4((a.x * inv) * g.x, (a.y * inv) * g.y, (a.z * inv) * g.z, (a.w * inv) * g.w);
            if (out) reinterpret_cast<float4 *>(out + (size_t)blockIdx.x * n)[i] = v;
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
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);                 // half block (16 values)
        const int total = sum + __shfl_xor_sync(0xffffffffu, sum, 4);
        if (live) {
            const size_t blk = blk0 + (size_t)(i >> 3);
            reinterpret_cast<uint32_t *>(q + (size_t)blockIdx.x * n)[i] =
                (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
            if ((i & 3) == 0) s16[blk * 2 + ((i >> 2) & 1)] = (int16_t)sum;
            if ((i & 7) == 0) {
                const __half h = __float2half_rn(scale);
                const float df = __half2float(h);
                d[blk] = df;
                dbits[blk] = __half_as_ushort(h);
                sd[blk] = df * (float)total;
            }
        }
    }
}

__global__ void rmsnorm_row_kernel(const float *__restrict__ src, const float *__restrict__ w, float *__restrict__ dst,
                                   int n, float rms_inv)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = (src[i] * rms_inv) * w[i];
}

// ---------------------------------------------------------------------------- SwiGLU / SiLU
__global__ void __launch_bounds__(256) swiglu_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                     float *__restrict__ dst, int rows, int F, int ld, int vec)
{
    smc_grid_dep_sync();
    long long total = (long long)rows * F;
    long long stride = (long long)gridDim.x * blockDim.x;
    if (vec) {
        long long total4 = total / 4;
        int F4 = F / 4;
        for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total4; t += stride) {
            long long r = t / F4;
            int c = (int)(t % F4) * 4;
            float4 g = *reinterpret_cast<const float4 *>(gate + r * ld + c);
            float4 u = *reinterpret_cast<const float4 *>(up + r * ld + c);
            float4 o = make_float4(silu_ref(g.x) * u.x, silu_ref(g.y) * u.y, silu_ref(g.z) * u.z, silu_ref(g.w) * u.w);
            *reinterpret_cast<float4 *>(dst + r * F + c) = o;
        }
    } else {
        for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
            long long r = t / F;
            int c = (int)(t % F);
            dst[t] = silu_ref(gate[r * ld + c]) * up[r * ld + c];
        }
    }
}

__global__ void __launch_bounds__(256) silu_kernel(const float *__restrict__ src, float *__restrict__ dst, long long n)
{
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += stride) dst[t] = silu_ref(src[t]);
}

// ---------------------------------------------------------------------------- softmax
// One CTA per row.  Pass 1 keeps a running (max, sum) per thread (online softmax), pass 2 re-reads
// the row -- it was just streamed, so rows up to the L2 size come back from L2 -- and writes
// exp(x - max) / sum.  HBM traffic: one read and one write per element.
__global__ void __launch_bounds__(1024) softmax_kernel(const float *__restrict__ src, float *__restrict__ dst, int n, int vec)
{
    __shared__ float red[32];
    const float *p = src + (size_t)blockIdx.x * n;
    float *o = dst + (size_t)blockIdx.x * n;
    float mx = -INFINITY, sum = 0.f;
    if (vec) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            float4 v = p4[i];
            float m4 = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
            if (m4 > mx) {
                sum *= expf(mx - m4);
                mx = m4;
            }
            if (mx > -INFINITY) sum += (expf(v.x - mx) + expf(v.y - mx)) + (expf(v.z - mx) + expf(v.w - mx));
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            float v = p[i];
            if (v > mx) {
                sum *= expf(mx - v);
                mx = v;
            }
            if (mx > -INFINITY) sum += expf(v - mx);
        }
    }
    float gmax = block_max(mx, red);
    float part = (mx == -INFINITY) ? 0.f : sum * expf(mx - gmax);
    float total = block_sum(part, red);
    float inv = __fdiv_rn(1.0f, total);
    if (vec) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p);
        float4 *o4 = reinterpret_cast<float4 *>(o);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            float4 v = p4[i];
            o4[i] = make_float4(expf(v.x - gmax) * inv, expf(v.y - gmax) * inv, expf(v.z - gmax) * inv,
                                expf(v.w - gmax) * inv);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = expf(p[i] - gmax) * inv;
    }
}

// ---------------------------------------------------------------------------- RoPE
// One thread per rotated pair.
__global__ void __launch_bounds__(256) rope_kernel(float *__restrict__ x, int seq, int heads, int headDim, int ropeDim,
                                                   int posOffset, const float *__restrict__ cosT,
                                                   const float *__restrict__ sinT, int neox)
{
    const int pairs = ropeDim / 2;
    long long total = (long long)seq * heads * pairs;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        int i = (int)(t % pairs);
        long long sh = t / pairs;  // s * heads + h
        int s = (int)(sh / heads);
        float c = __ldg(cosT + (size_t)(posOffset + s) * pairs + i);
        float sn = __ldg(sinT + (size_t)(posOffset + s) * pairs + i);
        float *p = x + sh * headDim;
        int ia = neox ? i : 2 * i, ib = neox ? i + pairs : 2 * i + 1;
        float a = p[ia], b = p[ib];
        p[ia] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
        p[ib] = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn));
    }
}

// Four pairs per thread with 16-byte accesses (ropeDim % 8 == 0, 16-byte aligned rows): NEOX pairing rotates
// (d .. d+3) against (d+half .. d+half+3), adjacent pairing the two float4 that hold pairs 4q .. 4q+3.  The arithmetic
// per pair is that of rope_kernel (unfused products, one add), so both give the same bits.
__global__ void __launch_bounds__(256) rope_vec_kernel(float *__restrict__ x, int seq, int heads, int headDim, int ropeDim,
                                                       int posOffset, const float *__restrict__ cosT,
                                                       const float *__restrict__ sinT, int neox)
{
    const int pairs = ropeDim / 2, quads = pairs / 4;
    const long long total = (long long)seq * heads * quads;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int q = (int)(t % quads);
        const long long sh = t / quads;  // s * heads + h
        const int s = (int)(sh / heads);
        const float4 c = __ldg(reinterpret_cast<const float4 *>(cosT + (size_t)(posOffset + s) * pairs) + q);
        const float4 sn = __ldg(reinterpret_cast<const float4 *>(sinT + (size_t)(posOffset + s) * pairs) + q);
        float *p = x + sh * headDim;
        if (neox) {
            float4 *pa = reinterpret_cast<float4 *>(p) + q, *pb = reinterpret_cast<float4 *>(p + pairs) + q;
            const float4 a = *pa, b = *pb;
            *pa = make_float4(__fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(b.x, sn.x)), __fsub_rn(__fmul_rn(a.y, c.y), __fmul_rn(b.y, sn.y)),
                              __fsub_rn(__fmul_rn(a.z, c.z), __fmul_rn(b.z, sn.z)), __fsub_rn(__fmul_rn(a.w, c.w), __fmul_rn(b.w, sn.w)));
            *pb = make_float4(__fadd_rn(__fmul_rn(b.x, c.x), __fmul_rn(a.x, sn.x)), __fadd_rn(__fmul_rn(b.y, c.y), __fmul_rn(a.y, sn.y)),
                              __fadd_rn(__fmul_rn(b.z, c.z), __fmul_rn(a.z, sn.z)), __fadd_rn(__fmul_rn(b.w, c.w), __fmul_rn(a.w, sn.w)));
        } else {
            float4 *pv = reinterpret_cast<float4 *>(p) + 2 * q;
            const float4 u = pv[0], v = pv[1];  // pairs (u.x, u.y), (u.z, u.w), (v.x, v.y), (v.z, v.w)
            pv[0] = make_float4(__fsub_rn(__fmul_rn(u.x, c.x), __fmul_rn(u.y, sn.x)), __fadd_rn(__fmul_rn(u.y, c.x), __fmul_rn(u.x, sn.x)),
                                __fsub_rn(__fmul_rn(u.z, c.y), __fmul_rn(u.w, sn.y)), __fadd_rn(__fmul_rn(u.w, c.y), __fmul_rn(u.z, sn.y)));
            pv[1] = make_float4(__fsub_rn(__fmul_rn(v.x, c.z), __fmul_rn(v.y, sn.z)), __fadd_rn(__fmul_rn(v.y, c.z), __fmul_rn(v.x, sn.z)),
                                __fsub_rn(__fmul_rn(v.z, c.w), __fmul_rn(v.w, sn.w)), __fadd_rn(__fmul_rn(v.w, c.w), __fmul_rn(v.z, sn.w)));
        }
    }
}

// ---------------------------------------------------------------------------- add / argmax / embed
// LinearLayer.AddBiasInPlace (SharpMind.Model/Layers/Linearlayer.cs:154-163): out[r, j] += bias[j].
__global__ void __launch_bounds__(256) add_bias_kernel(float *__restrict__ out, const float *__restrict__ bias, long long total, int n)
{
    smc_grid_dep_sync();
    long long stride = (long long)gridDim.x * blockDim.x;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) out[t] = out[t] + __ldg(bias + t % n);
}

__global__ void __launch_bounds__(256) add_kernel(float *__restrict__ x, const float *__restrict__ y, long long n)
{
    long long stride = (long long)gridDim.x * blockDim.x;
    long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if ((n & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
        float4 *x4 = reinterpret_cast<float4 *>(x);
        const float4 *y4 = reinterpret_cast<const float4 *>(y);
        for (; t < n / 4; t += stride) {
            float4 a = x4[t], b = y4[t];
            x4[t] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        }
    } else {
        for (; t < n; t += stride) x[t] = x[t] + y[t];
    }
}

// First index of the largest value per row (Sampler.Argmax keeps the first maximum).  A row is cut into
// chunks scanned by one CTA each; the CTA that finishes a row last combines the chunk results.
constexpr int ARGMAX_CHUNK = 2048;

__device__ __forceinline__ bool argmax_better(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ logits, int n, int chunks, float *part_v,
                                                     int *part_i, unsigned *tickets, int *__restrict__ out)
{
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int s_last;
    smc_grid_dep_sync();
    const int row = blockIdx.y, c = blockIdx.x;
    const float *p = logits + (size_t)row * n;
    const int lo = c * ARGMAX_CHUNK, hi = min(n, lo + ARGMAX_CHUNK);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = p[i];
        if (v > best || idx == 0x7fffffff) best = v, idx = i;  // strict > keeps the first maximum of the stride
    }
    auto reduce_warp = [&]() {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (argmax_better(ov, oi, best, idx)) best = ov, idx = oi;
        }
    };
    reduce_warp();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) sv[wid] = best, si[wid] = idx;
    __syncthreads();
    if (wid == 0) {
        best = lane < 8 ? sv[lane] : -INFINITY;
        idx = lane < 8 ? si[lane] : 0x7fffffff;
        reduce_warp();
        if (lane == 0) {
            part_v[(size_t)row * chunks + c] = best;
            part_i[(size_t)row * chunks + c] = idx;
            __threadfence();
            s_last = atomicAdd(&tickets[row], 1u) == (unsigned)chunks - 1 ? 1 : 0;
        }
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = -INFINITY, idx = 0x7fffffff;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
        const float v = __ldcg(part_v + (size_t)row * chunks + i);
        const int vi = __ldcg(part_i + (size_t)row * chunks + i);
        if (argmax_better(v, vi, best, idx)) best = v, idx = vi;
    }
    reduce_warp();
    __syncthreads();
    if (lane == 0) sv[wid] = best, si[wid] = idx;
    __syncthreads();
    if (wid == 0) {
        best = lane < 8 ? sv[lane] : -INFINITY;
        idx = lane < 8 ? si[lane] : 0x7fffffff;
        reduce_warp();
        if (lane == 0) {
            out[row] = idx;
            tickets[row] = 0;
        }
    }
}

// out[i, :] = dequantised row tokens[i] of a Q8_0 table (planes or raw layout).
__global__ void __launch_bounds__(256) embed_q8_0_kernel(const int8_t *__restrict__ qs, const __half *__restrict__ d,
                                                         const uint8_t *__restrict__ raw, const int *__restrict__ tokens,
                                                         int K, int vocab, float *__restrict__ out)
{
    smc_grid_dep_sync();
    int tok = tokens[blockIdx.x];
    if (tok < 0 || tok >= vocab) {  // out-of-range ids produce NaN rows instead of reading outside the table
        for (int i = threadIdx.x; i < K; i += blockDim.x) out[(size_t)blockIdx.x * K + i] = __int_as_float(0x7fc00000);
        return;
    }
    int nb = K / 32;
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        float scale, q;
        if (qs) {
            scale = __half2float(d[(size_t)tok * nb + i / 32]);
            q = (float)qs[(size_t)tok * K + i];
        } else {
            const uint8_t *b = raw + ((size_t)tok * nb + i / 32) * 34;
            scale = smc_h2f((uint16_t)(b[0] | (b[1] << 8)));
            q = (float)(int8_t)b[2 + (i & 31)];
        }
        out[(size_t)blockIdx.x * K + i] = q * scale;
    }
}

int ew_grid(long long items, int cap)
{
    long long g = (items + 255) / 256;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

// Residual add (d_y may be null: none) + RMSNorm with the row leaving as Q8_0 activations in `a`, and as fp32 too when
// d_out is given.  Returns SMC_E_UNSUPPORTED without launching when the shape or alignment needs the separate kernels.
int smc_launch_add_rmsnorm_q8(smc_ctx *ctx, float *d_x, const float *d_y, const float *d_w, float *d_out, int rows, int n, float eps,
                              smc_q8act *a, cudaStream_t s)
{
    const bool aligned = ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_y) | reinterpret_cast<uintptr_t>(d_out) |
                           reinterpret_cast<uintptr_t>(d_w)) & 15) == 0;
    if (!aligned || n % 32 || n <= 256) return SMC_E_UNSUPPORTED;
    if (rows > a->max_rows || n > a->max_k || (size_t)rows * n > (size_t)a->max_rows * a->max_k)
        return smc_fail(ctx, SMC_E_INVALID, "q8act buffer %d x %d too small for %d x %d", a->max_rows, a->max_k, rows, n);
    a->M = rows;
    a->K = n;
    smc_launch_dep(ctx->use_pdl, add_rmsnorm_q8_kernel, dim3(rows), dim3(256), 0, s, d_x, d_y, d_w, d_out, n, eps, a->q, a->d, a->dbits,
                   a->sd, a->s16);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

// ------------------------------------------------------------------------------------------ C ABI
extern "C" {

int smc_rmsnorm_dev(smc_ctx *ctx, const float *d_x, const float *d_w, float *d_out, int rows, int n, float eps,
                    void *stream)
{
    if (ctx && rows == 0) return SMC_OK;  // an empty tensor has no data pointer to check
    if (!ctx || !d_x || !d_w || !d_out || rows < 0 || n <= 0) return smc_fail(ctx, SMC_E_INVALID, "rmsnorm: bad arguments");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    bool aligned = ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_out) |
                     reinterpret_cast<uintptr_t>(d_w)) & 15) == 0;
    if (n <= 256) {
        // short rows (per-head QK norm): a warp per row
        smc_launch_dep(ctx->use_pdl, rmsnorm_warp_kernel, dim3((rows + 7) / 8), dim3(256), 0, s, d_x, d_w, d_out, rows, n, eps);
    } else {
        smc_launch_dep(ctx->use_pdl, rmsnorm_cta_kernel, dim3(rows), dim3(256), 0, s, d_x, d_w, d_out, n, eps,
                       (aligned && (n & 3) == 0) ? 1 : 0);
    }
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_add_rmsnorm_dev(smc_ctx *ctx, float *d_x, const float *d_y, const float *d_w, float *d_out, int rows, int n,
                        float eps, void *stream)
{
    if (ctx && rows == 0) return SMC_OK;
    if (!ctx || !d_x || !d_y || !d_w || !d_out || rows < 0 || n <= 0)
        return smc_fail(ctx, SMC_E_INVALID, "add_rmsnorm: bad arguments");
    if (n <= 256) {  // short rows: the two separate kernels (a warp per row)
        int rc = smc_add_dev(ctx, d_x, d_y, (int64_t)rows * n, stream);
        if (rc) return rc;
        return smc_rmsnorm_dev(ctx, d_x, d_w, d_out, rows, n, eps, stream);
    }
    // the vector form needs what both separate kernels need: add_kernel vectorises on the whole tensor
    const bool aligned = ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_y) |
                           reinterpret_cast<uintptr_t>(d_out) | reinterpret_cast<uintptr_t>(d_w)) & 15) == 0;
    smc_launch_dep(ctx->use_pdl, add_rmsnorm_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), d_x, d_y, d_w, d_out,
                   n, eps, (aligned && (n & 3) == 0) ? 1 : 0);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_add_rmsnorm_q8_dev(smc_ctx *ctx, float *d_x, const float *d_y, const float *d_w, float *d_out, int rows, int n, float eps,
                           smc_q8act *a, void *stream)
{
    if (!ctx || !d_x || !d_w || !a || rows <= 0 || n <= 0) return smc_fail(ctx, SMC_E_INVALID, "add_rmsnorm_q8: bad arguments");
    const int rc = smc_launch_add_rmsnorm_q8(ctx, d_x, d_y, d_w, d_out, rows, n, eps, a, static_cast<cudaStream_t>(stream));
    if (rc == SMC_E_UNSUPPORTED)
        return smc_fail(ctx, rc, "add_rmsnorm_q8: rows of %d floats (needs a multiple of 32 above 256 and 16-byte aligned pointers)", n);
    return rc;
}

int smc_swiglu_dev(smc_ctx *ctx, const float *d_gate, const float *d_up, float *d_dst, int rows, int F, int ld,
                   void *stream)
{
    if (!ctx || !d_gate || !d_up || !d_dst || rows < 0 || F <= 0 || ld < F)
        return smc_fail(ctx, SMC_E_INVALID, "swiglu: bad arguments");
    if (rows == 0) return SMC_OK;
    bool aligned = ((reinterpret_cast<uintptr_t>(d_gate) | reinterpret_cast<uintptr_t>(d_up) |
                     reinterpret_cast<uintptr_t>(d_dst)) & 15) == 0;
    int vec = (aligned && ((F | ld) & 3) == 0) ? 1 : 0;
    long long total = (long long)rows * F;
    smc_launch_dep(ctx->use_pdl, swiglu_kernel, dim3(ew_grid(vec ? total / 4 : total, ctx->sm_count * 8)), dim3(256), 0,
                   static_cast<cudaStream_t>(stream), 
        d_gate, d_up, d_dst, rows, F, ld, vec);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_silu_dev(smc_ctx *ctx, const float *d_src, float *d_dst, int64_t n, void *stream)
{
    if (ctx && n == 0) return SMC_OK;
    if (!ctx || !d_src || !d_dst || n < 0) return smc_fail(ctx, SMC_E_INVALID, "silu: bad arguments");
    silu_kernel<<<ew_grid(n, ctx->sm_count * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_src, d_dst, n);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_softmax_dev(smc_ctx *ctx, const float *d_src, float *d_dst, int rows, int n, void *stream)
{
    if (ctx && rows == 0) return SMC_OK;
    if (!ctx || !d_src || !d_dst || rows < 0 || n <= 0) return smc_fail(ctx, SMC_E_INVALID, "softmax: bad arguments");
    int vec = ((n & 3) == 0 && ((reinterpret_cast<uintptr_t>(d_src) | reinterpret_cast<uintptr_t>(d_dst)) & 15) == 0) ? 1 : 0;
    int threads = n >= 8192 ? 1024 : (n >= 1024 ? 256 : 64);
    softmax_kernel<<<rows, threads, 0, static_cast<cudaStream_t>(stream)>>>(d_src, d_dst, n, vec);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_rope_tables(smc_ctx *ctx, float theta, int ropeDim, int maxSeq, float *d_cos, float *d_sin)
{
    if (!ctx || !d_cos || !d_sin || ropeDim <= 0 || (ropeDim & 1) || maxSeq <= 0)
        return smc_fail(ctx, SMC_E_INVALID, "rope_tables: bad arguments");
    // Set-up work, done on the host with the same libm calls as the reference's MathF.Pow/Cos/Sin so
    // that the tables are the reference's tables; the rotation itself runs on the device.
    const int half = ropeDim / 2;
    std::vector<float> freqs(half), c((size_t)maxSeq * half), s((size_t)maxSeq * half);
    for (int i = 0; i < half; ++i) {
        float e = 2.f * (float)i / (float)ropeDim;
        freqs[i] = 1.f / powf(theta, e);
    }
    for (int pos = 0; pos < maxSeq; ++pos)
        for (int i = 0; i < half; ++i) {
            float angle = (float)pos * freqs[i];
            c[(size_t)pos * half + i] = cosf(angle);
            s[(size_t)pos * half + i] = sinf(angle);
        }
    std::lock_guard<std::mutex> lock(ctx->mu);
    SMC_CUDA(ctx, cudaMemcpy(d_cos, c.data(), c.size() * sizeof(float), cudaMemcpyHostToDevice));
    SMC_CUDA(ctx, cudaMemcpy(d_sin, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice));
    // a copy from pageable memory returns once it is staged; the tables may be read next from any stream
    SMC_CUDA(ctx, cudaDeviceSynchronize());
    return SMC_OK;
}

int smc_rope_dev(smc_ctx *ctx, float *d_x, int seq, int heads, int headDim, int ropeDim, int posOffset,
                 const float *d_cos, const float *d_sin, int neox, void *stream)
{
    if (!ctx || !d_x || !d_cos || !d_sin || seq < 0 || heads <= 0 || headDim <= 0 || (headDim & 1) || ropeDim <= 0 ||
        ropeDim > headDim || (ropeDim & 1) || posOffset < 0)
        return smc_fail(ctx, SMC_E_INVALID, "rope: bad arguments");
    if (seq == 0) return SMC_OK;
    long long total = (long long)seq * heads * (ropeDim / 2);
    const bool vec = (ropeDim % 8) == 0 && (headDim % 4) == 0 &&
                     ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_cos) | reinterpret_cast<uintptr_t>(d_sin)) & 15) == 0;
    if (vec)
        rope_vec_kernel<<<ew_grid(total / 4, ctx->sm_count * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            d_x, seq, heads, headDim, ropeDim, posOffset, d_cos, d_sin, neox);
    else
        rope_kernel<<<ew_grid(total, ctx->sm_count * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
            d_x, seq, heads, headDim, ropeDim, posOffset, d_cos, d_sin, neox);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_add_dev(smc_ctx *ctx, float *d_x, const float *d_y, int64_t n, void *stream)
{
    if (!ctx || !d_x || !d_y || n < 0) return smc_fail(ctx, SMC_E_INVALID, "add: bad arguments");
    if (n == 0) return SMC_OK;
    add_kernel<<<ew_grid(n / 4 + 1, ctx->sm_count * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_x, d_y, n);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_add_bias_dev(smc_ctx *ctx, float *d_out, const float *d_bias, int rows, int n, void *stream)
{
    if (!ctx || !d_out || !d_bias || rows < 0 || n <= 0) return smc_fail(ctx, SMC_E_INVALID, "add_bias: bad arguments");
    if (rows == 0) return SMC_OK;
    const long long total = (long long)rows * n;
    smc_launch_dep(ctx->use_pdl, add_bias_kernel, dim3(ew_grid(total, ctx->sm_count * 8)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                   d_out, d_bias, total, n);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_linear_dev(smc_ctx *ctx, const float *d_in, const smc_weight *w, const float *d_bias, float *d_out, int M, int mode,
                   void *stream)
{
    int rc = smc_qmatmul_dev(ctx, d_in, w, d_out, M, mode, stream);
    if (rc || !d_bias || M == 0) return rc;
    return smc_add_bias_dev(ctx, d_out, d_bias, M, w->N, stream);
}

int smc_argmax_dev(smc_ctx *ctx, const float *d_logits, int rows, int n, int *d_out, void *stream)
{
    if (!ctx || !d_logits || !d_out || rows < 0 || n <= 0) return smc_fail(ctx, SMC_E_INVALID, "argmax: bad arguments");
    if (rows == 0) return SMC_OK;
    const int chunks = (n + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    {
        // scratch for the chunk results and the per-row tickets, grown on demand (the first call of a larger
        // shape allocates: make it outside stream capture).  Layout: values [rows x chunks] | indices | tickets.
        std::lock_guard<std::mutex> lock(ctx->mu);
        if (rows > ctx->argmax_rows || chunks > ctx->argmax_chunks) {
            const int big_rows = rows > ctx->argmax_rows ? rows : ctx->argmax_rows;
            const int big_chunks = chunks > ctx->argmax_chunks ? chunks : ctx->argmax_chunks;
            if (ctx->d_argmax) {
                cudaDeviceSynchronize();
                cudaFree(ctx->d_argmax);
                ctx->d_argmax = nullptr, ctx->argmax_rows = ctx->argmax_chunks = 0;
            }
            const size_t bytes = (size_t)big_rows * big_chunks * 8 + (size_t)big_rows * 4;
            SMC_CUDA(ctx, cudaMalloc(&ctx->d_argmax, bytes));
            SMC_CUDA(ctx, cudaMemset(ctx->d_argmax, 0, bytes));
            ctx->argmax_rows = big_rows, ctx->argmax_chunks = big_chunks;
        }
    }
    const size_t cap_cells = (size_t)ctx->argmax_rows * ctx->argmax_chunks;
    float *pv = reinterpret_cast<float *>(ctx->d_argmax);
    int *pi = reinterpret_cast<int *>(pv + cap_cells);
    unsigned *tk = reinterpret_cast<unsigned *>(pi + cap_cells);
    smc_launch_dep(ctx->use_pdl, argmax_kernel, dim3(chunks, rows), dim3(256), 0, static_cast<cudaStream_t>(stream), d_logits, n, chunks,
                   pv, pi, tk, d_out);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_embed_q8_0_dev(smc_ctx *ctx, const smc_weight *table, const int *d_tokens, int count, float *d_out,
                       void *stream)
{
    if (!ctx || !table || !d_tokens || !d_out || count < 0) return smc_fail(ctx, SMC_E_INVALID, "embed: bad arguments");
    if (table->dtype != SMC_Q8_0 || table->K % 32)
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "embed: table must be Q8_0 with K %% 32 == 0");
    if (!table->q8_qs && !table->d_raw) return smc_fail(ctx, SMC_E_INVALID, "embed: table holds no data");
    if (count == 0) return SMC_OK;
    smc_launch_dep(ctx->use_pdl, embed_q8_0_kernel, dim3(count), dim3(256), 0, static_cast<cudaStream_t>(stream), table->q8_qs, table->q8_d, table->d_raw,
                                                                            d_tokens, table->K, table->N, d_out);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

}  // extern "C"

int smc_launch_rmsnorm_row(smc_ctx *ctx, const float *src, const float *w, float *dst, int n, float rms_inv,
                           cudaStream_t s)
{
    rmsnorm_row_kernel<<<(n + 255) / 256, 256, 0, s>>>(src, w, dst, n, rms_inv);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}
