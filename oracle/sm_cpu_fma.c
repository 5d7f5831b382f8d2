/*
 * sm_cpu_fma.c -- C restatement of the reference's AVX2/FMA CPU tier, threaded the
 * way the reference threads it.  It is the TIMED CPU BASELINE that the benchmark
 * reports beside the GPU numbers, and a second opinion for the scalar oracle.
 *
 * THIS IS TEST / BENCHMARK INFRASTRUCTURE, NOT PRODUCT CODE.  The shipped CUDA
 * library never links or calls it.  It is a port (the reference is C# and cannot
 * be compiled where this runs), so numbers taken with it are labelled "port".
 *
 * Build: gcc -O2 -mavx2 -mfma -mf16c -fopenmp -ffp-contract=off
 */
#include <immintrin.h>
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <string.h>

#define QK 32
#define QK_K 256
#define SMF_API __attribute__((visibility("default")))

enum { SMF_Q8_0 = 8, SMF_Q4_K = 12, SMF_Q6_K = 14 };

static inline float h2f(const uint8_t *p)
{
    uint16_t h;
    memcpy(&h, p, 2);
    return _cvtsh_ss(h); /* HalfToFloat_F16C, QuantizationKernels.cs:111-114 */
}

/* SharpMind.Core/MathHelpers.cs:10-17 (HSum256_Avx) */
static inline float hsum256(__m256 v)
{
    __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
    __m128 s = _mm_add_ps(lo, hi);
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    return _mm_cvtss_f32(_mm_add_ss(s, _mm_shuffle_ps(s, s, 1)));
}

/* SharpMind.Core/MathHelpers.cs:20-30 (HMax256_Avx) */
static inline float hmax256(__m256 v)
{
    __m128 m = _mm_max_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    m = _mm_max_ps(m, _mm_shuffle_ps(m, m, 0x4E));
    m = _mm_max_ps(m, _mm_shuffle_ps(m, m, 0xB1));
    return _mm_cvtss_f32(m);
}

static inline int k4_scale(int j, const uint8_t *sc)
{
    return j < 4 ? (sc[j] & 0x3F) : ((sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4));
}
static inline int k4_min(int j, const uint8_t *sc)
{
    return j < 4 ? (sc[j + 4] & 0x3F) : ((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
}

/* SharpMind.Core/Quantization/QuantizationKernels.Q8.cs:69-106 (VecDotQ8_0_FMA) */
SMF_API float smf_vecdot_q8_0(const float *input, const uint8_t *raw, int col, int K)
{
    int nBlocks = (K + QK - 1) / QK;
    double sum = 0;
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    for (int b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + ((int64_t)col * nBlocks + b) * 34;
        float d = h2f(block);
        const int8_t *q = (const int8_t *)(block + 2);
        int end = K - b * QK;
        if (end > QK) end = QK;
        const float *pIn = input + b * QK;
        __m256 vd = _mm256_set1_ps(d);
        int i = 0;
        for (; i <= end - 16; i += 16) {
            __m256 w0 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i *)(q + i))));
            __m256 w1 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i *)(q + i + 8))));
            acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + i), _mm256_mul_ps(w0, vd), acc0);
            acc1 = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + i + 8), _mm256_mul_ps(w1, vd), acc1);
        }
        for (; i <= end - 8; i += 8) {
            __m256 w = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i *)(q + i))));
            acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + i), _mm256_mul_ps(w, vd), acc0);
        }
        for (; i < end; i++) {
            float w = (float)q[i] * d;
            float p = pIn[i] * w;
            sum += p;
        }
    }
    sum += hsum256(_mm256_add_ps(acc0, acc1));
    return (float)sum;
}

/* SharpMind.Core/Quantization/QuantizationKernels.Q4.cs:687-747 (VecDotQ4K_FMA), including
 * its nibble extraction through an 8-float stack buffer. */
SMF_API float smf_vecdot_q4_K(const float *input, const uint8_t *raw, int col, int K)
{
    int64_t flat = (int64_t)col * K;
    int64_t startBlock = flat / QK_K;
    int colBlockStart = (int)(flat % QK_K);
    int nBlocks = (K + QK_K - 1) / QK_K;
    double sum = 0;
    float vv[8];
    __m256 acc = _mm256_setzero_ps();
    for (int b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + (startBlock + b) * 144;
        float dS = h2f(block), mS = h2f(block + 2);
        const uint8_t *sc = block + 4, *qs = block + 16;
        int cur = (b == 0) ? colBlockStart : 0;
        int end = K + colBlockStart - b * QK_K;
        if (end > QK_K) end = QK_K;
        const float *pIn = input + b * QK_K - colBlockStart;
        for (int n16 = cur; n16 < end; n16 += 128) {
            for (int j = 0; j < 4 && n16 + j * 32 < end; j++) {
                int base = n16 + j * 32;
                int isc = (n16 / 128) * 4 + j;
                float s = (float)k4_scale(isc, sc), m = (float)k4_min(isc, sc);
                __m256 vs = _mm256_set1_ps(s * dS), vm = _mm256_set1_ps(m * mS);
                int rem = end - base;
                if (rem > 32) rem = 32;
                int l = 0;
                for (; l <= rem - 8; l += 8) {
                    for (int sub = 0; sub < 8; sub++) {
                        int idx = base + l + sub;
                        vv[sub] = (float)((qs[(idx / 64) * 32 + (idx % 32)] >> (((idx % 64) / 32) * 4)) & 0x0F);
                    }
                    __m256 w = _mm256_sub_ps(_mm256_mul_ps(_mm256_loadu_ps(vv), vs), vm);
                    acc = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + base + l), w, acc);
                }
                for (; l < rem; l++) {
                    int idx = base + l;
                    int v = (qs[(idx / 64) * 32 + (idx % 32)] >> (((idx % 64) / 32) * 4)) & 0x0F;
                    float sv = s * (float)v;
                    float w = sv * dS;
                    float mm = m * mS;
                    w = w - mm;
                    float p = pIn[idx] * w;
                    sum += p;
                }
            }
        }
    }
    sum += hsum256(acc);
    return (float)sum;
}

/* SharpMind.Core/Quantization/QuantizationKernels.Q6.cs:130-235 (VecDotQ6K_FMA) */
SMF_API float smf_vecdot_q6_K(const float *input, const uint8_t *raw, int col, int K)
{
    int64_t flat = (int64_t)col * K;
    int64_t startBlock = flat / QK_K;
    int colBlockStart = (int)(flat % QK_K);
    int nBlocks = (K + QK_K - 1) / QK_K;
    double sum = 0;
    float vv[8];
    __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
    for (int b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + (startBlock + b) * 210;
        const uint8_t *ql = block, *qh = block + 128;
        const int8_t *scales = (const int8_t *)(block + 192);
        float d = h2f(block + 208);
        int cur = (b == 0) ? colBlockStart : 0;
        int end = K + colBlockStart - b * QK_K;
        if (end > QK_K) end = QK_K;
        const float *pIn = input + b * QK_K - colBlockStart;
        for (int nOff = cur; nOff < end; nOff += 128) {
            const uint8_t *pql = ql + (nOff == 0 ? 0 : 64);
            const uint8_t *pqh = qh + (nOff == 0 ? 0 : 32);
            const int8_t *psc = scales + (nOff == 0 ? 0 : 8);
            int halfRem = end - nOff;
            if (halfRem > 128) halfRem = 128;
            int l = 0;
            for (; l + 103 < halfRem && l < 32; l += 8) {
                int sOff = (l / 16) == 0 ? 0 : 1;
                for (int s = 0; s < 8; s++) {
                    int q = (pql[l + s] & 0x0F) | ((pqh[l + s] & 0x03) << 4);
                    float t = d * (float)psc[sOff + 0];
                    vv[s] = t * (float)(q - 32);
                }
                a0 = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + nOff + l), _mm256_loadu_ps(vv), a0);
                for (int s = 0; s < 8; s++) {
                    int q = (pql[l + s + 32] & 0x0F) | (((pqh[l + s] >> 2) & 0x03) << 4);
                    float t = d * (float)psc[sOff + 2];
                    vv[s] = t * (float)(q - 32);
                }
                a1 = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + nOff + l + 32), _mm256_loadu_ps(vv), a1);
                for (int s = 0; s < 8; s++) {
                    int q = ((pql[l + s] >> 4) & 0x0F) | (((pqh[l + s] >> 4) & 0x03) << 4);
                    float t = d * (float)psc[sOff + 4];
                    vv[s] = t * (float)(q - 32);
                }
                a2 = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + nOff + l + 64), _mm256_loadu_ps(vv), a2);
                for (int s = 0; s < 8; s++) {
                    int q = ((pql[l + s + 32] >> 4) & 0x0F) | (((pqh[l + s] >> 6) & 0x03) << 4);
                    float t = d * (float)psc[sOff + 6];
                    vv[s] = t * (float)(q - 32);
                }
                a3 = _mm256_fmadd_ps(_mm256_loadu_ps(pIn + nOff + l + 96), _mm256_loadu_ps(vv), a3);
            }
            for (; l < halfRem && l < 32; l++) {
                int is = l / 16;
                int q1 = (pql[l] & 0x0F) | ((pqh[l] & 0x03) << 4);
                int q2 = (pql[l + 32] & 0x0F) | (((pqh[l] >> 2) & 0x03) << 4);
                int q3 = ((pql[l] >> 4) & 0x0F) | (((pqh[l] >> 4) & 0x03) << 4);
                int q4 = ((pql[l + 32] >> 4) & 0x0F) | (((pqh[l] >> 6) & 0x03) << 4);
                int i1 = nOff + l, i2 = nOff + l + 32;
                float t1 = d * (float)psc[is + 0];
                t1 = t1 * (float)(q1 - 32);
                if (i2 >= end) {
                    if (i1 < end) { float p = pIn[i1] * t1; sum += p; }
                    break;
                }
                float t2 = d * (float)psc[is + 2]; t2 = t2 * (float)(q2 - 32);
                float t3 = d * (float)psc[is + 4]; t3 = t3 * (float)(q3 - 32);
                float t4 = d * (float)psc[is + 6]; t4 = t4 * (float)(q4 - 32);
                float p;
                p = pIn[i1] * t1; sum += p;
                p = pIn[i2] * t2; sum += p;
                p = pIn[nOff + l + 64] * t3; sum += p;
                p = pIn[nOff + l + 96] * t4; sum += p;
            }
        }
    }
    sum += hsum256(_mm256_add_ps(_mm256_add_ps(a0, a1), _mm256_add_ps(a2, a3)));
    return (float)sum;
}

static inline float vecdot(int dtype, const float *in, const uint8_t *raw, int col, int K)
{
    switch (dtype) {
    case SMF_Q8_0: return smf_vecdot_q8_0(in, raw, col, K);
    case SMF_Q4_K: return smf_vecdot_q4_K(in, raw, col, K);
    default: return smf_vecdot_q6_K(in, raw, col, K);
    }
}

SMF_API int smf_num_threads(void) { return omp_get_max_threads(); }
/* A launcher may have pinned OMP_NUM_THREADS to 1 in the environment: the caller states the thread count itself. */
SMF_API void smf_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

/* QuantizedMatMul*_Parallel_FMA (e.g. QuantizationKernels.Q8.cs:556-574) with
 * DecodeParallel's chunking rule (QuantizationKernels.cs:73-108): for M <= 1 split N into
 * at most `cores` chunks of a multiple of 16 columns when N*K >= 65536; for M > 1 one
 * parallel task per input row, each sweeping all N columns. */
SMF_API int smf_qmatmul_parallel(int dtype, const float *input, const uint8_t *raw, float *output,
                                 int M, int K, int N)
{
    if (dtype != SMF_Q8_0 && dtype != SMF_Q4_K && dtype != SMF_Q6_K)
        return -1;
    if (M <= 1) {
        int cores = omp_get_max_threads();
        int numChunks = ((int64_t)N * K >= 65536) ? (cores < N / 16 ? cores : N / 16) : 1;
        if (numChunks <= 1) {
            for (int c = 0; c < N; c++)
                output[c] = vecdot(dtype, input, raw, c, K);
            return 0;
        }
        int chunk = (N + numChunks - 1) / numChunks;
        chunk = (chunk + 15) / 16 * 16;
        numChunks = (N + chunk - 1) / chunk;
#pragma omp parallel for schedule(dynamic, 1)
        for (int ci = 0; ci < numChunks; ci++) {
            int c0 = ci * chunk, c1 = c0 + chunk < N ? c0 + chunk : N;
            for (int c = c0; c < c1; c++)
                output[c] = vecdot(dtype, input, raw, c, K);
        }
        return 0;
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < M; r++) {
        const float *in = input + (int64_t)r * K;
        float *out = output + (int64_t)r * N;
        for (int c = 0; c < N; c++)
            out[c] = vecdot(dtype, in, raw, c, K);
    }
    return 0;
}

/* SharpMind.Core/Activations/ActivationKernels.cs:45-83 (FastExp) */
static inline __m256 fast_exp(__m256 x)
{
    x = _mm256_min_ps(_mm256_max_ps(x, _mm256_set1_ps(-88.0f)), _mm256_set1_ps(88.0f));
    __m256 z = _mm256_mul_ps(x, _mm256_set1_ps(1.4426950408889634f));
    __m256 magic = _mm256_set1_ps(12582912.0f);
    __m256 nF = _mm256_sub_ps(_mm256_add_ps(z, magic), magic);
    __m256i nI = _mm256_cvtps_epi32(nF);
    __m256 r = _mm256_sub_ps(z, nF);
    __m256 u = _mm256_mul_ps(r, _mm256_set1_ps(0.6931471805599453f));
    __m256 p = _mm256_mul_ps(u, _mm256_set1_ps(1.0f / 720.0f));
    p = _mm256_mul_ps(u, _mm256_add_ps(_mm256_set1_ps(1.0f / 120.0f), p));
    p = _mm256_mul_ps(u, _mm256_add_ps(_mm256_set1_ps(1.0f / 24.0f), p));
    p = _mm256_mul_ps(u, _mm256_add_ps(_mm256_set1_ps(1.0f / 6.0f), p));
    p = _mm256_mul_ps(u, _mm256_add_ps(_mm256_set1_ps(0.5f), p));
    p = _mm256_mul_ps(u, _mm256_add_ps(_mm256_set1_ps(1.0f), p));
    p = _mm256_add_ps(_mm256_set1_ps(1.0f), p);
    __m256i e = _mm256_add_epi32(nI, _mm256_set1_epi32(127));
    e = _mm256_min_epi32(_mm256_max_epi32(e, _mm256_setzero_si256()), _mm256_set1_epi32(254));
    return _mm256_mul_ps(p, _mm256_castsi256_ps(_mm256_slli_epi32(e, 23)));
}

/* SharpMind.Core/Activations/ActivationKernels.cs:174-192 (SwiGLUAVX2) */
SMF_API void smf_swiglu(const float *gate, const float *up, float *dst, int n)
{
    __m256 one = _mm256_set1_ps(1.0f);
    int i = 0;
    for (; i <= n - 8; i += 8) {
        __m256 g = _mm256_loadu_ps(gate + i), u = _mm256_loadu_ps(up + i);
        __m256 e = fast_exp(_mm256_sub_ps(_mm256_setzero_ps(), g));
        __m256 sig = _mm256_div_ps(one, _mm256_add_ps(one, e));
        _mm256_storeu_ps(dst + i, _mm256_mul_ps(_mm256_mul_ps(g, sig), u));
    }
    for (; i < n; i++)
        dst[i] = (gate[i] / (1.f + expf(-gate[i]))) * up[i];
}

/* FfnKernels.Gated's activation loop (SharpMind.Model/Layers/Ffn/FfnKernels.cs:52-56): rows of
 * a fused [M, 2F] gate||up buffer, serial over rows like the reference. */
SMF_API void smf_swiglu_rows(const float *fused, float *dst, int M, int F)
{
    for (int r = 0; r < M; r++)
        smf_swiglu(fused + (int64_t)r * 2 * F, fused + (int64_t)r * 2 * F + F, dst + (int64_t)r * F, F);
}

/* SharpMind.Core/Activations/ActivationKernels.cs:257-314 (SoftmaxRowAVX2) */
SMF_API void smf_softmax_row(const float *src, float *dst, int n)
{
    if (n < 8) {
        float mx = src[0];
        for (int i = 1; i < n; i++) if (src[i] > mx) mx = src[i];
        float sum = 0.f;
        for (int i = 0; i < n; i++) { dst[i] = expf(src[i] - mx); sum += dst[i]; }
        float inv = 1.f / sum;
        for (int i = 0; i < n; i++) dst[i] *= inv;
        return;
    }
    int i = 0;
    __m256 vmax = _mm256_set1_ps(src[0]);
    for (; i <= n - 8; i += 8) vmax = _mm256_max_ps(vmax, _mm256_loadu_ps(src + i));
    float mx = hmax256(vmax);
    for (; i < n; i++) if (src[i] > mx) mx = src[i];
    __m256 vsum = _mm256_setzero_ps(), vm = _mm256_set1_ps(mx);
    for (i = 0; i <= n - 8; i += 8) {
        __m256 e = fast_exp(_mm256_sub_ps(_mm256_loadu_ps(src + i), vm));
        _mm256_storeu_ps(dst + i, e);
        vsum = _mm256_add_ps(vsum, e);
    }
    float sum = hsum256(vsum);
    for (; i < n; i++) { float e = expf(src[i] - mx); dst[i] = e; sum += e; }
    float inv = 1.f / sum;
    __m256 vinv = _mm256_set1_ps(inv);
    for (i = 0; i <= n - 8; i += 8) _mm256_storeu_ps(dst + i, _mm256_mul_ps(_mm256_loadu_ps(dst + i), vinv));
    for (; i < n; i++) dst[i] *= inv;
}

/* SharpMind.Model/Layers/NormKernels.cs:13-60 (RMSNormParamAVX2 + RMSNormRowAVX2) per row */
SMF_API void smf_rmsnorm(const float *x, const float *w, float *out, int rows, int n, float eps)
{
    for (int r = 0; r < rows; r++) {
        const float *p = x + (int64_t)r * n;
        float *o = out + (int64_t)r * n;
        __m256 vs = _mm256_setzero_ps();
        int i = 0;
        for (; i <= n - 8; i += 8) {
            __m256 v = _mm256_loadu_ps(p + i);
            vs = _mm256_add_ps(vs, _mm256_mul_ps(v, v));
        }
        float ss = hsum256(vs);
        for (; i < n; i++) { float sq = p[i] * p[i]; ss += sq; }
        float mean = ss / (float)n;
        float inv = 1.f / sqrtf(mean + eps);
        __m256 vi = _mm256_set1_ps(inv);
        for (i = 0; i <= n - 8; i += 8)
            _mm256_storeu_ps(o + i, _mm256_mul_ps(_mm256_mul_ps(_mm256_loadu_ps(p + i), vi), _mm256_loadu_ps(w + i)));
        for (; i < n; i++) { float t = p[i] * inv; o[i] = t * w[i]; }
    }
}

/* SharpMind.Core/Tensors/Tensor.cs:273-282,328-332 (AddInPlace through Vector<T>) */
SMF_API void smf_add_inplace(float *x, const float *y, int64_t n)
{
    int64_t i = 0;
    for (; i <= n - 8; i += 8)
        _mm256_storeu_ps(x + i, _mm256_add_ps(_mm256_loadu_ps(x + i), _mm256_loadu_ps(y + i)));
    for (; i < n; i++) x[i] = x[i] + y[i];
}
