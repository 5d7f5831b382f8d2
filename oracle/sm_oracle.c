/*
 * sm_oracle.c -- CPU restatement of SharpMind's quantized vec-dot / matmul path and
 * the fp32 ops the decoder runs around it.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It exists so that the CUDA
 * library can be checked against the reference's arithmetic.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may load it; the
 * shipped library never links or calls anything in this file.
 *
 * Every function names the reference source it follows (paths are relative to
 * the SharpMind repository root).  Rounding rules that matter:
 *   - C# `float * float` is an fp32 product; `double += float` widens the
 *     already-rounded product.  Build with -ffp-contract=off so gcc never fuses.
 *   - MathF.Round(x, MidpointRounding.AwayFromZero) == roundf(x)
 *   - MathF.Round(x) == round-half-to-even == nearbyintf(x) in the default mode
 *   - (Half)f == IEEE round-to-nearest-even conversion
 *
 * Parity pins: the reference's own known-answer tests (single-block vec-dots,
 * fp16 bit patterns, RoPE expected values, K-quant round-trip bounds) and the
 * reference's own C oracle (tools/ReferenceDataGenerator/vecdot_ref.c) compiled
 * from its source tree; see tests/test_oracle_pins.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK 32
#define QK_K 256

#define SMO_API __attribute__((visibility("default")))

/* QuantDType numbering: SharpMind.Core/Quantization/QuantDType.cs:2-18 */
enum { SMO_Q8_0 = 8, SMO_Q4_K = 12, SMO_Q6_K = 14 };

/* ------------------------------------------------------------------------- */
/* fp16 helpers                                                               */
/* ------------------------------------------------------------------------- */

/* SharpMind.Core/Quantization/QuantizationKernels.cs:117-146 (HalfToFloat_Scalar) */
SMO_API float smo_half_to_float(uint16_t h)
{
    uint32_t sign = ((uint32_t)(h & 0x8000u)) << 16;
    int exp5 = (h >> 10) & 0x1F;
    uint32_t mant = h & 0x3FFu;
    uint32_t bits;
    if (exp5 == 0) {
        if (mant == 0) {
            bits = sign;
        } else {
            int k = 31 - __builtin_clz(mant); /* position of the leading one */
            bits = sign | ((uint32_t)(k + 103) << 23) | ((mant - (1u << k)) << (23 - k));
        }
    } else if (exp5 == 31) {
        bits = sign | 0x7F800000u | (mant ? 0x00400000u : 0u);
    } else {
        bits = sign | ((uint32_t)(exp5 + 112) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* SharpMind.Core/Quantization/QuantizationKernels.cs:149 (FloatToHalf_F16C == (Half)f,
 * IEEE round-to-nearest-even, subnormals honoured). */
SMO_API uint16_t smo_float_to_half(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? (0x0200u | ((absx >> 13) & 0x3FFu)) : 0u));
    if (absx >= 0x477FF000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    if (absx < 0x33000001u) /* below half of the smallest subnormal -> zero */
        return (uint16_t)sign;
    int e = (int)(absx >> 23) - 127;
    uint32_t m = (absx & 0x007FFFFFu) | 0x00800000u;
    int shift; /* how many low bits of the 24-bit significand are dropped */
    int he;
    if (e < -14) {
        shift = 13 + (-14 - e);
        he = 0;
    } else {
        shift = 13;
        he = e + 15;
    }
    uint32_t kept = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u)))
        kept++;
    uint32_t out;
    if (he == 0)
        out = kept; /* a carry into bit 10 lands on the min normal */
    else
        out = ((uint32_t)he << 10) + (kept - 0x400u); /* mantissa carry bumps the exponent */
    return (uint16_t)(sign | out);
}

/* SharpMind.Core/Quantization/QuantizationKernels.cs:152-175 (FloatToHalf_Scalar,
 * which truncates the mantissa; kept to document that it differs from F16C). */
SMO_API uint16_t smo_float_to_half_trunc(float f)
{
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int exp = (int)((bits >> 23) & 0xFF) - 127 + 15;
    uint32_t mant = bits & 0x007FFFFFu;
    if (exp <= 0) {
        if (exp < -10)
            return (uint16_t)sign;
        mant = (mant | 0x00800000u) >> (1 - exp);
        return (uint16_t)(sign | (mant >> 13));
    }
    if (exp >= 31) {
        if (exp > 31)
            return (uint16_t)(sign | 0x7C00u | (mant >> 13));
        return (uint16_t)(sign | 0x7C00u | (mant != 0 ? 0x200u : 0u));
    }
    return (uint16_t)(sign | ((uint32_t)exp << 10) | (mant >> 13));
}

/* SharpMind.Core/Quantization/QuantizationKernels.cs:177-189 (GetScaleMinK4_*) */
static int k4_scale(int j, const uint8_t *sc)
{
    if (j < 4)
        return sc[j] & 0x3F;
    return (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4);
}
static int k4_min(int j, const uint8_t *sc)
{
    if (j < 4)
        return sc[j + 4] & 0x3F;
    return (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
}
SMO_API void smo_scale_min_k4(const uint8_t *sc12, int *scales8, int *mins8)
{
    for (int j = 0; j < 8; j++) {
        scales8[j] = k4_scale(j, sc12);
        mins8[j] = k4_min(j, sc12);
    }
}

static uint16_t rd16(const uint8_t *p)
{
    uint16_t v;
    memcpy(&v, p, 2);
    return v;
}

/* ------------------------------------------------------------------------- */
/* tensor byte counts                                                         */
/* ------------------------------------------------------------------------- */

/* SharpMind.Core/Quantization/QuantizationOps.cs:15-72 (GetRawTensorByteCount for [N,K]) */
SMO_API int64_t smo_raw_bytes(int dtype, int64_t N, int64_t K)
{
    switch (dtype) {
    case SMO_Q8_0: return N * ((K + 31) / 32) * 34;
    case SMO_Q4_K: return ((N * K + 255) / 256) * 144;
    case SMO_Q6_K: return ((N * K + 255) / 256) * 210;
    default: return -1;
    }
}

/* ------------------------------------------------------------------------- */
/* scalar vec-dots (the reference's ground truth tier)                        */
/* ------------------------------------------------------------------------- */

/* SharpMind.Core/Quantization/QuantizationKernels.Q8.cs:11-26 (VecDotQ8_0_Scalar) */
SMO_API float smo_vecdot_q8_0(const float *input, const uint8_t *raw, int col, int K)
{
    int nBlocks = (K + QK - 1) / QK;
    double sum = 0.0;
    for (int b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + ((int64_t)col * nBlocks + b) * 34;
        float d = smo_half_to_float(rd16(block));
        const int8_t *q = (const int8_t *)(block + 2);
        int end = K - b * QK;
        if (end > QK) end = QK;
        for (int i = 0; i < end; i++) {
            float w = (float)q[i] * d;
            float p = input[b * QK + i] * w;
            sum += p;
        }
    }
    return (float)sum;
}

/* SharpMind.Core/Quantization/QuantizationKernels.Q4.cs:586-623 (VecDotQ4K_Scalar).
 * The flat-tensor addressing (startBlock / colBlockStart) and the way the scale
 * index is derived from the loop start are kept as the reference has them, so
 * rows that begin mid-block behave identically. The reference computes
 * col*K in 32-bit; the products used by every supported shape stay below 2^31. */
SMO_API float smo_vecdot_q4_K(const float *input, const uint8_t *raw, int col, int K)
{
    int64_t flat = (int64_t)col * K;
    int64_t startBlock = flat / QK_K;
    int colBlockStart = (int)(flat % QK_K);
    int nBlocks = (K + QK_K - 1) / QK_K;
    double sum = 0.0;
    for (int b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + (startBlock + b) * 144;
        float dS = smo_half_to_float(rd16(block));
        float mS = smo_half_to_float(rd16(block + 2));
        const uint8_t *sc = block + 4;
        const uint8_t *qs = block + 16;
        int cur = (b == 0) ? colBlockStart : 0;
        int end = K + colBlockStart - b * QK_K;
        if (end > QK_K) end = QK_K;
        for (int n16 = cur; n16 < end; n16 += 128) {
            for (int j = 0; j < 4 && n16 + j * 32 < end; j++) {
                int base = n16 + j * 32;
                int isc = (n16 / 128) * 4 + j;
                float s = (float)k4_scale(isc, sc);
                float m = (float)k4_min(isc, sc);
                for (int l = 0; l < 32 && base + l < end; l++) {
                    int idx = base + l;
                    int v = (qs[(idx / 64) * 32 + (idx % 32)] >> (((idx % 64) / 32) * 4)) & 0x0F;
                    float sv = s * (float)v;
                    float w = sv * dS;
                    float mm = m * mS;
                    w = w - mm;
                    float p = input[b * QK_K + idx - colBlockStart] * w;
                    sum += p;
                }
            }
        }
    }
    return (float)sum;
}

/* SharpMind.Core/Quantization/QuantizationKernels.Q6.cs:12-65 (VecDotQ6K_Scalar) */
SMO_API float smo_vecdot_q6_K(const float *input, const uint8_t *raw, int col, int K)
{
    int64_t flat = (int64_t)col * K;
    int64_t startBlock = flat / QK_K;
    int colBlockStart = (int)(flat % QK_K);
    int nBlocks = (K + QK_K - 1) / QK_K;
    double sum = 0.0;
    for (int b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + (startBlock + b) * 210;
        const uint8_t *ql = block;
        const uint8_t *qh = block + 128;
        const int8_t *scales = (const int8_t *)(block + 192);
        float d = smo_half_to_float(rd16(block + 208));
        int cur = (b == 0) ? colBlockStart : 0;
        int end = K + colBlockStart - b * QK_K;
        if (end > QK_K) end = QK_K;
        for (int nOff = cur; nOff < end; nOff += 128) {
            const uint8_t *pql = ql + (nOff == 0 ? 0 : 64);
            const uint8_t *pqh = qh + (nOff == 0 ? 0 : 32);
            const int8_t *psc = scales + (nOff == 0 ? 0 : 8);
            int halfRem = end - nOff;
            if (halfRem > 128) halfRem = 128;
            for (int l = 0; l < 32 && l < halfRem; l++) {
                int is = l / 16;
                int q1 = (pql[l] & 0x0F) | ((pqh[l] & 0x03) << 4);
                int q2 = (pql[l + 32] & 0x0F) | (((pqh[l] >> 2) & 0x03) << 4);
                int q3 = ((pql[l] >> 4) & 0x0F) | (((pqh[l] >> 4) & 0x03) << 4);
                int q4 = ((pql[l + 32] >> 4) & 0x0F) | (((pqh[l] >> 6) & 0x03) << 4);
                int i1 = b * QK_K + nOff + l - colBlockStart;
                int i2 = i1 + 32;
                int lim = b * QK_K + end - colBlockStart;
                float w1 = d * (float)psc[is + 0];
                w1 = w1 * (float)(q1 - 32);
                if (i2 >= lim) {
                    if (i1 < lim) {
                        float p = input[i1] * w1;
                        sum += p;
                    }
                    break;
                }
                int i3 = i1 + 64, i4 = i1 + 96;
                float w2 = d * (float)psc[is + 2];
                w2 = w2 * (float)(q2 - 32);
                float w3 = d * (float)psc[is + 4];
                w3 = w3 * (float)(q3 - 32);
                float w4 = d * (float)psc[is + 6];
                w4 = w4 * (float)(q4 - 32);
                float p1 = input[i1] * w1; sum += p1;
                float p2 = input[i2] * w2; sum += p2;
                float p3 = input[i3] * w3; sum += p3;
                float p4 = input[i4] * w4; sum += p4;
            }
        }
    }
    return (float)sum;
}

SMO_API float smo_vecdot(int dtype, const float *input, const uint8_t *raw, int col, int K)
{
    switch (dtype) {
    case SMO_Q8_0: return smo_vecdot_q8_0(input, raw, col, K);
    case SMO_Q4_K: return smo_vecdot_q4_K(input, raw, col, K);
    case SMO_Q6_K: return smo_vecdot_q6_K(input, raw, col, K);
    default: return NAN;
    }
}

/* SharpMind.Core/Quantization/QuantizationKernels.cs:11-22 (QuantizedMatMul_Serial_Wrapper):
 * out[r, c] = vecdot(in[r, :], W, c, K). */
SMO_API int smo_qmatmul(int dtype, const float *input, const uint8_t *raw, float *output,
                        int M, int K, int N)
{
    if (dtype != SMO_Q8_0 && dtype != SMO_Q4_K && dtype != SMO_Q6_K)
        return -1;
    /* outputs are independent: spreading the columns over threads changes no bit of any of them */
    for (int r = 0; r < M; r++) {
#pragma omp parallel for schedule(static) if ((int64_t)N * K >= 262144)
        for (int c = 0; c < N; c++)
            output[(int64_t)r * N + c] = smo_vecdot(dtype, input + (int64_t)r * K, raw, c, K);
    }
    return 0;
}

/* Same, columns [c0, c1) only: lets a test check sampled rows of a big matrix. */
SMO_API int smo_qmatmul_cols(int dtype, const float *input, const uint8_t *raw, float *output,
                             int M, int K, int N, int c0, int c1)
{
    if (dtype != SMO_Q8_0 && dtype != SMO_Q4_K && dtype != SMO_Q6_K)
        return -1;
    for (int r = 0; r < M; r++)
        for (int c = c0; c < c1; c++)
            output[(int64_t)r * N + c] = smo_vecdot(dtype, input + (int64_t)r * K, raw, c, K);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* dequantising readers                                                       */
/* ------------------------------------------------------------------------- */

/* SharpMind.Core/Quantization/QuantizationKernels.Q8.cs:412-433 (ReadQ8_0_Scalar) */
SMO_API void smo_read_q8_0(const uint8_t *raw, float *data, int64_t n)
{
    int64_t nBlocks = (n + QK - 1) / QK;
    for (int64_t b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + b * 34;
        float d = smo_half_to_float(rd16(block));
        const int8_t *q = (const int8_t *)(block + 2);
        int64_t valid = n - b * QK;
        if (valid > QK) valid = QK;
        for (int j = 0; j < valid; j++)
            data[b * QK + j] = (float)q[j] * d;
    }
}

/* SharpMind.Core/Quantization/QuantizationKernels.Q4.cs:951-981 (ReadQ4K_Scalar) */
SMO_API void smo_read_q4_K(const uint8_t *raw, float *data, int64_t n)
{
    int64_t nBlocks = (n + QK_K - 1) / QK_K;
    for (int64_t b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + b * 144;
        float dS = smo_half_to_float(rd16(block));
        float mS = smo_half_to_float(rd16(block + 2));
        const uint8_t *sc = block + 4, *qs = block + 16;
        for (int i = 0; i < QK_K && b * QK_K + i < n; i++) {
            float s = (float)k4_scale(i / 32, sc);
            float m = (float)k4_min(i / 32, sc);
            int v = (qs[(i / 64) * 32 + (i % 32)] >> (((i % 64) / 32) * 4)) & 0x0F;
            float sv = s * (float)v;
            float w = sv * dS;
            float mm = m * mS;
            data[b * QK_K + i] = w - mm;
        }
    }
}

/* SharpMind.Core/Quantization/QuantizationKernels.Q6.cs:237-292 (ReadQ6K_Scalar), whole blocks */
SMO_API void smo_read_q6_K(const uint8_t *raw, float *data, int64_t n)
{
    int64_t nBlocks = n / QK_K;
    for (int64_t b = 0; b < nBlocks; b++) {
        const uint8_t *block = raw + b * 210;
        const uint8_t *ql = block, *qh = block + 128;
        const int8_t *scales = (const int8_t *)(block + 192);
        float d = smo_half_to_float(rd16(block + 208));
        for (int h = 0; h < 2; h++) {
            const uint8_t *pql = ql + 64 * h, *pqh = qh + 32 * h;
            const int8_t *psc = scales + 8 * h;
            float *o = data + b * QK_K + 128 * h;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q1 = (pql[l] & 0x0F) | ((pqh[l] & 0x03) << 4);
                int q2 = (pql[l + 32] & 0x0F) | (((pqh[l] >> 2) & 0x03) << 4);
                int q3 = ((pql[l] >> 4) & 0x0F) | (((pqh[l] >> 4) & 0x03) << 4);
                int q4 = ((pql[l + 32] >> 4) & 0x0F) | (((pqh[l] >> 6) & 0x03) << 4);
                float t;
                t = d * (float)psc[is + 0]; o[l] = t * (float)(q1 - 32);
                t = d * (float)psc[is + 2]; o[l + 32] = t * (float)(q2 - 32);
                t = d * (float)psc[is + 4]; o[l + 64] = t * (float)(q3 - 32);
                t = d * (float)psc[is + 6]; o[l + 96] = t * (float)(q4 - 32);
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* weight quantisers (make the test weights)                                  */
/* ------------------------------------------------------------------------- */

static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
static void wr16(uint8_t *p, uint16_t v) { memcpy(p, &v, 2); }

/* SharpMind.Core/Quantization/TensorQuantizer.cs:80-144 (WriteBlock, Q8_0 branch).
 * n must be a multiple of 32; returns -1 otherwise (the reference throws). */
SMO_API int smo_quantize_q8_0(const float *values, int64_t n, uint8_t *out)
{
    if (n % QK != 0)
        return -1;
    int64_t nBlocks = n / QK;
    memset(out, 0, (size_t)(nBlocks * 34));
    for (int64_t b = 0; b < nBlocks; b++) {
        const float *v = values + b * QK;
        uint8_t *o = out + b * 34;
        float amax = 0.f;
        for (int j = 0; j < QK; j++) {
            float a = fabsf(v[j]);
            if (a > amax) amax = a;
        }
        if (amax == 0.f)
            continue; /* scale 0, quants 0 */
        float d = amax / 127.f;
        wr16(o, smo_float_to_half(d));
        for (int j = 0; j < QK; j++) {
            float scaled = v[j] / d;
            int q = (int)roundf(scaled);
            q = clampi(q, -128, 127);
            o[2 + j] = (uint8_t)(int8_t)q;
        }
    }
    return 0;
}

/* SharpMind.Core/Quantization/TensorQuantizer.KQuant.cs:173-225 (WriteKQ4) with
 * PackScaleMinK4 (:451-459), GroupMinMax (:420-431), BlockAbsMax (:408-418). */
SMO_API int smo_quantize_q4_K(const float *values, int64_t n, uint8_t *out)
{
    if (n % QK_K != 0)
        return -1;
    int64_t nBlocks = n / QK_K;
    memset(out, 0, (size_t)(nBlocks * 144));
    int sc[8], mn[8];
    for (int64_t b = 0; b < nBlocks; b++) {
        const float *v = values + b * QK_K;
        uint8_t *o = out + b * 144;
        float amax = 0.f;
        for (int j = 0; j < QK_K; j++) {
            float a = fabsf(v[j]);
            if (a > amax) amax = a;
        }
        if (amax == 0.f)
            continue;
        float step = amax / 63.f;
        wr16(o, smo_float_to_half(step));
        wr16(o + 2, smo_float_to_half(step));
        for (int sub = 0; sub < 8; sub++) {
            const float *g = v + sub * 32;
            float gmn = 3.402823466e+38f, gmx = -3.402823466e+38f;
            for (int j = 0; j < 32; j++) {
                if (g[j] < gmn) gmn = g[j];
                if (g[j] > gmx) gmx = g[j];
            }
            float range = gmx - gmn;
            float negmin = -gmn;
            mn[sub] = clampi((int)roundf(negmin / step), 0, 63);
            if (range <= 0.f) {
                sc[sub] = 0;
                continue; /* codes stay 0 */
            }
            float den = 15.f * step;
            sc[sub] = clampi((int)roundf(range / den), 1, 63);
            float scF = (float)sc[sub] * step;
            for (int j = 0; j < 32; j++) {
                float off = (float)mn[sub] * step;
                float num = g[j] + off;
                int code = clampi((int)roundf(num / scF), 0, 15);
                int i = sub * 32 + j;
                o[16 + (i / 64) * 32 + (i % 32)] |= (uint8_t)(code << (((i % 64) / 32) * 4));
            }
        }
        for (int j = 0; j < 4; j++) {
            o[4 + j] = (uint8_t)((sc[j] & 0x3F) | ((sc[4 + j] >> 4) << 6));
            o[4 + 4 + j] = (uint8_t)((mn[j] & 0x3F) | ((mn[4 + j] >> 4) << 6));
            o[4 + 8 + j] = (uint8_t)((sc[4 + j] & 0x0F) | ((mn[4 + j] & 0x0F) << 4));
        }
    }
    return 0;
}

/* SharpMind.Core/Quantization/TensorQuantizer.KQuant.cs:303-376 (WriteKQ6, WriteQ6Code) */
SMO_API int smo_quantize_q6_K(const float *values, int64_t n, uint8_t *out)
{
    if (n % QK_K != 0)
        return -1;
    int64_t nBlocks = n / QK_K;
    memset(out, 0, (size_t)(nBlocks * 210));
    for (int64_t b = 0; b < nBlocks; b++) {
        const float *v = values + b * QK_K;
        uint8_t *o = out + b * 210;
        float amax = 0.f;
        for (int j = 0; j < QK_K; j++) {
            float a = fabsf(v[j]);
            if (a > amax) amax = a;
        }
        if (amax == 0.f)
            continue;
        float d = amax / 4064.f;
        wr16(o + 208, smo_float_to_half(d));
        for (int g = 0; g < 16; g++) {
            const float *gv = v + g * 16;
            float gmx = 0.f;
            for (int j = 0; j < 16; j++) {
                float a = fabsf(gv[j]);
                if (a > gmx) gmx = a;
            }
            float den = 32.f * d;
            int scale = (gmx == 0.f) ? 0 : clampi((int)roundf(gmx / den), 1, 127);
            o[192 + g] = (uint8_t)(int8_t)scale;
            float scf = d * (float)scale;
            for (int j = 0; j < 16; j++) {
                int i = g * 16 + j;
                int code = (gmx == 0.f) ? 32 : clampi((int)roundf(gv[j] / scf) + 32, 0, 63);
                int nOff = (i / 128) * 128;
                int local = i - nOff;
                int l = local % 32, colq = local / 32;
                int qlIdx = (nOff == 0 ? 0 : 64) + ((colq == 1 || colq == 3) ? l + 32 : l);
                if (colq == 2 || colq == 3)
                    o[qlIdx] = (uint8_t)((o[qlIdx] & 0x0F) | ((code & 0x0F) << 4));
                else
                    o[qlIdx] = (uint8_t)((o[qlIdx] & 0xF0) | (code & 0x0F));
                int qhIdx = 128 + (nOff == 0 ? 0 : 32) + l;
                int shift = colq * 2;
                o[qhIdx] = (uint8_t)((o[qhIdx] & ~(0x03 << shift)) | (((code >> 4) & 0x03) << shift));
            }
        }
    }
    return 0;
}

SMO_API int smo_quantize(int dtype, const float *values, int64_t n, uint8_t *out)
{
    switch (dtype) {
    case SMO_Q8_0: return smo_quantize_q8_0(values, n, out);
    case SMO_Q4_K: return smo_quantize_q4_K(values, n, out);
    case SMO_Q6_K: return smo_quantize_q6_K(values, n, out);
    default: return -1;
    }
}

/* ------------------------------------------------------------------------- */
/* run-time activation quantiser and integer block sums                       */
/* ------------------------------------------------------------------------- */

/* SharpMind.Model/QuantizedKVCache.cs:191-223 (QuantizeRowQ8_0): the reference's only
 * run-time fp32 -> Q8_0 row quantiser. d = amax/127 (1 when the block is all zero),
 * q = round-half-to-even(x / d) clamped, partial last block padded with zeros. */
SMO_API void smo_quantize_row_q8_0(const float *src, uint8_t *dst, int n)
{
    int nBlocks = (n + QK - 1) / QK;
    for (int b = 0; b < nBlocks; b++) {
        int end = n - b * QK;
        if (end > QK) end = QK;
        const float *p = src + b * QK;
        uint8_t *o = dst + b * 34;
        float amax = 0.f;
        for (int i = 0; i < end; i++) {
            float a = fabsf(p[i]);
            if (a > amax) amax = a;
        }
        float d = amax / 127.f;
        if (amax == 0.f) d = 1.f;
        wr16(o, smo_float_to_half(d));
        int8_t *q = (int8_t *)(o + 2);
        for (int i = 0; i < end; i++) {
            float t = p[i] / d;
            int v = (int)nearbyintf(t);
            q[i] = (int8_t)clampi(v, -128, 127);
        }
        for (int i = end; i < QK; i++)
            q[i] = 0;
    }
}

/* Integer dot of one weight row with a Q8_0-quantised activation row, one int32 per
 * 32-element block: sums[b] = sum_i qw(b, i) * qx(b, i), with qw the raw integer code
 * the vec-dots above read (Q8_0: the int8; Q4_K: the 4-bit code; Q6_K: code - 32).
 * Requires K % 32 == 0 (Q8_0) or K % 256 == 0 (K-quants). */
SMO_API int smo_block_isums(int dtype, const uint8_t *raw, const uint8_t *xq8, int col, int K,
                            int32_t *sums)
{
    int nb32 = K / 32;
    if (dtype == SMO_Q8_0) {
        if (K % 32) return -1;
        for (int b = 0; b < nb32; b++) {
            const int8_t *qw = (const int8_t *)(raw + ((int64_t)col * nb32 + b) * 34 + 2);
            const int8_t *qx = (const int8_t *)(xq8 + (int64_t)b * 34 + 2);
            int32_t s = 0;
            for (int i = 0; i < 32; i++) s += (int32_t)qw[i] * qx[i];
            sums[b] = s;
        }
        return 0;
    }
    if (K % 256) return -1;
    int nbk = K / 256;
    for (int kb = 0; kb < nbk; kb++) {
        int64_t blk = (int64_t)col * nbk + kb;
        for (int i = 0; i < 256; i++) {
            int code;
            if (dtype == SMO_Q4_K) {
                const uint8_t *qs = raw + blk * 144 + 16;
                code = (qs[(i / 64) * 32 + (i % 32)] >> (((i % 64) / 32) * 4)) & 0x0F;
            } else if (dtype == SMO_Q6_K) {
                const uint8_t *block = raw + blk * 210;
                int h = i / 128, local = i % 128, l = local % 32, c = local / 32;
                const uint8_t *pql = block + 64 * h, *pqh = block + 128 + 32 * h;
                int lo = (c & 1) ? pql[l + 32] : pql[l];
                lo = (c >= 2) ? (lo >> 4) & 0x0F : lo & 0x0F;
                code = (lo | (((pqh[l] >> (2 * c)) & 0x03) << 4)) - 32;
            } else {
                return -1;
            }
            int xb = kb * 8 + i / 32;
            const int8_t *qx = (const int8_t *)(xq8 + (int64_t)xb * 34 + 2);
            if (i % 32 == 0) sums[xb] = 0;
            sums[xb] += code * (int32_t)qx[i % 32];
        }
    }
    return 0;
}

/* Dequantise a Q8_0 activation row back to fp32 (x_hat = q * d): what the fp32
 * outputs of the quantised-activation kernels are compared against after being
 * fed through the scalar vec-dots above. */
SMO_API void smo_dequant_row_q8_0(const uint8_t *xq8, float *dst, int n)
{
    smo_read_q8_0(xq8, dst, n);
}

/* ------------------------------------------------------------------------- */
/* fp32 ops around the matmuls                                                */
/* ------------------------------------------------------------------------- */

/* SharpMind.Model/Layers/NormKernels.cs:40-60 (RMSNormParamAVX2). The AVX2 form is the one
 * RmsNormLayer runs on any AVX2 host (RmsNormLayer.cs:8-20): eight fp32 lane accumulators
 * over the body, horizontal sum, scalar tail, then 1/sqrt(ss/n + eps). */
SMO_API float smo_rmsnorm_param(const float *row, int n, float eps)
{
    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i <= n - 8; i += 8)
        for (int k = 0; k < 8; k++) {
            float sq = row[i + k] * row[i + k];
            lane[k] = lane[k] + sq;
        }
    /* MathHelpers.HSum256_Avx (SharpMind.Core/MathHelpers.cs:10-17): lo+hi, then
     * (0+2, 1+3), then the two partials. */
    float s0 = lane[0] + lane[4], s1 = lane[1] + lane[5], s2 = lane[2] + lane[6], s3 = lane[3] + lane[7];
    float t0 = s0 + s2, t1 = s1 + s3;
    float ss = t0 + t1;
    for (; i < n; i++) {
        float sq = row[i] * row[i];
        ss += sq;
    }
    float mean = ss / (float)n;
    return 1.f / sqrtf(mean + eps);
}

/* SharpMind.Model/Layers/NormKernels.cs:13-33 (RMSNormRow*): out = src * rmsInv * w, left to right */
SMO_API void smo_rmsnorm_row(const float *src, const float *w, float *dst, int n, float rmsInv)
{
    for (int i = 0; i < n; i++) {
        float t = src[i] * rmsInv;
        dst[i] = t * w[i];
    }
}

/* NormLayer.Forward (SharpMind.Model/Layers/NormLayer.cs:42-57): per row param + apply */
SMO_API void smo_rmsnorm(const float *x, const float *w, float *out, int rows, int n, float eps)
{
    for (int r = 0; r < rows; r++) {
        float p = smo_rmsnorm_param(x + (int64_t)r * n, n, eps);
        smo_rmsnorm_row(x + (int64_t)r * n, w, out + (int64_t)r * n, n, p);
    }
}

/* SharpMind.Core/Activations/ActivationKernels.cs:161-168 (SiLUScalar) */
SMO_API void smo_silu(const float *src, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; i++) {
        float x = src[i];
        dst[i] = x / (1.f + expf(-x));
    }
}

/* SharpMind.Core/Activations/ActivationKernels.cs:194-201 (SwiGLUScalar) */
SMO_API void smo_swiglu(const float *gate, const float *up, float *dst, int64_t n)
{
    for (int64_t i = 0; i < n; i++) {
        float g = gate[i];
        float s = g / (1.f + expf(-g));
        dst[i] = s * up[i];
    }
}

/* SharpMind.Core/Activations/ActivationKernels.cs:316-348 (SoftmaxRowScalar / ...Small) */
SMO_API void smo_softmax_row(const float *src, float *dst, int n)
{
    float mx = src[0];
    for (int i = 1; i < n; i++)
        if (src[i] > mx) mx = src[i];
    float sum = 0.f;
    for (int i = 0; i < n; i++) {
        dst[i] = expf(src[i] - mx);
        sum += dst[i];
    }
    float inv = 1.f / sum;
    for (int i = 0; i < n; i++)
        dst[i] *= inv;
}

/* SharpMind.Core/Embeddings/RoPE.cs:103-147 (table build, no scaling): freq_i = 1/powf(theta, 2i/ropeDim),
 * angle = (float)pos * freq_i, cos/sin tables [maxSeq, ropeDim/2]. */
SMO_API void smo_rope_tables(float theta, int ropeDim, int maxSeq, float *cosT, float *sinT)
{
    int half = ropeDim / 2;
    float *freqs = (float *)malloc(sizeof(float) * (size_t)half);
    for (int i = 0; i < half; i++) {
        float e = 2.f * (float)i / (float)ropeDim;
        freqs[i] = 1.f / powf(theta, e);
    }
    for (int pos = 0; pos < maxSeq; pos++)
        for (int i = 0; i < half; i++) {
            float angle = (float)pos * freqs[i];
            cosT[(int64_t)pos * half + i] = cosf(angle);
            sinT[(int64_t)pos * half + i] = sinf(angle);
        }
    free(freqs);
}

/* SharpMind.Core/Embeddings/RoPE.cs:168-259 (Apply) on x[seq, heads, headDim], in place.
 * neox = pairs (d, d + ropeDim/2); otherwise adjacent pairs (2i, 2i+1). */
SMO_API void smo_rope_apply(float *x, int seq, int heads, int headDim, int ropeDim, int posOffset,
                            const float *cosT, const float *sinT, int neox)
{
    int pairs = ropeDim / 2;
    for (int s = 0; s < seq; s++) {
        const float *c = cosT + (int64_t)(posOffset + s) * pairs;
        const float *sn = sinT + (int64_t)(posOffset + s) * pairs;
        for (int h = 0; h < heads; h++) {
            float *p = x + ((int64_t)s * heads + h) * headDim;
            for (int i = 0; i < pairs; i++) {
                int ia = neox ? i : 2 * i;
                int ib = neox ? i + pairs : 2 * i + 1;
                float a = p[ia], b = p[ib];
                float ac = a * c[i], bs = b * sn[i];
                float bc = b * c[i], as = a * sn[i];
                p[ia] = ac - bs;
                p[ib] = bc + as;
            }
        }
    }
}

/* SharpMind.Core/Tensors/Tensor.cs:328-332 (AddInPlace) */
SMO_API void smo_add_inplace(float *x, const float *y, int64_t n)
{
    for (int64_t i = 0; i < n; i++)
        x[i] = x[i] + y[i];
}

/* SharpMind.Inference/Sampler.cs:50-58 (Argmax: first maximum wins, strict >) */
SMO_API int smo_argmax(const float *logits, int n)
{
    int best = 0;
    float mx = logits[0];
    for (int i = 1; i < n; i++)
        if (logits[i] > mx) {
            mx = logits[i];
            best = i;
        }
    return best;
}

/* SharpMind.Model/Layers/MedusaHeads.cs:80-101 (PredictQuantized, the head transform): head h maps the normed hidden
 * state to SiLU(b_h + hidden W_h), W_h stored [j * H + i], the sum taken over j in order from the bias.
 * w [k][H][H], b [k][H], out [k][H]. */
SMO_API void smo_medusa_heads(const float *hidden, const float *w, const float *b, float *out, int k, int H)
{
    for (int h = 0; h < k; h++) {
        const float *wh = w + (int64_t)h * H * H;
        float *o = out + (int64_t)h * H;
        for (int i = 0; i < H; i++) {
            float sum = b[(int64_t)h * H + i];
            for (int j = 0; j < H; j++)
                sum += hidden[j] * wh[(int64_t)j * H + i];
            o[i] = sum;
        }
        for (int i = 0; i < H; i++)
            o[i] = o[i] / (1.0f + expf(-o[i]));
    }
}

/* SharpMind.Inference/MedusaGenerator.cs:269-283: token 0 of the draft is the model's own greedy choice and always
 * accepted; head guess i + 1 is accepted while the verification pass's greedy pick after token i equals it. */
SMO_API int smo_verify_greedy(const int *argmax, const int *draft, int heads)
{
    int accepted = 1;
    for (int i = 0; i < heads; i++) {
        if (argmax[i] != draft[i + 1]) break;
        accepted++;
    }
    return accepted;
}

/* SharpMind.Model/Layers/Attention/AttentionKernels.cs:409-475 (ScaledDotProductFlashScalar),
 * alibiSlope = 0. Tiles of 64 keys, running max / sum, O rescaled per tile. */
SMO_API void smo_sdpa_flash(const float *q, const float *k, const float *v, float *out, int seqLen,
                            int kvLen, int headDim, float scale, int causal, int qStride, int oStride)
{
    float tile[64];
    int queryBase = causal ? kvLen - seqLen : 0;
    for (int i = 0; i < seqLen; i++) {
        const float *qi = q + (int64_t)i * qStride;
        int absQ = queryBase + i;
        int eff = causal ? (absQ + 1 < kvLen ? absQ + 1 : kvLen) : kvLen;
        float mMax = -INFINITY, lSum = 0.f;
        float *o = out + (int64_t)i * oStride;
        for (int d = 0; d < headDim; d++) o[d] = 0.f;
        for (int start = 0; start < eff; start += 64) {
            int end = start + 64 < eff ? start + 64 : eff;
            int len = end - start;
            float tmax = -INFINITY;
            for (int j = start; j < end; j++) {
                const float *kj = k + (int64_t)j * headDim;
                float dot = 0.f;
                for (int d = 0; d < headDim; d++) {
                    float p = qi[d] * kj[d];
                    dot += p;
                }
                dot = dot * scale;
                tile[j - start] = dot;
                if (dot > tmax) tmax = dot;
            }
            float newMax = mMax > tmax ? mMax : tmax;
            float scaleOld = expf(mMax - newMax);
            float scaleNew = 0.f;
            for (int t = 0; t < len; t++) {
                tile[t] = expf(tile[t] - newMax);
                scaleNew += tile[t];
            }
            float so = scaleOld * lSum;
            float newL = so + scaleNew;
            for (int d = 0; d < headDim; d++) o[d] *= scaleOld;
            for (int t = 0; t < len; t++) {
                const float *vj = v + (int64_t)(start + t) * headDim;
                for (int d = 0; d < headDim; d++) {
                    float p = tile[t] * vj[d];
                    o[d] += p;
                }
            }
            mMax = newMax;
            lSum = newL;
        }
        if (lSum > 0.f)
            for (int d = 0; d < headDim; d++) o[d] /= lSum;
        else
            for (int d = 0; d < headDim; d++) o[d] = 0.f;
    }
}

/* ------------------------------------------------------------------------- */
/* one decode step of a Qwen3-shaped decoder                                  */
/* ------------------------------------------------------------------------- */

typedef struct {
    int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq;
    int dtype; /* QuantDType of every matrix */
    float eps, rope_theta;
    int neox, qk_norm;
    /* per layer, arrays of n_layers pointers */
    const uint8_t **wq, **wk, **wv, **wo, **wgu, **wdown;
    const float **norm1, **norm2, **qnorm, **knorm;
    const float *final_norm;
    const uint8_t *lm_head; /* [vocab, hidden] raw; tied models pass the embedding bytes */
    const float *embedding; /* fp32 [vocab, hidden], dequantised table */
    const float *cosT, *sinT;
    /* formats of the down projection and of the LM head / embedding when they differ from `dtype`
     * (GGUF files mix formats per tensor); 0 = same as `dtype` */
    int down_dtype, head_dtype;
    /* bias vectors of the linear layers (LinearLayer._bias): null, or n_layers pointers whose entries may be null */
    const float **bq, **bk, **bv, **bo, **bgu, **bdown;
    /* != 0: the cache is a QuantizedKVCache with Q8_0 rows (SharpMind.Model/QuantizedKVCache.cs:84-126): every appended K
     * and V head row is quantised by QuantizeRowQ8_0; the cache here keeps the values those blocks decode to (val * d),
     * which is what ScaledDotProductFlashQ8_0* multiplies by. */
    int kv_q8;
} smo_model;

/* LinearLayer.AddBiasInPlace (SharpMind.Model/Layers/Linearlayer.cs:154-163): row[j] += bias[j] for every row. */
static void add_bias(float *out, const float **per_layer, int layer, int rows, int n)
{
    if (!per_layer || !per_layer[layer]) return;
    const float *bias = per_layer[layer];
    for (int i = 0; i < rows; i++)
        for (int j = 0; j < n; j++) out[(size_t)i * n + j] += bias[j];
}

/* The matmul of the decode step.  act_q8 == 0: the reference's own arithmetic (fp32 activations into the scalar
 * vec-dot).  act_q8 != 0: what the CUDA library's SMC_ACT_Q8 mode is specified to compute -- every activation row is
 * first quantised to Q8_0 blocks by the rules of QuantizedKVCache.QuantizeRowQ8_0
 * (SharpMind.Model/QuantizedKVCache.cs:191-223, restated in smo_quantize_row_q8_0) and the scalar vec-dot is fed the
 * dequantised row -- so that a decode step in that mode can be held to the same bound as a single matmul. */
static int step_matmul(int act_q8, int dtype, const float *in, const uint8_t *raw, float *out, int M, int K, int N)
{
    if (!act_q8) return smo_qmatmul(dtype, in, raw, out, M, K, N);
    if (K % 32) return -5;
    uint8_t *q = malloc((size_t)(K / 32) * 34);
    float *hat = malloc(sizeof(float) * (size_t)M * K);
    if (!q || !hat) { free(q); free(hat); return -2; }
    for (int r = 0; r < M; r++) {
        smo_quantize_row_q8_0(in + (size_t)r * K, q, K);
        smo_dequant_row_q8_0(q, hat + (size_t)r * K, K);
    }
    int rc = smo_qmatmul(dtype, hat, raw, out, M, K, N);
    free(q); free(hat);
    return rc;
}

/* Follows Transformer.ForwardLastLogits (SharpMind.Model/Transformer.cs:417-463),
 * DecoderArch.Forward (SharpMind.Model/Arch/DecoderArch.cs:115-134),
 * UnhookedTransformerBlock.Forward (SharpMind.Model/Layers/UnhookedTransformerBlock.cs:12-47),
 * AttentionLayer.Forward (SharpMind.Model/Layers/Attention/AttentionLayer.cs:260-422),
 * FfnKernels.Gated (SharpMind.Model/Layers/Ffn/FfnKernels.cs:35-59),
 * KVCache.Update (SharpMind.Model/KVCache.cs:84-150) for seqLen == 1 and `batch`
 * lock-step sequences.  kcache / vcache are [layer][batch][kvHead][max_seq][head_dim]
 * fp32 and already hold positions [0, pos).  Writes logits [batch, vocab].
 * act_q8: see step_matmul. */
SMO_API int smo_decode_step_ex(const smo_model *m, const int *tokens, int batch, int pos, float *kcache,
                               float *vcache, float *logits, int act_q8)
{
    int H = m->hidden, nh = m->n_heads, nkv = m->n_kv_heads, hd = m->head_dim, F = m->ffn;
    int qDim = nh * hd, kvDim = nkv * hd;
    float scale = 1.f / sqrtf((float)hd);
    size_t B = (size_t)batch;
    float *x = malloc(sizeof(float) * B * H), *xn = malloc(sizeof(float) * B * H);
    float *q = malloc(sizeof(float) * B * qDim), *k = malloc(sizeof(float) * B * kvDim);
    float *v = malloc(sizeof(float) * B * kvDim), *att = malloc(sizeof(float) * B * qDim);
    float *tmp = malloc(sizeof(float) * B * H), *gu = malloc(sizeof(float) * B * 2 * F);
    float *act = malloc(sizeof(float) * B * F);
    int rc = 0;
    if (!x || !xn || !q || !k || !v || !att || !tmp || !gu || !act) { rc = -2; goto done; }
    if (pos + 1 > m->max_seq) { rc = -3; goto done; }
    for (int b = 0; b < batch; b++) {
        if (tokens[b] < 0 || tokens[b] >= m->vocab) { rc = -4; goto done; }
        memcpy(x + (size_t)b * H, m->embedding + (size_t)tokens[b] * H, sizeof(float) * H);
    }
    size_t layerStride = B * nkv * (size_t)m->max_seq * hd;
    for (int L = 0; L < m->n_layers; L++) {
        smo_rmsnorm(x, m->norm1[L], xn, batch, H, m->eps);
        if ((rc = step_matmul(act_q8, m->dtype, xn, m->wq[L], q, batch, H, qDim))) goto done;
        if ((rc = step_matmul(act_q8, m->dtype, xn, m->wk[L], k, batch, H, kvDim))) goto done;
        if ((rc = step_matmul(act_q8, m->dtype, xn, m->wv[L], v, batch, H, kvDim))) goto done;
        add_bias(q, m->bq, L, batch, qDim), add_bias(k, m->bk, L, batch, kvDim), add_bias(v, m->bv, L, batch, kvDim);
        if (m->qk_norm) {
            smo_rmsnorm(q, m->qnorm[L], q, batch * nh, hd, m->eps);
            smo_rmsnorm(k, m->knorm[L], k, batch * nkv, hd, m->eps);
        }
        for (int b = 0; b < batch; b++) {
            smo_rope_apply(q + (size_t)b * qDim, 1, nh, hd, hd, pos, m->cosT, m->sinT, m->neox);
            smo_rope_apply(k + (size_t)b * kvDim, 1, nkv, hd, hd, pos, m->cosT, m->sinT, m->neox);
        }
        float *kc = kcache + (size_t)L * layerStride, *vc = vcache + (size_t)L * layerStride;
        for (int b = 0; b < batch; b++)
            for (int h = 0; h < nkv; h++) {
                size_t dst = (((size_t)b * nkv + h) * m->max_seq + pos) * hd;
                float *krow = k + (size_t)b * kvDim + (size_t)h * hd, *vrow = v + (size_t)b * kvDim + (size_t)h * hd;
                if (m->kv_q8) {
                    uint8_t blocks[8 * 34];
                    if (hd > 256 || hd % 32) { rc = -6; goto done; }
                    smo_quantize_row_q8_0(krow, blocks, hd);
                    smo_dequant_row_q8_0(blocks, krow, hd);
                    smo_quantize_row_q8_0(vrow, blocks, hd);
                    smo_dequant_row_q8_0(blocks, vrow, hd);
                }
                memcpy(kc + dst, krow, sizeof(float) * hd);
                memcpy(vc + dst, vrow, sizeof(float) * hd);
            }
        int kvLen = pos + 1;
        int group = nh / nkv;
        for (int b = 0; b < batch; b++)
            for (int h = 0; h < nh; h++) {
                int kvh = h / group;
                size_t base = ((size_t)b * nkv + kvh) * m->max_seq * hd;
                smo_sdpa_flash(q + (size_t)b * qDim + (size_t)h * hd, kc + base, vc + base,
                               att + (size_t)b * qDim + (size_t)h * hd, 1, kvLen, hd, scale, 1, qDim, qDim);
            }
        if ((rc = step_matmul(act_q8, m->dtype, att, m->wo[L], tmp, batch, qDim, H))) goto done;
        add_bias(tmp, m->bo, L, batch, H);
        smo_add_inplace(x, tmp, (int64_t)B * H);
        smo_rmsnorm(x, m->norm2[L], xn, batch, H, m->eps);
        if ((rc = step_matmul(act_q8, m->dtype, xn, m->wgu[L], gu, batch, H, 2 * F))) goto done;
        add_bias(gu, m->bgu, L, batch, 2 * F);
        for (int b = 0; b < batch; b++)
            smo_swiglu(gu + (size_t)b * 2 * F, gu + (size_t)b * 2 * F + F, act + (size_t)b * F, F);
        if ((rc = step_matmul(act_q8, m->down_dtype ? m->down_dtype : m->dtype, act, m->wdown[L], tmp, batch, F, H))) goto done;
        add_bias(tmp, m->bdown, L, batch, H);
        smo_add_inplace(x, tmp, (int64_t)B * H);
    }
    smo_rmsnorm(x, m->final_norm, x, batch, H, m->eps);
    rc = step_matmul(act_q8, m->head_dtype ? m->head_dtype : m->dtype, x, m->lm_head, logits, batch, H, m->vocab);
done:
    free(x); free(xn); free(q); free(k); free(v); free(att); free(tmp); free(gu); free(act);
    return rc;
}

SMO_API int smo_decode_step(const smo_model *m, const int *tokens, int batch, int pos, float *kcache,
                            float *vcache, float *logits)
{
    return smo_decode_step_ex(m, tokens, batch, pos, kcache, vcache, logits, 0);
}

/* ------------------------------------------------------------------------- */
/* sampler                                                                    */
/* ------------------------------------------------------------------------- */

/* RepetitionPenalty.Apply (SharpMind.Inference/RepetitionPenalty.cs:15-27): every DISTINCT id of the window
 * scales its logit once: positive logits are divided by the penalty, negative ones multiplied. */
SMO_API void smo_repetition_penalty(float *logits, int n, const int *ids, int count, float penalty)
{
    for (int i = 0; i < count; i++) {
        int id = ids[i], seen = 0;
        for (int j = 0; j < i; j++)
            if (ids[j] == id) { seen = 1; break; }
        if (seen || id < 0 || id >= n) continue;
        logits[id] = logits[id] >= 0.f ? logits[id] / penalty : logits[id] * penalty;
    }
}

static void sift_down(float *vals, int *idxs, int pos, int heap)
{
    for (;;) {
        int smallest = pos, l = 2 * pos + 1, r = 2 * pos + 2;
        if (l < heap && vals[l] < vals[smallest]) smallest = l;
        if (r < heap && vals[r] < vals[smallest]) smallest = r;
        if (smallest == pos) break;
        float tv = vals[pos]; vals[pos] = vals[smallest]; vals[smallest] = tv;
        int ti = idxs[pos]; idxs[pos] = idxs[smallest]; idxs[smallest] = ti;
        pos = smallest;
    }
}

typedef struct { float v; int i; } smo_vi;
static int cmp_vi(const void *a, const void *b)
{
    const smo_vi *x = a, *y = b;
    if (x->v < y->v) return -1;
    if (x->v > y->v) return 1;
    return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0); /* the reference's sort leaves the order of equal values open */
}

/* Sampler.Sample (SharpMind.Inference/Sampler.cs:16-46) with the uniform number `r` that rng.NextSingle() would
 * have produced handed in by the caller: temperature (:62-66), guarded softmax (:70-100), min-p (:222-229),
 * top-k by heap select (:109-161), top-p over an ascending sort walked from the top (:189-225), normalise
 * (:233-240), categorical draw (:244-257).  temperature <= 0 is the greedy shortcut (Argmax, :50-58). */
SMO_API int smo_sample_ex(const float *logits, int n, float temperature, int topK, float topP, float minP, float r,
                          float *probs_out);
SMO_API int smo_sample(const float *logits, int n, float temperature, int topK, float topP, float minP, float r)
{
    return smo_sample_ex(logits, n, temperature, topK, topP, minP, r, NULL);
}

/* The same; probs_out (n floats, may be null) receives the normalised probabilities the draw was made from. */
SMO_API int smo_sample_ex(const float *logits, int n, float temperature, int topK, float topP, float minP, float r,
                          float *probs_out)
{
    if (temperature <= 0.f) return smo_argmax(logits, n);
    float *p = malloc(sizeof(float) * (size_t)n);
    float *vals = malloc(sizeof(float) * (size_t)n);
    int *idxs = malloc(sizeof(int) * (size_t)n);
    int result = 0;
    if (!p || !vals || !idxs) { result = -1; goto done; }
    float inv = 1.f / temperature;
    for (int i = 0; i < n; i++) p[i] = logits[i] * inv;
    /* softmax */
    int bad = 0;
    for (int i = 0; i < n; i++)
        if (isinf(p[i]) || isnan(p[i])) { bad = 1; break; }
    if (bad) {
        memset(p, 0, sizeof(float) * (size_t)n);
        p[0] = 1.f;
    } else {
        float mx = p[0];
        for (int i = 0; i < n; i++) if (p[i] > mx) mx = p[i];
        float sum = 0.f;
        for (int i = 0; i < n; i++) {
            float e = p[i] - mx;
            if (e > 80.f) e = 80.f; else if (e < -80.f) e = -80.f;
            p[i] = expf(e);
            sum += p[i];
        }
        float is = 1.f / sum;
        for (int i = 0; i < n; i++) p[i] *= is;
    }
    if (minP > 0.f) {
        float mx = 0.f;
        for (int i = 0; i < n; i++) if (p[i] > mx) mx = p[i];
        float thr = minP * mx;
        for (int i = 0; i < n; i++) if (p[i] < thr) p[i] = 0.f;
    }
    if (topK > 0 && topK < n) {
        int count = 0;
        for (int i = 0; i < n; i++) if (p[i] > 0.f) { vals[count] = p[i]; idxs[count] = i; count++; }
        if (count > topK) {
            for (int i = topK / 2 - 1; i >= 0; i--) sift_down(vals, idxs, i, topK);
            for (int i = topK; i < count; i++)
                if (vals[i] > vals[0]) {
                    float tv = vals[0]; vals[0] = vals[i]; vals[i] = tv;
                    int ti = idxs[0]; idxs[0] = idxs[i]; idxs[i] = ti;
                    sift_down(vals, idxs, 0, topK);
                }
            for (int i = topK; i < count; i++) p[idxs[i]] = 0.f;
        }
    }
    if (topP < 1.0f && topP > 0.f) {
        smo_vi *s = malloc(sizeof(smo_vi) * (size_t)n);
        if (!s) { result = -1; goto done; }
        int count = 0;
        for (int i = 0; i < n; i++) if (p[i] > 0.f) { s[count].v = p[i]; s[count].i = i; count++; }
        qsort(s, (size_t)count, sizeof(smo_vi), cmp_vi);
        float cum = 0.f;
        for (int i = count - 1; i >= 0; i--) {
            cum += s[i].v;
            if (cum >= topP) {
                for (int j = i - 1; j >= 0; j--) p[s[j].i] = 0.f;
                break;
            }
        }
        free(s);
    }
    {
        float sum = 0.f;
        for (int i = 0; i < n; i++) sum += p[i];
        if (sum > 0.f) {
            float is = 1.f / sum;
            for (int i = 0; i < n; i++) p[i] *= is;
        }
    }
    if (probs_out) memcpy(probs_out, p, sizeof(float) * (size_t)n);
    {
        float cum = 0.f;
        result = -2;
        for (int i = 0; i < n; i++) {
            cum += p[i];
            if (r <= cum) { result = i; break; }
        }
        if (result == -2) {
            result = 0;
            for (int i = n - 1; i >= 0; i--) if (p[i] > 0.f) { result = i; break; }
        }
    }
done:
    free(p); free(vals); free(idxs);
    return result;
}

/* SharpMind.Model/Layers/Attention/AttentionKernels.cs:724-813 (ScaledDotProductFlashQ8_0Scalar), alibiSlope = 0:
 * keys and values are rows of Q8_0 blocks (fp16 d + 32 int8, headDim/32 blocks per row, colStride bytes apart);
 * the key dot is summed in fp64 over (q * (val * d)) products formed in fp32, the rest is the fp32 flash recurrence. */
SMO_API void smo_sdpa_flash_q8(const float *q, const uint8_t *kQuant, const uint8_t *vQuant, float *out, int seqLen,
                               int kvLen, int headDim, float scale, int causal, int qStride, int oStride)
{
    float tile[64];
    int nBlocks = (headDim + 31) / 32, colStride = nBlocks * 34;
    int queryBase = causal ? kvLen - seqLen : 0;
    for (int i = 0; i < seqLen; i++) {
        const float *qi = q + (int64_t)i * qStride;
        int absQ = queryBase + i;
        int eff = causal ? (absQ + 1 < kvLen ? absQ + 1 : kvLen) : kvLen;
        float mMax = -INFINITY, lSum = 0.f;
        float *o = out + (int64_t)i * oStride;
        for (int d = 0; d < headDim; d++) o[d] = 0.f;
        for (int start = 0; start < eff; start += 64) {
            int end = start + 64 < eff ? start + 64 : eff;
            int len = end - start;
            float tmax = -INFINITY;
            for (int j = start; j < end; j++) {
                const uint8_t *kj = kQuant + (int64_t)j * colStride;
                double dot = 0;
                for (int b = 0; b < nBlocks; b++) {
                    const uint8_t *bp = kj + b * 34;
                    float d = smo_half_to_float((uint16_t)(bp[0] | (bp[1] << 8)));
                    const int8_t *vals = (const int8_t *)(bp + 2);
                    int blockEnd = headDim - b * 32 < 32 ? headDim - b * 32 : 32;
                    for (int k = 0; k < blockEnd; k++) {
                        float w = (float)vals[k] * d;
                        float p = qi[b * 32 + k] * w;
                        dot += p;
                    }
                }
                float score = (float)dot * scale;
                tile[j - start] = score;
                if (score > tmax) tmax = score;
            }
            float newMax = mMax > tmax ? mMax : tmax;
            float scaleOld = expf(mMax - newMax);
            float scaleNew = 0.f;
            for (int t = 0; t < len; t++) {
                tile[t] = expf(tile[t] - newMax);
                scaleNew += tile[t];
            }
            float so = scaleOld * lSum;
            float newL = so + scaleNew;
            for (int d = 0; d < headDim; d++) o[d] *= scaleOld;
            for (int t = 0; t < len; t++) {
                const uint8_t *vj = vQuant + (int64_t)(start + t) * colStride;
                float sm = tile[t];
                for (int b = 0; b < nBlocks; b++) {
                    const uint8_t *bp = vj + b * 34;
                    float d = smo_half_to_float((uint16_t)(bp[0] | (bp[1] << 8)));
                    const int8_t *vals = (const int8_t *)(bp + 2);
                    int blockEnd = headDim - b * 32 < 32 ? headDim - b * 32 : 32;
                    for (int k = 0; k < blockEnd; k++) {
                        float w = (float)vals[k] * d;
                        float p = sm * w;
                        o[b * 32 + k] += p;
                    }
                }
            }
            mMax = newMax;
            lSum = newL;
        }
        if (lSum > 0.f)
            for (int d = 0; d < headDim; d++) o[d] /= lSum;
        else
            for (int d = 0; d < headDim; d++) o[d] = 0.f;
    }
}
