// Shared declarations of the CUDA backend: context / weight / activation-buffer objects and the
// small device helpers every kernel file uses.  Built for sm_100a only, with -fmad=false: every
// fused multiply-add in this library is written explicitly (fmaf), so that code restating the
// reference's unfused arithmetic keeps its roundings.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>
#include <unordered_map>

#include "../../include/sharpmind_cuda.h"

#define SMC_QK 32
#define SMC_QK_K 256

struct smc_weight {
    int dtype = 0, N = 0, K = 0, flags = 0;
    size_t raw_bytes = 0;
    const void *host_key = nullptr;
    uint8_t *d_raw = nullptr;  // GGUF layout (compute layout for Q4_K)
    bool fast = false;         // shape and layout allow the vectorised kernels
    // Q8_0 planes: quants [N][K] int8 and scales [N][K/32] fp16
    int8_t *q8_qs = nullptr;
    __half *q8_d = nullptr;
    // Q6_K compute layout: units of eight 256-element blocks in flat-tensor order, SMC_Q6U_BYTES each (see below)
    uint8_t *q6u = nullptr;
};

// Q6_K compute layout.  Eight consecutive blocks (2048 elements) form one unit of 1680 bytes, the same byte
// count as their GGUF form, laid out for the lanes of a warp: "lane slot" s = 4*b + 2*h + o names block b (0..7)
// of the unit, half h (128 elements) and sixteen o (elements l = 16*o .. 16*o + 15 of each 32-element column).
//   [   0,  512)  X: 16 bytes per lane slot; byte i = code(c=0, l) | (code(c=3, l) & 3) << 6        l = 16*o + i
//   [ 512, 1024)  Y: byte i = code(c=1, l) | ((code(c=3, l) >> 2) & 3) << 6
//   [1024, 1536)  Z: byte i = code(c=2, l) | ((code(c=3, l) >> 4) & 3) << 6
//   [1536, 1664)  the sixteen int8 scales of each block, 16 bytes per block
//   [1664, 1680)  the fp16 d of each block
// code(c, l) is the six-bit value of element 128*h + 32*c + l of the block (VecDotQ6K_Scalar's q1..q4 for c = 0..3,
// QuantizationKernels.Q6.cs:28-41).  Three of the four code words of a lane are one AND away; a quarter warp reads
// 128 contiguous bytes of each of X, Y, Z, so shared-memory reads of a unit are free of bank conflicts.
#define SMC_Q6U_BYTES 1680
#define SMC_Q6U_Y 512
#define SMC_Q6U_Z 1024
#define SMC_Q6U_SC 1536
#define SMC_Q6U_D 1664
// byte offset of lane slot (blk & 7, h, o) inside the X plane of block blk's unit (add SMC_Q6U_Y / _Z for the others)
__host__ __device__ inline size_t smc_q6u_slot(size_t blk, int h, int o)
{
    return (blk >> 3) * SMC_Q6U_BYTES + 16 * (4 * (blk & 7) + 2 * h + o);
}
__host__ __device__ inline size_t smc_q6u_scales(size_t blk) { return (blk >> 3) * SMC_Q6U_BYTES + SMC_Q6U_SC + 16 * (blk & 7); }
__host__ __device__ inline size_t smc_q6u_d(size_t blk) { return (blk >> 3) * SMC_Q6U_BYTES + SMC_Q6U_D + 2 * (blk & 7); }
__host__ __device__ inline size_t smc_q6u_bytes(size_t nblk) { return ((nblk + 7) >> 3) * SMC_Q6U_BYTES; }

// Q8_0-quantised activations in structure-of-arrays form.
struct smc_q8act {
    int max_rows = 0, max_k = 0;
    int M = 0, K = 0;          // shape of the rows currently held
    int8_t *q = nullptr;       // [M][K]
    float *d = nullptr;        // [M][K/32]  fp16-rounded block scale widened to fp32
    uint16_t *dbits = nullptr; // [M][K/32]  the fp16 bit pattern itself
    float *sd = nullptr;       // [M][K/32]  d * sum(q) over the block (Q4_K's min term)
    int16_t *s16 = nullptr;    // [M][K/16]  sum(q) over each half block (Q6_K's -32 offset)
};

struct smc_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;  // used by the host-pointer entry points
    std::mutex mu;
    std::mutex mu_scratch;  // guards the kernels' own scratch buffers (taken with or without `mu` held)
    std::mutex mu_error;    // guards last_error
    std::string last_error;
    std::unordered_map<const void *, smc_weight *> by_host;
    // staging for host-pointer calls (grown on demand)
    float *d_stage_in = nullptr, *d_stage_out = nullptr, *d_stage_aux = nullptr;
    size_t stage_in_cap = 0, stage_out_cap = 0, stage_aux_cap = 0;
    void *h_pin = nullptr;
    size_t h_pin_cap = 0;
    // scratch owned by the context
    smc_q8act *act = nullptr;          // activations of smc_qmatmul_dev(SMC_ACT_Q8)
    const void *pin_seen[4] = {nullptr, nullptr, nullptr, nullptr};  // host buffers lately classified as page-locked or not (under mu)
    bool pin_is[4] = {false, false, false, false};
    unsigned pin_next = 0;
    smc_q8act *digits = nullptr;       // the three int8 digit planes of fp32 activations, stacked as 3 M rows (SMC_ACT_F32)
    size_t digits_cap = 0;             // values it holds
    float *d_digit_out = nullptr;      // their products [3 M, N]
    size_t digit_out_cap = 0;
    int f32_digits = 1;                // that path on (0: the CUDA-core kernel at every batch size)
    int f32_digits_row_mb = 32;        // one row: K-quant matrices of at least this many MB take that path too (0: never)
    int *d_status = nullptr;           // raised by a kernel whose bounded wait ran out
    bool use_pdl = true;               // programmatic dependent launch (smc_set_option "pdl")
    int tma_slots = 0, tma_ss = 0, tma_ctas = 0;  // one-row GEMV ring geometry and grid, 0 = built-in choice (smc_set_option)
    int tma_warps = 0;                            // warps per CTA of the one-row GEMV: 24 (one CTA per SM, default) or 12 (two)
    int tma_pre = 1;                              // stages requested before the activation loads are issued
    int attn_mma = 1;                             // prompt attention on the tensor cores (0: the fp32 CUDA-core kernel)
    int tma_cluster = 1;                          // one-row kernel: SM pairs share the quantisation of a long fp32 row
    int q8_prefill_tc = 1;                        // SMC_ACT_Q8, Q4_K, 64 rows and more: contraction on the tcgen05 kernel
    int ffn_fuse_max = 16384;                     // one-row decode: widest FFN whose SiLU-gate rides in the down projection's staging
    int attn_hpc = 0;                             // query heads per CTA of that kernel: 0 = two where heads share a KV head, 1 = always one
    int mt_ring = 0;                              // 2..32 rows, weights through the bulk-copy ring: 0 never, 1 Q4_K, 2 every format
    void *d_argmax = nullptr;          // chunk results and tickets of the argmax
    int argmax_rows = 0, argmax_chunks = 0;
    void *d_prefill = nullptr;         // activation image of the tensor-core matmul
    size_t prefill_cap = 0;
    float *d_attn_part = nullptr;      // split-KV partial results
    size_t attn_part_cap = 0;
};

int smc_fail(smc_ctx *ctx, int code, const char *fmt, ...);

#define SMC_CUDA(ctx, call)                                                                     \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess)                                                                  \
            return smc_fail((ctx), SMC_E_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

#define SMC_LAUNCH_CHECK(ctx)                                                                            \
    do {                                                                                                 \
        cudaError_t e_ = cudaGetLastError();                                                             \
        if (e_ != cudaSuccess)                                                                           \
            return smc_fail((ctx), SMC_E_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(e_), \
                            __FILE__, __LINE__);                                                         \
    } while (0)

// ---- launchers implemented across the .cu files (all asynchronous on `s`) ----
int smc_launch_gemv_f32(smc_ctx *, const float *x, const smc_weight *, float *out, int M, cudaStream_t s);
int smc_launch_gemv_q8(smc_ctx *, const smc_q8act *, const smc_weight *, float *out, cudaStream_t s);
bool smc_tma_supported(const smc_weight *, int M);
int smc_launch_gemv_tma(smc_ctx *, const smc_q8act *, const smc_weight *, float *out, cudaStream_t s);
int smc_launch_gemv_tma_f32in(smc_ctx *, const float *x, const smc_weight *, float *out, cudaStream_t s);
struct smc_gather_dev;
struct smc_gather;
int smc_launch_gemv_tma_xg(smc_ctx *, const smc_q8act *, const float *xf, const smc_weight *, float *out,
                           const smc_gather_dev *, cudaStream_t s);
// Residual add + RMSNorm folded into the staging of a one-row matmul: row = RMSNorm(x + add) * w, x + add -> sum.
struct smc_norm_prologue {
    const float *add;  // may be null
    const float *w;
    float *sum;        // may be null
    float eps;
};
int smc_launch_gemv_tma_full(smc_ctx *, const smc_q8act *, const float *xf, const float *xu, const smc_norm_prologue *,
                             const smc_weight *, float *out, const smc_gather_dev *, cudaStream_t s);
int smc_launch_gemv_tma_any(smc_ctx *, const smc_q8act *, const float *xf, const float *xu, const smc_norm_prologue *,
                            const smc_weight *, float *out, const smc_gather_dev *, bool reduce, bool pairs, cudaStream_t);
int smc_launch_gemv_tma_addnorm(smc_ctx *, const float *x, const smc_norm_prologue *, const smc_weight *, float *out,
                                cudaStream_t s);
int smc_launch_gemv_tma_swiglu(smc_ctx *, const float *gate, const float *up, const smc_weight *, float *out, cudaStream_t s);
int smc_launch_gemv_tma_gather(smc_ctx *, const float *x, const smc_weight *, float *out, const smc_gather_dev *,
                               cudaStream_t s);
int smc_qmatmul_dev_gather(smc_ctx *, const float *d_in, const smc_weight *, float *d_out, int M, int mode, cudaStream_t s,
                           const smc_gather_dev *, bool *fused);
bool smc_prefill_supported(const smc_weight *, int M);
int smc_launch_prefill_q4k(smc_ctx *, const float *x, const smc_weight *, float *out, int M, cudaStream_t s);
int smc_launch_prefill_q4k_q8(smc_ctx *, const smc_q8act *a, const smc_weight *, float *out, cudaStream_t s, bool scratch_locked = false);
bool smc_mma_supported(const smc_weight *, int M);
bool smc_mt_supported(const smc_weight *, int M);
bool smc_sdpa_prefill_mma_supported(int nh, int nkv, int hd);
int smc_launch_sdpa_prefill_mma(smc_ctx *, const float *q, const float *kc, const float *vc, float *out, int T, int nh, int nkv, int hd,
                                int pos0, int maxSeq, float scale, cudaStream_t s);
int smc_launch_sdpa_prefill_mma_q8(smc_ctx *ctx, const float *q, const int8_t *kq, const __half *kd, const int8_t *vq, const __half *vd,
                                   float *out, int T, int nh, int nkv, int hd, int pos0, int maxSeq, float scale, cudaStream_t s);
int smc_launch_gemv_mt(smc_ctx *, const smc_q8act *, const smc_weight *, float *out, cudaStream_t s);
int smc_launch_gemv_mma(smc_ctx *, const smc_q8act *, const smc_weight *, float *out, cudaStream_t s);
int smc_launch_gemv_ref(smc_ctx *, const float *x, const smc_weight *, float *out, int M, int col0, int col1,
                        cudaStream_t s);
int smc_launch_add_rmsnorm_q8(smc_ctx *ctx, float *d_x, const float *d_y, const float *d_w, float *d_out, int rows, int n, float eps,
                              smc_q8act *a, cudaStream_t s);
int smc_launch_quantize_q8_digits(smc_ctx *ctx, const float *x, int M, int K, smc_q8act *a, cudaStream_t s);
int smc_launch_sum3(smc_ctx *ctx, const float *y, float *out, long long n, cudaStream_t s);
int smc_launch_swiglu_quantize_q8(smc_ctx *ctx, const float *gate, const float *up, int M, int K, int ld, smc_q8act *a,
                                  cudaStream_t s);
int smc_launch_quantize_q8(smc_ctx *, const float *x, int M, int K, smc_q8act *, cudaStream_t s);
int smc_launch_block_isums(smc_ctx *, const smc_q8act *, int m, const smc_weight *, int col0, int col1,
                           int32_t *sums, cudaStream_t s);
int smc_launch_quantize_weights(smc_ctx *, int dtype, const float *v, int64_t n, void *raw, cudaStream_t s);
int smc_launch_repack(smc_ctx *, smc_weight *, cudaStream_t s);
int smc_sdpa_decode_any(smc_ctx *, const float *d_q, const void *d_k, const void *d_v, const __half *d_kd, const __half *d_vd,
                        float *d_out, int batch, int heads, int kvHeads, int headDim, int kvLen, int maxSeq, float scale,
                        cudaStream_t stream);
int smc_launch_sdpa_q8_rows(smc_ctx *ctx, const float *q, const int8_t *kq, const __half *kd, const int8_t *vq, const __half *vd, float *out,
                            int batch, int seqLen, int heads, int kvHeads, int hd, int kvLen, int maxSeq, float scale, cudaStream_t s);
int smc_sdpa_decode_reserve(smc_ctx *, int max_batch, int heads, int kvHeads, int headDim, int maxSeq);
int smc_launch_sdpa_prefill(smc_ctx *ctx, const float *q, const float *kc, const float *vc, float *out, int T, int nh, int nkv,
                            int hd, int pos0, int maxSeq, float scale, cudaStream_t s);
int smc_launch_sdpa_tile(smc_ctx *, const float *q, const float *k, const float *v, float *o, int seqLen, int kvLen,
                         int hd, float scale, int causal, int qStride, int oStride, float alibi, cudaStream_t s);
int smc_launch_rmsnorm_row(smc_ctx *, const float *src, const float *w, float *dst, int n, float rms_inv,
                           cudaStream_t s);
int smc_q8act_alloc(smc_ctx *, int max_rows, int max_k, smc_q8act **out);
void smc_q8act_free(smc_q8act *);

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------------------------
// Kernels of a decode step are a few microseconds each, so the gap between two dependent launches costs as much
// as the kernels.  A kernel launched through smc_launch_dep may be scheduled while its predecessor in the stream
// is still running; it must call smc_grid_dep_sync() before it touches anything the predecessor wrote or still
// reads (everything but weights and its own shared memory).  The wait returns when the predecessor has completed
// and its memory is visible; the trigger that follows lets the next kernel in the stream be scheduled in turn
// (only once every CTA of this grid is resident or done, so a dependent can never starve its predecessor).
// Launched the ordinary way, the same kernels run unchanged: both instructions are then no-ops.
__device__ __forceinline__ void smc_grid_dep_sync()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <class... KArgs, class... Args>
inline void smc_launch_dep(bool allow_overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                           Args... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = allow_overlap ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the grid's CTAs paired into thread-block clusters of `cluster_x` (the grid must be a multiple of it).
template <class... KArgs, class... Args>
inline void smc_launch_dep_cluster(bool allow_overlap, int cluster_x, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                   cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)cluster_x, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at, cfg.numAttrs = allow_overlap ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float smc_h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

// 16-byte streaming load: weights are read once, keep them out of L1.
__device__ __forceinline__ uint4 smc_ldg_stream16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ float4 smc_ldg_stream16f(const float *p)
{
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 smc_ldg_stream8(const void *p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t smc_ldg_stream4(const void *p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t smc_ldg_stream2(const void *p)
{
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ int smc_dp4a(uint32_t a, uint32_t b, int c)
{
    return __dp4a((int)a, (int)b, c);  // signed x signed bytes
}
__device__ __forceinline__ int smc_dp4a_us(uint32_t a_unsigned, uint32_t b_signed, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
    return d;
}

// Byte j (0..3) of w as an exact float, through the 2^23 mantissa trick: one PRMT and one FADD,
// both full-rate, instead of a quarter-rate integer-to-float conversion.
__device__ __forceinline__ float smc_ubyte_to_float(uint32_t w, int j)
{
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | j)) - 8388608.0f;
}

template <int LANES>
__device__ __forceinline__ float smc_group_sum(float v)
{
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float smc_group_sum_rt(float v, int lanes)
{
    for (int o = lanes / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The four code words of a lane slot's word j (bytes l = 16*o + 4*j .. + 3) from its X, Y, Z words: q[c] holds the
// six-bit codes of column c, one per byte.
__device__ __forceinline__ void smc_q6u_codes(uint32_t X, uint32_t Y, uint32_t Z, uint32_t (&q)[4])
{
    const uint32_t M6 = 0x3F3F3F3Fu;
    q[0] = X & M6;
    q[1] = Y & M6;
    q[2] = Z & M6;
    q[3] = ((X >> 6) & 0x03030303u) | ((Y >> 4) & 0x0C0C0C0Cu) | ((Z >> 2) & 0x30303030u);
}

// Q4_K / Q5_K 6-bit scale and min of sub-block j (0..7) from the 12 packed bytes held as three
// little-endian words (GetScaleMinK4_*, QuantizationKernels.cs:177-189).
__device__ __forceinline__ void smc_k4_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, int &sc, int &mn)
{
    // bytes 0..3 = s0, 4..7 = s1, 8..11 = s2
    if (j < 4) {
        sc = (s0 >> (8 * j)) & 0x3F;
        mn = (s1 >> (8 * j)) & 0x3F;
    } else {
        int jj = j - 4;
        uint32_t b8 = (s2 >> (8 * jj)) & 0xFF;   // scales[j + 4]
        uint32_t lo = (s0 >> (8 * jj)) & 0xFF;   // scales[j - 4]
        uint32_t mid = (s1 >> (8 * jj)) & 0xFF;  // scales[j]
        sc = (b8 & 0x0F) | ((lo >> 6) << 4);
        mn = (b8 >> 4) | ((mid >> 6) << 4);
    }
}
#endif  // __CUDACC__
