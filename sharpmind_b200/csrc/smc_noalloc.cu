// smc_qmatmul_q8_noalloc: the quantised-activation matmul for callers that must not allocate.
//
// Who needs it.  smc_qmatmul_dev(SMC_ACT_Q8) keeps the Q8_0 form of the activations in a buffer that
// the context allocates (and grows) with cudaMalloc on first use.  Some hosts cannot afford that call:
// a serving loop that sized all of its GPU memory at start-up (weights, KV caches) may have nothing left
// to give, cudaMalloc synchronises the whole device and so stalls every other stream of the process, and
// some embedding applications simply forbid driver allocations once initialisation is over.  For them this
// entry point does the same two launches (quantise the rows, run the GEMV) with the intermediate buffer
// placed in a fixed array that is part of the library image.
//
// What it costs.  The array below is SMC_NOALLOC_MAX_ELEMS activations large (about 0.75 MB) and exists on
// every GPU that loads the library, from load until the process exits, whether or not this entry point is
// ever called.  Shapes with M * K beyond that limit are refused with SMC_E_RANGE.
//
// Rules of use.  All calls on a device share the one array, and it keeps whatever the previous call left
// in it.  Nothing has to be cleared: the quantiser writes every entry the GEMV will read before the GEMV
// starts (same stream, in order).  Two calls whose kernels can run at the same time on one GPU (different
// streams, or different host threads) would overwrite each other's activations: callers must order them.
// The very first call on a device looks up the array's device address; make that first call during
// set-up, outside any stream capture.  No allocation routine (cudaMalloc, cudaFree, cudaMallocAsync, or any
// library that allocates) is called here or by the launchers this file uses.
#include "smc_common.cuh"

namespace {

constexpr size_t kMaxElems = SMC_NOALLOC_MAX_ELEMS;  // M * K
// layout inside the array (all offsets multiples of 256 bytes):
//   q     int8   [kMaxElems]
//   d     float  [kMaxElems / 32]
//   sd    float  [kMaxElems / 32]
//   dbits uint16 [kMaxElems / 32]
//   s16   int16  [kMaxElems / 16]
constexpr size_t kOffQ = 0;
constexpr size_t kOffD = kOffQ + kMaxElems;
constexpr size_t kOffSd = kOffD + kMaxElems / 32 * sizeof(float);
constexpr size_t kOffBits = kOffSd + kMaxElems / 32 * sizeof(float);
constexpr size_t kOffS16 = kOffBits + kMaxElems / 32 * sizeof(uint16_t);
constexpr size_t kBytes = kOffS16 + kMaxElems / 16 * sizeof(int16_t);

// In host code this name is only a handle for the runtime, not an address a kernel may be given.
static __device__ __align__(256) unsigned char g_act_scratch[kBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char *g_dev_ptr[kMaxDevices] = {};

// Device address of the array on `device` (which must be current), looked up once per device.
int scratch_address(smc_ctx *ctx, int device, unsigned char **out)
{
    if (device < 0 || device >= kMaxDevices) return smc_fail(ctx, SMC_E_INVALID, "noalloc: device index %d out of range", device);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_dev_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_act_scratch);
        if (e != cudaSuccess || !p)
            return smc_fail(ctx, SMC_E_CUDA, "noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_dev_ptr[device] = static_cast<unsigned char *>(p);
    }
    *out = g_dev_ptr[device];
    return SMC_OK;
}

}  // namespace

extern "C" int smc_qmatmul_q8_noalloc(smc_ctx *ctx, const float *d_in, const smc_weight *w, float *d_out, int M,
                                      void *stream)
{
    if (!ctx || !d_in || !w || !d_out || M < 0) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_q8_noalloc: bad arguments");
    if (M == 0) return SMC_OK;
    if (!w->fast)
        return smc_fail(ctx, SMC_E_UNSUPPORTED,
                        "qmatmul_q8_noalloc needs a weight registered with SMC_W_REPACK and K %% %d == 0",
                        w->dtype == SMC_Q8_0 ? 32 : 256);
    if ((size_t)M * (size_t)w->K > kMaxElems)
        return smc_fail(ctx, SMC_E_RANGE,
                        "qmatmul_q8_noalloc: M * K = %zu activations exceed the built-in buffer of %zu; use "
                        "smc_qmatmul_dev for larger shapes",
                        (size_t)M * (size_t)w->K, kMaxElems);
    int current = -1;
    SMC_CUDA(ctx, cudaGetDevice(&current));
    if (current != ctx->device) SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    unsigned char *base = nullptr;
    int rc = scratch_address(ctx, ctx->device, &base);
    if (rc) return rc;

    smc_q8act act;  // a view into the fixed array, sized for this call
    act.max_rows = M, act.max_k = w->K;
    act.q = reinterpret_cast<int8_t *>(base + kOffQ);
    act.d = reinterpret_cast<float *>(base + kOffD);
    act.sd = reinterpret_cast<float *>(base + kOffSd);
    act.dbits = reinterpret_cast<uint16_t *>(base + kOffBits);
    act.s16 = reinterpret_cast<int16_t *>(base + kOffS16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = smc_launch_quantize_q8(ctx, d_in, M, w->K, &act, s);
    if (rc) return rc;
    return smc_launch_gemv_q8(ctx, &act, w, d_out, s);
}
