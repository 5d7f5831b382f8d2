// Host side of the peer-memory exchange (see smc_gather.cuh for the protocol): allocation, CUDA IPC export /
// import of the per-rank buffers, and the entry points that run a row-split matmul followed by the exchange.
#include "smc_gather.cuh"

#include <string.h>

#include "smc_common.cuh"

struct smc_gather {
    int rank = 0, world = 1;
    size_t capacity = 0;           // floats in the dense data area (and packets in each of the two packet areas)
    unsigned char *base = nullptr;  // own allocation: [control block | dense data | packet area 0 | packet area 1]
    void *peer_base[SMC_GATHER_MAX_RANKS] = {};
    bool connected = false;
    smc_gather_dev view{};          // host copy of the device-resident view
    smc_gather_dev *d_view = nullptr;
};

static_assert(sizeof(smc_gather_ctrl) <= SMC_GATHER_CTRL_BYTES, "control block grew past its slot");
static_assert(sizeof(cudaIpcMemHandle_t) == SMC_IPC_HANDLE_BYTES, "IPC handle size");

namespace {

// Exchange of a chunk that earlier launches wrote: the CTAs send stripes of it to every peer as packets, then
// unpack the stripes of the peers' packets.
__global__ void __launch_bounds__(512) gather_exchange_kernel(const smc_gather_dev *g, size_t count)
{
    const unsigned tag = smc_gather_tag(g);
    const float *src = g->data + (size_t)g->rank * count;
    const size_t nth = (size_t)gridDim.x * blockDim.x;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < count; t += nth)
        smc_gather_send(g, count, t, __ldcg(src + t), tag);
    smc_gather_collect(g, count, blockIdx.x, gridDim.x, tag);
    smc_gather_done(g, gridDim.x);
}

// Partial sums gathered as [world][count]: dense[i] = their sum in rank order (the order the fused one-row kernel uses).
__global__ void __launch_bounds__(256) reduce_chunks_kernel(float *data, size_t count, int world)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float sum = 0.f;
    for (int p = 0; p < world; ++p) sum += data[(size_t)p * count + i];
    data[i] = sum;
}

// Exchange of a large chunk: stripes of 16-byte stores straight into every peer's dense area.
__global__ void __launch_bounds__(512) gather_bulk_kernel(const smc_gather_dev *g, size_t count)
{
    __shared__ int s_ok;
    const unsigned tag = smc_gather_tag(g);
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) smc_gather_post_ready(g);
        s_ok = smc_gather_wait_ready(g, tag) ? 1 : 0;
    }
    __syncthreads();
    if (s_ok) {
        const float4 *src = reinterpret_cast<const float4 *>(g->data + (size_t)g->rank * count);
        const size_t n4 = count / 4, nth = (size_t)gridDim.x * blockDim.x;
        for (int i = 1; i < g->world; ++i) {
            const int p = (g->rank + i) % g->world;
            float4 *dst = reinterpret_cast<float4 *>(g->peer_data[p] + (size_t)g->rank * count);
            for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < n4; t += nth) dst[t] = __ldcg(src + t);
        }
    }
    smc_gather_finish_bulk(g, gridDim.x, tag);
}

int upload_view(smc_ctx *ctx, smc_gather *g)
{
    SMC_CUDA(ctx, cudaMemcpy(g->d_view, &g->view, sizeof(g->view), cudaMemcpyHostToDevice));
    SMC_CUDA(ctx, cudaDeviceSynchronize());  // staged copies complete before a kernel on any stream reads the view
    return SMC_OK;
}

}  // namespace

const smc_gather_dev *smc_gather_view(const smc_gather *g) { return g->d_view; }
float *smc_gather_local_chunk(const smc_gather *g, size_t count)
{
    return reinterpret_cast<float *>(g->base + SMC_GATHER_CTRL_BYTES) + (size_t)g->rank * count;
}

extern "C" {

int smc_gather_create(smc_ctx *ctx, int rank, int world, size_t capacity_floats, smc_gather **out)
{
    if (!ctx || !out || world < 1 || world > SMC_GATHER_MAX_RANKS || rank < 0 || rank >= world || capacity_floats == 0)
        return smc_fail(ctx, SMC_E_INVALID, "gather_create: bad arguments (world 1..%d)", SMC_GATHER_MAX_RANKS);
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    smc_gather *g = new smc_gather();
    g->rank = rank, g->world = world;
    g->capacity = (capacity_floats + 3) & ~(size_t)3;
    const size_t bytes = SMC_GATHER_CTRL_BYTES + g->capacity * (sizeof(float) + 2 * sizeof(unsigned long long));
    cudaError_t e = cudaMalloc(&g->base, bytes);
    if (e == cudaSuccess) e = cudaMemset(g->base, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&g->d_view, sizeof(smc_gather_dev));
    if (e != cudaSuccess) {
        cudaFree(g->base);
        delete g;
        return smc_fail(ctx, SMC_E_CUDA, "gather_create: %s", cudaGetErrorString(e));
    }
    g->view.rank = rank, g->view.world = world, g->view.status = ctx->d_status;
    g->view.wait_ns = SMC_GATHER_WAIT_NS;
    g->view.capacity = g->capacity;
    g->view.ctrl[rank] = reinterpret_cast<smc_gather_ctrl *>(g->base);
    g->view.data = reinterpret_cast<float *>(g->base + SMC_GATHER_CTRL_BYTES);
    g->view.peer_data[rank] = g->view.data;
    g->view.pkt[rank] = reinterpret_cast<unsigned long long *>(g->base + SMC_GATHER_CTRL_BYTES + g->capacity * sizeof(float));
    g->connected = world == 1;
    int rc = upload_view(ctx, g);
    if (rc) {
        cudaFree(g->base), cudaFree(g->d_view);
        delete g;
        return rc;
    }
    *out = g;
    return SMC_OK;
}

int smc_gather_export(smc_ctx *ctx, smc_gather *g, unsigned char *handle)
{
    if (!ctx || !g || !handle) return smc_fail(ctx, SMC_E_INVALID, "gather_export: bad arguments");
    cudaIpcMemHandle_t h;
    SMC_CUDA(ctx, cudaIpcGetMemHandle(&h, g->base));
    memcpy(handle, &h, sizeof(h));
    return SMC_OK;
}

int smc_gather_connect(smc_ctx *ctx, smc_gather *g, const unsigned char *handles)
{
    if (!ctx || !g || !handles) return smc_fail(ctx, SMC_E_INVALID, "gather_connect: bad arguments");
    if (g->connected) return smc_fail(ctx, SMC_E_INVALID, "gather_connect: already connected");
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    for (int p = 0; p < g->world; ++p) {
        if (p == g->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)p * SMC_IPC_HANDLE_BYTES, sizeof(h));
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess)
            return smc_fail(ctx, SMC_E_CUDA, "gather_connect: cannot map rank %d's buffer: %s", p, cudaGetErrorString(e));
        g->peer_base[p] = ptr;
        g->view.ctrl[p] = reinterpret_cast<smc_gather_ctrl *>(ptr);
        g->view.pkt[p] = reinterpret_cast<unsigned long long *>(static_cast<unsigned char *>(ptr) + SMC_GATHER_CTRL_BYTES +
                                                                g->capacity * sizeof(float));
        g->view.peer_data[p] = reinterpret_cast<float *>(static_cast<unsigned char *>(ptr) + SMC_GATHER_CTRL_BYTES);
    }
    int rc = upload_view(ctx, g);
    if (rc) return rc;
    g->connected = true;
    return SMC_OK;
}

int smc_gather_connect_local(smc_ctx *ctx, smc_gather *g, smc_gather *const *all)
{
    if (!ctx || !g || !all) return smc_fail(ctx, SMC_E_INVALID, "gather_connect_local: bad arguments");
    if (g->connected) return smc_fail(ctx, SMC_E_INVALID, "gather_connect_local: already connected");
    for (int p = 0; p < g->world; ++p)
        if (!all[p] || all[p]->world != g->world || all[p]->rank != p || all[p]->capacity != g->capacity || (p == g->rank && all[p] != g))
            return smc_fail(ctx, SMC_E_INVALID, "gather_connect_local: entry %d is not rank %d of a world of %d with this capacity", p, p, g->world);
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    for (int p = 0; p < g->world; ++p) {
        if (p == g->rank) continue;
        unsigned char *ptr = all[p]->base;  // same process: the peer's allocation is addressed directly
        g->view.ctrl[p] = reinterpret_cast<smc_gather_ctrl *>(ptr);
        g->view.pkt[p] = reinterpret_cast<unsigned long long *>(ptr + SMC_GATHER_CTRL_BYTES + g->capacity * sizeof(float));
        g->view.peer_data[p] = reinterpret_cast<float *>(ptr + SMC_GATHER_CTRL_BYTES);
    }
    int rc = upload_view(ctx, g);
    if (rc) return rc;
    g->connected = true;
    return SMC_OK;
}

int smc_gather_set_wait_ns(smc_ctx *ctx, smc_gather *g, unsigned long long ns)
{
    if (!ctx || !g || ns == 0) return smc_fail(ctx, SMC_E_INVALID, "gather_set_wait_ns: bad arguments");
    SMC_CUDA(ctx, cudaSetDevice(ctx->device));
    g->view.wait_ns = ns;
    return upload_view(ctx, g);
}

int smc_gather_buffer(smc_ctx *ctx, smc_gather *g, float **d_buf)
{
    if (!ctx || !g || !d_buf) return smc_fail(ctx, SMC_E_INVALID, "gather_buffer: bad arguments");
    *d_buf = reinterpret_cast<float *>(g->base + SMC_GATHER_CTRL_BYTES);
    return SMC_OK;
}

int smc_gather_exchange_dev(smc_ctx *ctx, smc_gather *g, size_t count, void *stream)
{
    if (!ctx || !g) return smc_fail(ctx, SMC_E_INVALID, "gather_exchange: bad arguments");
    if (!g->connected) return smc_fail(ctx, SMC_E_NOT_REGISTERED, "gather_exchange: peers are not connected");
    if (count * (size_t)g->world > g->capacity)
        return smc_fail(ctx, SMC_E_RANGE, "gather_exchange: %zu floats x %d ranks exceed the buffer of %zu", count, g->world,
                        g->capacity);
    if (g->world == 1 || count == 0) return SMC_OK;
    if (count >= (1u << 18) && (count & 3) == 0) {  // a megabyte or more per rank: bulk stores, one fence, one flag
        gather_bulk_kernel<<<ctx->sm_count, 512, 0, static_cast<cudaStream_t>(stream)>>>(g->d_view, count);
        SMC_LAUNCH_CHECK(ctx);
        return SMC_OK;
    }
    int ctas = (int)((count + 1023) / 1024);
    if (ctas < 1) ctas = 1;
    if (ctas > ctx->sm_count) ctas = ctx->sm_count;
    gather_exchange_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(g->d_view, count);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_qmatmul_gather_dev(smc_ctx *ctx, smc_gather *g, const float *d_in, const smc_weight *w, int M, int mode,
                           void *stream)
{
    if (!ctx || !g || !d_in || !w || M < 0) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_gather: bad arguments");
    if (!g->connected) return smc_fail(ctx, SMC_E_NOT_REGISTERED, "qmatmul_gather: peers are not connected");
    const size_t count = (size_t)M * (size_t)w->N;
    if (count * (size_t)g->world > g->capacity)
        return smc_fail(ctx, SMC_E_RANGE, "qmatmul_gather: %d x %d outputs x %d ranks exceed the buffer of %zu floats", M, w->N,
                        g->world, g->capacity);
    if (M == 0) return SMC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float *chunk = smc_gather_local_chunk(g, count);
    if (g->world == 1) return smc_qmatmul_dev(ctx, d_in, w, chunk, M, mode, stream);
    // one row through the TMA kernel: the exchange runs inside the same launch
    bool fused = false;
    int rc = smc_qmatmul_dev_gather(ctx, d_in, w, chunk, M, mode, s, g->d_view, &fused);
    if (rc || fused) return rc;
    return smc_gather_exchange_dev(ctx, g, count, stream);
}

int smc_qmatmul_reduce_dev(smc_ctx *ctx, smc_gather *g, const float *d_in, const float *d_up, const smc_weight *w, int M, int mode,
                           void *stream)
{
    if (!ctx || !g || !d_in || !w || M < 0) return smc_fail(ctx, SMC_E_INVALID, "qmatmul_reduce: bad arguments");
    if (!g->connected) return smc_fail(ctx, SMC_E_NOT_REGISTERED, "qmatmul_reduce: peers are not connected");
    const size_t count = (size_t)M * (size_t)w->N;
    if (count * (size_t)g->world > g->capacity)
        return smc_fail(ctx, SMC_E_RANGE, "qmatmul_reduce: %d x %d partial sums x %d ranks exceed the buffer of %zu floats", M, w->N,
                        g->world, g->capacity);
    if (d_up && (M != 1 || mode != SMC_ACT_Q8 || !smc_tma_supported(w, 1)))
        return smc_fail(ctx, SMC_E_UNSUPPORTED, "qmatmul_reduce: the SiLU-gate input needs one row, SMC_ACT_Q8 and a K the one-row kernel takes");
    if (d_up && ((reinterpret_cast<uintptr_t>(d_in) | reinterpret_cast<uintptr_t>(d_up)) & 15))
        return smc_fail(ctx, SMC_E_INVALID, "qmatmul_reduce: gate and up must be 16-byte aligned");
    if (M == 0) return SMC_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float *dense = reinterpret_cast<float *>(g->base + SMC_GATHER_CTRL_BYTES);
    if (g->world == 1) {  // nothing to add
        if (d_up) return smc_launch_gemv_tma_swiglu(ctx, d_in, d_up, w, dense, s);
        return smc_qmatmul_dev(ctx, d_in, w, dense, M, mode, stream);
    }
    // one row through the bulk-copy kernel: partial sums leave as packets from the lanes that finish them, and the
    // kernel's tail adds the packets of all ranks
    if (M == 1 && mode == SMC_ACT_Q8 && smc_tma_supported(w, 1) && !((reinterpret_cast<uintptr_t>(d_in)) & 15))
        return smc_launch_gemv_tma_any(ctx, nullptr, d_in, d_up, nullptr, w, nullptr, g->d_view, true, false, s);
    // any other shape: partial sums into this rank's chunk, all chunks gathered, then added in the same order
    int rc = smc_qmatmul_dev(ctx, d_in, w, smc_gather_local_chunk(g, count), M, mode, stream);
    if (rc) return rc;
    rc = smc_gather_exchange_dev(ctx, g, count, stream);
    if (rc) return rc;
    reduce_chunks_kernel<<<(unsigned)((count + 255) / 256), 256, 0, s>>>(dense, count, g->world);
    SMC_LAUNCH_CHECK(ctx);
    return SMC_OK;
}

int smc_gather_destroy(smc_ctx *ctx, smc_gather *g)
{
    if (!ctx || !g) return smc_fail(ctx, SMC_E_INVALID, "gather_destroy: bad arguments");
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    for (int p = 0; p < g->world; ++p)
        if (g->peer_base[p]) cudaIpcCloseMemHandle(g->peer_base[p]);
    cudaFree(g->base);
    cudaFree(g->d_view);
    delete g;
    return SMC_OK;
}

}  // extern "C"
