// Exchange step of a row-split matmul over peer memory: every rank's output slice is stored straight into
// every other rank's receive area through NVLink by the kernel that computes it, instead of a library
// all-gather after it.
//
// One object per rank owns a single device allocation [control block | dense data | two packet areas]; peers map
// it through CUDA IPC.  The dense data is [world][count] floats (chunk r = rank r's slice), what later
// launches read.  A value travels as one 8-byte packet {float bits, tag}, written with a single 64-bit store
// (single-copy atomic), so the receiver needs no fence and no separate flag: a packet whose tag equals the
// number of the running exchange is complete.  System-scope fences cost several microseconds each on this
// platform (measured: a fence + flag protocol took 12 us per exchange, a plain peer copy 2 us), which is why
// none is used.  Protocol for exchange number t = epoch + 1 (a counter in device memory, so a captured graph replays):
//   1. a thread that has produced an output value stores it into the local dense chunk and as a packet tagged t
//      into packet area (t & 1) of every peer;
//   2. when a CTA has finished its own rows it turns a stripe of the incoming packets of every peer into
//      dense floats, polling each packet until its tag is t.  The kernel therefore completes when the whole
//      gathered row is in local memory, and later launches on the stream just read it;
//   3. the CTA that finishes last advances the exchange counter.
// Why two packet areas make a hand-shake unnecessary: a packet of exchange t overwrites one of exchange t - 2.  A rank
// starts sending for t only after its own exchange t - 1 has completed, i.e. after it has received every peer's
// packets of t - 1; a peer sends those only after ITS exchange t - 2 has completed (its kernels are ordered on its
// stream, and a dependent launch sends only behind its grid-dependency wait), which includes having read all packets
// of t - 2.  So nobody can still be reading what is overwritten.  (A single area needed a "my readers are done" flag
// per peer and one more NVLink round trip per exchange.)
// Partial sums (a matmul split along K) use the same packets in "reduce" form: every rank sends its partial of EVERY
// output, to itself as well, and step 2 adds the `world` packets of an output in rank order into dense[i] — the same
// fp32 additions in the same order on every rank, so all ranks hold bit-identical sums.
// Large chunks go as plain stores into the peers' dense areas behind the ready / arrived flags below (bulk form).
// Every wait is bounded by wall time; a wait that runs out raises the context's status word and the kernel
// still finishes (the context stays usable, the data of that exchange is invalid).
#pragma once

#include <stdint.h>

#define SMC_GATHER_MAX_RANKS 8
#define SMC_GATHER_CTRL_BYTES 256
#define SMC_GATHER_WAIT_NS 2000000000ull  // default limit of every wait: 2 s (smc_gather_set_wait_ns changes it per object)

// Control block at the start of each rank's allocation (what peers address).
struct smc_gather_ctrl {
    unsigned ready[SMC_GATHER_MAX_RANKS];    // bulk form: ready[r] = tag: rank r's readers of the previous exchange are done
    unsigned arrived[SMC_GATHER_MAX_RANKS];  // bulk exchanges: arrived[r] = e+1 once rank r's whole chunk is here
    unsigned ticket;                       // CTAs of the running producer that have finished
    unsigned epoch;                        // exchanges completed by this rank
};

// Per-rank view, resident in device memory, handed to kernels by pointer.
struct smc_gather_dev {
    smc_gather_ctrl *ctrl[SMC_GATHER_MAX_RANKS];     // ctrl[r]: rank r's control block as mapped on this device
    unsigned long long *pkt[SMC_GATHER_MAX_RANKS];   // pkt[r]: rank r's two packet areas (2 x capacity packets) as mapped on this device
    size_t capacity;                                 // packets per area
    float *peer_data[SMC_GATHER_MAX_RANKS];          // peer_data[r]: rank r's dense data area as mapped on this device
    float *data;                                     // this rank's dense data area
    int rank, world;
    int *status;  // the context's status word
    unsigned long long wait_ns;  // limit of every wait of an exchange on this object
};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned smc_ld_relaxed_sys(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void smc_st_relaxed_sys(unsigned *p, unsigned v)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long smc_ld_relaxed_sys64(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void smc_st_relaxed_sys64(unsigned long long *p, unsigned long long v)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long smc_globaltimer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned smc_gather_tag(const smc_gather_dev *g)
{
    return *(volatile unsigned *)&g->ctrl[g->rank]->epoch + 1u;
}

// Bulk form only (stores go straight into the peers' dense areas, which their later launches read): one thread of one
// CTA tells every peer at the start of the kernel "my readers of the previous exchange are done" (ready[rank] = tag, a
// relaxed store: stream order already put those readers before this kernel).
__device__ __forceinline__ void smc_gather_post_ready(const smc_gather_dev *g)
{
    const unsigned tag = smc_gather_tag(g);
    for (int p = 0; p < g->world; ++p)
        if (p != g->rank) smc_st_relaxed_sys(&g->ctrl[p]->ready[g->rank], tag);
}

// Bulk form only: a thread calls this before the first store into a peer's dense area.  False when a peer did not
// show up in time: the caller then sends nothing.
__device__ __forceinline__ bool smc_gather_wait_ready(const smc_gather_dev *g, unsigned tag)
{
    const smc_gather_ctrl *me = g->ctrl[g->rank];
    unsigned long long t0 = 0;
    for (int p = 0; p < g->world; ++p) {
        if (p == g->rank) continue;
        unsigned polls = 0;
        while ((int)(smc_ld_relaxed_sys(&me->ready[p]) - tag) < 0) {
            if ((++polls & 63u) == 0) {
                if (!t0) t0 = smc_globaltimer();
                else if (smc_globaltimer() - t0 > g->wait_ns) {
                    atomicExch(g->status, 2);
                    return false;
                }
            }
        }
    }
    return true;
}

// Packet area of exchange `tag` inside rank r's allocation.
__device__ __forceinline__ unsigned long long *smc_gather_area(const smc_gather_dev *g, int r, unsigned tag)
{
    return g->pkt[r] + (size_t)(tag & 1u) * g->capacity;
}

// Step 1 for a whole warp that holds `v` in every lane: lane p sends to peer p (`self`: to this rank as well, the
// reduce form).
__device__ __forceinline__ void smc_gather_send_warp(const smc_gather_dev *g, size_t count, size_t idx, float v, unsigned tag,
                                                     bool self = false)
{
    const int lane = threadIdx.x & 31;
    if (lane < g->world && (self || lane != g->rank))
        smc_st_relaxed_sys64(smc_gather_area(g, lane, tag) + (size_t)g->rank * count + idx,
                             ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v));
}

// Step 1: element `idx` of this rank's chunk of `count` floats.
__device__ __forceinline__ void smc_gather_send(const smc_gather_dev *g, size_t count, size_t idx, float v, unsigned tag,
                                                bool self = false)
{
    const unsigned long long pk = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    for (int p = 0; p < g->world; ++p)
        if (self || p != g->rank) smc_st_relaxed_sys64(smc_gather_area(g, p, tag) + (size_t)g->rank * count + idx, pk);
}

// Step 2: every thread of every CTA, after the CTA's own sends.  CTA `cta` of `total` unpacks its stripe of every
// peer's chunk; the (peer, element) pairs are spread over the threads so that all peers are polled at once.
__device__ __forceinline__ void smc_gather_collect(const smc_gather_dev *g, size_t count, unsigned cta, unsigned total,
                                                   unsigned tag)
{
    const size_t per = (count + total - 1) / total;
    const size_t lo = (size_t)cta * per, hi = lo + per < count ? lo + per : count;
    if (lo >= hi) return;
    const size_t span = hi - lo, items = span * (size_t)(g->world - 1);
    bool dead = false;
    for (size_t it = threadIdx.x; it < items; it += blockDim.x) {
        const int p = (g->rank + 1 + (int)(it / span)) % g->world;
        const size_t t = lo + it % span;
        const unsigned long long *src = smc_gather_area(g, g->rank, tag) + (size_t)p * count + t;
        unsigned long long pk = smc_ld_relaxed_sys64(src);
        if ((unsigned)(pk >> 32) != tag && !dead) {
            const unsigned long long t0 = smc_globaltimer();
            unsigned polls = 0;
            while ((unsigned)((pk = smc_ld_relaxed_sys64(src)) >> 32) != tag) {
                if ((++polls & 63u) == 0 && smc_globaltimer() - t0 > g->wait_ns) {
                    dead = true;
                    atomicExch(g->status, 2);
                    break;
                }
            }
        }
        g->data[(size_t)p * count + t] = __uint_as_float((unsigned)pk);
    }
}

// Step 2 in reduce form: dense[i] = sum over ranks, in rank order, of the packets of output i (this rank's own
// included).  All `world` packets of an output are requested at once; the ones that have not arrived are polled.
__device__ __forceinline__ void smc_gather_collect_reduce(const smc_gather_dev *g, size_t count, unsigned cta, unsigned total,
                                                          unsigned tag)
{
    const size_t per = (count + total - 1) / total;
    const size_t lo = (size_t)cta * per, hi = lo + per < count ? lo + per : count;
    bool dead = false;
    const unsigned long long *area = smc_gather_area(g, g->rank, tag);
    for (size_t t = lo + threadIdx.x; t < hi; t += blockDim.x) {
        unsigned long long pk[SMC_GATHER_MAX_RANKS];
#pragma unroll
        for (int p = 0; p < SMC_GATHER_MAX_RANKS; ++p)
            if (p < g->world) pk[p] = smc_ld_relaxed_sys64(area + (size_t)p * count + t);
        float sum = 0.f;
#pragma unroll
        for (int p = 0; p < SMC_GATHER_MAX_RANKS; ++p) {
            if (p >= g->world) break;
            if ((unsigned)(pk[p] >> 32) != tag && !dead) {
                const unsigned long long *src = area + (size_t)p * count + t;
                const unsigned long long t0 = smc_globaltimer();
                unsigned polls = 0;
                while ((unsigned)((pk[p] = smc_ld_relaxed_sys64(src)) >> 32) != tag) {
                    if ((++polls & 63u) == 0 && smc_globaltimer() - t0 > g->wait_ns) {
                        dead = true;
                        atomicExch(g->status, 2);
                        break;
                    }
                }
            }
            sum += __uint_as_float((unsigned)pk[p]);
        }
        g->data[t] = sum;
    }
}

// Large slices (megabytes) go as plain 16-byte stores into the peers' dense areas instead of packets: half the bytes
// on the wire, at the price of one system-scope fence and a flag per exchange, which no longer matters at that size.
__device__ __forceinline__ unsigned smc_ld_acquire_sys(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void smc_st_release_sys(unsigned *p, unsigned v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Every thread of every CTA, after the CTA's stores into the peers' dense areas.  The CTA that arrives last posts
// "chunk complete" to every peer, waits for theirs and advances the exchange counter.
__device__ __forceinline__ void smc_gather_finish_bulk(const smc_gather_dev *g, unsigned total_ctas, unsigned tag)
{
    __shared__ unsigned s_last;
    smc_gather_ctrl *me = g->ctrl[g->rank];
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();  // this CTA's stores into peer memory are performed before the ticket is taken
        s_last = (atomicAdd(&me->ticket, 1u) == total_ctas - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int p = 0; p < g->world; ++p)
            if (p != g->rank) smc_st_release_sys(&g->ctrl[p]->arrived[g->rank], tag);
    }
    if (threadIdx.x < (unsigned)g->world && (int)threadIdx.x != g->rank) {
        const unsigned long long t0 = smc_globaltimer();
        unsigned polls = 0;
        while ((int)(smc_ld_acquire_sys(&me->arrived[threadIdx.x]) - tag) < 0) {
            if ((++polls & 63u) == 0 && smc_globaltimer() - t0 > g->wait_ns) {
                atomicExch(g->status, 2);
                break;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        me->ticket = 0;
        me->epoch = tag;
    }
}

// Step 4: every thread of every CTA, last thing in the kernel.
__device__ __forceinline__ void smc_gather_done(const smc_gather_dev *g, unsigned total_ctas)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        smc_gather_ctrl *me = g->ctrl[g->rank];
        const unsigned e = *(volatile unsigned *)&me->epoch;
        __threadfence();
        if (atomicAdd(&me->ticket, 1u) == total_ctas - 1) {
            me->ticket = 0;
            me->epoch = e + 1;
        }
    }
}
#endif
