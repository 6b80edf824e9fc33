// Tensor-parallel row split of a projection across the GPUs of one node: the sum of the ranks' partial results without
// a host-launched collective.
//
// A weight W[N, K] that is split by input columns (on 256-column boundaries, the rule of the reference's two-GPU
// operator pair, src/backend/rocm/expert.rs:182-207) gives every rank a partial y_r[m, N]; the result is their sum,
// which the reference forms by exchanging the partials and adding them (src/backend/rocm/expert.rs:1394-1409; its
// fused peer-read join: src/kernel/rocm/hip/peer_copy/source.hip:64-81).  Here every rank owns an exchange buffer that
// all ranks of the node map (CUDA IPC) and the sum is ONE kernel per call, with one NVLink latency on its critical path:
//   push     every thread stores its elements of the rank's partial vector into every peer's buffer as 8-byte words
//            {value, epoch}: ordinary stores (no multicast of any kind, no TMA from or to peer memory).  An aligned 8-byte
//            store arrives whole, so the epoch next to the value says that the value is there: no fence, no separate flag;
//   wait     the same thread polls the words the peers stored for its elements until they show the call's epoch (bounded:
//            a limit in nanoseconds, after which the status word is set and the kernel goes on);
//   add      partials are added in rank order (the same order on every rank: results are identical on all ranks and
//            from run to run), the residual is added, the result is stored in the output dtype.
// Threads are independent of one another, so nothing on a GPU waits for anything else on the same GPU.  Two buffer
// halves alternate by epoch parity: a rank can be at most one call ahead of a peer, because finishing a call needs every
// peer's partial of that call.  The epoch lives in device memory and is advanced by the kernel itself, so the whole call
// (decode kernels + this kernel) can be captured in a CUDA graph and replayed.
#include "zq_dist.cuh"

namespace zq {

constexpr int kDistThreads = 512;
constexpr uint64_t kDistWaitNsDefault = 2000000000ull;  // 2 s

__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const uint2 *p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_v2(uint2 *p, uint2 v) { asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory"); }
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

struct ReduceJob {
    void *y;               // [count] elements in the output dtype
    const void *residual;  // or null
    int begin;             // first element of the job in the partial vector (jobs are padded to multiples of four)
    int count;             // f32 elements
};

struct ReduceArgs {
    ReduceJob jobs[kDistMaxJobs];
    uint8_t *peers[kDistMaxWorld];  // exchange buffer of every rank as mapped here (peers[rank] = the local one)
    int n_jobs, rank, world, y_dtype;
    int total;                      // f32 elements of the whole partial vector
    size_t slot_bytes;              // bytes of one (parity, source rank) slot: 8 per element
    const float *staging;           // this rank's partial vector (local memory)
    uint32_t *epoch;                // local: calls completed so far
    uint32_t *done;                 // local: CTAs of this call that have finished
    uint32_t *status;
    uint64_t wait_ns;
};

__device__ __forceinline__ uint2 *slot_of(uint8_t *base, int parity, int src, int world, size_t slot_bytes) {
    return reinterpret_cast<uint2 *>(base + ((size_t)parity * world + src) * slot_bytes);
}

__global__ void __launch_bounds__(kDistThreads) tp_allreduce_kernel(const __grid_constant__ ReduceArgs a) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // the partial vector is written by the kernels before this one
    const int tid = threadIdx.x, S = gridDim.x;
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(a.epoch);
    const uint32_t tag = e + 1u;  // never 0: the buffer starts zeroed
    const int parity = (int)(e & 1u);
    const int first = blockIdx.x * kDistThreads + tid, stride = S * kDistThreads;
    uint8_t *local = a.peers[a.rank];
    // ---- push: this thread's elements to every peer (their slot for source = this rank)
    for (int i = first; i < a.total; i += stride) {
        const uint2 word = make_uint2(__float_as_uint(a.staging[i]), tag);
        for (int d = 1; d < a.world; ++d) {
            const int dst = (a.rank + d) % a.world;  // start with a different peer on every rank: spreads the link load
            st_relaxed_sys_v2(slot_of(a.peers[dst], parity, a.rank, a.world, a.slot_bytes) + i, word);
        }
    }
    // ---- wait (bounded) and add in rank order, epilogue, store
    const uint64_t t0 = global_timer_ns();
    bool gave_up = false;
    int j = 0;
    for (int i = first; i < a.total; i += stride) {
        // all peers' words of this element are requested together (one round trip when they have already arrived), then
        // each is waited for
        uint2 got[kDistMaxWorld];
#pragma unroll
        for (int src = 0; src < kDistMaxWorld; ++src)
            if (src < a.world && src != a.rank) got[src] = ld_relaxed_sys_v2(slot_of(local, parity, src, a.world, a.slot_bytes) + i);
        float s = 0.f;
#pragma unroll
        for (int src = 0; src < kDistMaxWorld; ++src) {
            if (src >= a.world) break;
            float v;
            if (src == a.rank) {
                v = a.staging[i];
            } else {
                const uint2 *word = slot_of(local, parity, src, a.world, a.slot_bytes) + i;
                while (got[src].y != tag && !gave_up) {
                    if (global_timer_ns() - t0 > a.wait_ns) {  // give up: report, and let the kernel finish on whatever is there
                        gave_up = true;
                        atomicMax(a.status, (uint32_t)kStatusPeerTimeout);
                        break;
                    }
                    got[src] = ld_relaxed_sys_v2(word);
                }
                v = __uint_as_float(got[src].x);
            }
            s += v;
        }
        while (j + 1 < a.n_jobs && a.jobs[j + 1].begin <= i) ++j;
        const ReduceJob &jb = a.jobs[j];
        const int k = i - jb.begin;
        if (k < jb.count) {
            if (jb.residual) s += load_as_f32(jb.residual, a.y_dtype, (size_t)k);
            store_from_f32(jb.y, a.y_dtype, (size_t)k, s);
        }
    }
    // ---- the last CTA of the call advances the epoch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(a.done, 1u);
        if (old == (uint32_t)(S - 1)) {
            *a.done = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(a.epoch) = e + 1u;
        }
    }
}

size_t dist_exchange_bytes(size_t slot_bytes, int world) { return (size_t)2 * world * slot_bytes + 256; }

// Sums the staged partial vector over the ranks into the jobs' outputs.
int launch_tp_allreduce(zq_ctx *ctx, const DistReduceJob *jobs, size_t n_jobs, int y_dtype, zq_error *err) {
    zq_dist_state *d = ctx->dist;
    if (!d) return set_error(err, ZQ_ERR_DIST, "row-parallel reduce: the context has no peer group (zq_dist_init)");
    ReduceArgs a;
    a.n_jobs = (int)n_jobs;
    int total = 0;
    for (size_t i = 0; i < n_jobs; ++i) {
        a.jobs[i].y = jobs[i].y;
        a.jobs[i].residual = jobs[i].residual;
        a.jobs[i].begin = total;
        a.jobs[i].count = (int)jobs[i].count;
        total += (int)((jobs[i].count + 3) & ~size_t(3));
    }
    if ((size_t)total * 8 > d->slot_bytes) return set_error(err, ZQ_ERR_DIST, "row-parallel reduce: %d partial results need %zu bytes of exchange slot, it holds %zu", total, (size_t)total * 8, d->slot_bytes);
    for (int r = 0; r < kDistMaxWorld; ++r) a.peers[r] = r < d->world ? d->peers[r] : nullptr;
    a.rank = d->rank;
    a.world = d->world;
    a.y_dtype = y_dtype;
    a.total = total;
    a.slot_bytes = d->slot_bytes;
    a.staging = reinterpret_cast<const float *>(d->staging);
    a.epoch = d->epoch;
    a.done = d->done;
    a.status = ctx->status_dev;
    a.wait_ns = d->wait_ns ? d->wait_ns : kDistWaitNsDefault;
    // a few elements per thread: the same CTA count on every rank is not required (threads pair up by element index)
    int slices = (total + kDistThreads - 1) / kDistThreads;  // one element per thread while the CTAs last: every wait is one round trip
    if (slices < 1) slices = 1;
    if (slices > kDistMaxSlices) slices = kDistMaxSlices;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)slices);
    cfg.blockDim = dim3(kDistThreads);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tp_allreduce_kernel, a), err);
    ctx->launches++;
    return ZQ_OK;
}

}  // namespace zq

using namespace zq;

extern "C" {

int zq_dist_export(zq_ctx *ctx, size_t slot_bytes, void *out_handle, zq_error *err) {
    if (!ctx || !out_handle) return set_error(err, ZQ_ERR_ARG, "zq_dist_export: null argument");
    if (ctx->dist) return set_error(err, ZQ_ERR_DIST, "zq_dist_export: the context already has an exchange buffer");
    if (slot_bytes == 0 || slot_bytes > (size_t(1) << 30)) return set_error(err, ZQ_ERR_ARG, "zq_dist_export: slot size %zu out of range", slot_bytes);
    int rc = use_device(ctx, err);
    if (rc) return rc;
    slot_bytes = (slot_bytes + 255) & ~size_t(255);
    zq_dist_state *d = new zq_dist_state();
    d->slot_bytes = slot_bytes;
    d->max_world = kDistMaxWorld;
    d->exchange_bytes = dist_exchange_bytes(slot_bytes, kDistMaxWorld);
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&d->exchange), d->exchange_bytes);
    if (e == cudaSuccess) e = cudaMemset(d->exchange, 0, d->exchange_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&d->staging), slot_bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&d->epoch), 256);
    if (e == cudaSuccess) e = cudaMemset(d->epoch, 0, 256);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&d->handle, d->exchange);
    if (e != cudaSuccess) {
        if (d->exchange) cudaFree(d->exchange);
        if (d->staging) cudaFree(d->staging);
        if (d->epoch) cudaFree(d->epoch);
        delete d;
        return set_error(err, ZQ_ERR_CUDA, "zq_dist_export: %s", cudaGetErrorString(e));
    }
    d->done = d->epoch + 16;
    // exported blob: the IPC handle, then the slot size (every rank of a group must use the same one)
    memset(out_handle, 0, ZQ_DIST_HANDLE_BYTES);
    memcpy(out_handle, &d->handle, sizeof(cudaIpcMemHandle_t));
    const uint64_t sb = slot_bytes;
    memcpy(reinterpret_cast<uint8_t *>(out_handle) + sizeof(cudaIpcMemHandle_t), &sb, sizeof(sb));
    ctx->dist = d;
    return ZQ_OK;
}

int zq_dist_init(zq_ctx *ctx, int rank, int world, const void *all_handles, zq_error *err) {
    if (!ctx || !all_handles) return set_error(err, ZQ_ERR_ARG, "zq_dist_init: null argument");
    zq_dist_state *d = ctx->dist;
    if (!d) return set_error(err, ZQ_ERR_DIST, "zq_dist_init: call zq_dist_export first");
    if (d->world) return set_error(err, ZQ_ERR_DIST, "zq_dist_init: the peer group is already set up");
    if (world < 1 || world > kDistMaxWorld || rank < 0 || rank >= world) return set_error(err, ZQ_ERR_ARG, "zq_dist_init: rank %d of %d (at most %d ranks)", rank, world, kDistMaxWorld);
    int rc = use_device(ctx, err);
    if (rc) return rc;
    static_assert(sizeof(cudaIpcMemHandle_t) + sizeof(uint64_t) <= ZQ_DIST_HANDLE_BYTES, "exported blob too small");
    const uint8_t *blobs = reinterpret_cast<const uint8_t *>(all_handles);
    for (int r = 0; r < world; ++r) {
        uint64_t sb = 0;
        memcpy(&sb, blobs + (size_t)r * ZQ_DIST_HANDLE_BYTES + sizeof(cudaIpcMemHandle_t), sizeof(sb));
        if (sb != d->slot_bytes) return set_error(err, ZQ_ERR_DIST, "zq_dist_init: rank %d exported a slot of %llu bytes, this rank one of %zu", r, (unsigned long long)sb, d->slot_bytes);
    }
    for (int r = 0; r < world; ++r) {
        cudaIpcMemHandle_t h;
        memcpy(&h, blobs + (size_t)r * ZQ_DIST_HANDLE_BYTES, sizeof(h));
        // a handle that is this context's own (rank r == this rank, or a loop-back group for tests) maps to the local buffer
        if (r == rank || !memcmp(&h, &d->handle, sizeof(cudaIpcMemHandle_t))) {
            d->peers[r] = d->exchange;
            continue;
        }
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < r; ++q)
                if (d->peers[q] && d->peers[q] != d->exchange) cudaIpcCloseMemHandle(d->peers[q]);
            for (int q = 0; q < kDistMaxWorld; ++q) d->peers[q] = nullptr;
            return set_error(err, ZQ_ERR_DIST, "zq_dist_init: mapping the exchange buffer of rank %d failed: %s", r, cudaGetErrorString(e));
        }
        d->peers[r] = reinterpret_cast<uint8_t *>(p);
    }
    d->rank = rank;
    d->world = world;
    // the slot layout depends on the group size: re-derive it for `world` ranks inside the allocation made for the maximum
    return ZQ_OK;
}

int zq_dist_set_wait_ms(zq_ctx *ctx, unsigned milliseconds, zq_error *err) {
    if (!ctx || !ctx->dist) return set_error(err, ZQ_ERR_DIST, "zq_dist_set_wait_ms: the context has no peer group");
    ctx->dist->wait_ns = (uint64_t)milliseconds * 1000000ull;
    return ZQ_OK;
}

int zq_dist_rank(const zq_ctx *ctx) { return ctx && ctx->dist && ctx->dist->world ? ctx->dist->rank : 0; }
int zq_dist_world(const zq_ctx *ctx) { return ctx && ctx->dist && ctx->dist->world ? ctx->dist->world : 1; }

void zq_dist_shutdown(zq_ctx *ctx) {
    if (!ctx || !ctx->dist) return;
    zq_dist_state *d = ctx->dist;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < kDistMaxWorld; ++r)
        if (d->peers[r] && d->peers[r] != d->exchange) cudaIpcCloseMemHandle(d->peers[r]);
    if (d->exchange) cudaFree(d->exchange);
    if (d->staging) cudaFree(d->staging);
    if (d->epoch) cudaFree(d->epoch);
    delete d;
    ctx->dist = nullptr;
}

}  // extern "C"
