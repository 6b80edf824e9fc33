// Expert-parallel MoE forward across the GPUs of one node: token dispatch and combine over peer memory.
//
// Placement: the experts are split into contiguous blocks, rank r owns experts [r E / W, (r + 1) E / W); tokens stay
// data-parallel (every rank brings its own m tokens and their routes with GLOBAL expert ids); the shared expert is
// replicated and runs on the tokens' own rank while the exchange is in flight.  The reference has no such path (its
// experts are cached per device, src/backend/cuda/expert.rs:284-570); what is kept from it is the arithmetic of an
// expert (src/kernel/cpu/moe.rs:122-138) and the order of a token's sum: ascending expert id
// (src/backend/cpu/moe.rs:107-141) - here ascending within an owner rank, owner ranks in ascending order.
//
// One call = five small kernels around the rank's own expert kernels, all on the context's stream:
//   ep_plan       per destination rank, the tokens that have at least one route there, numbered in token order
//   ep_push       each such token ONCE per destination (not once per route): its row and its routes to that rank's
//                 experts (local ids, weights), stored into the destination's dispatch buffer with plain 16-byte
//                 stores over NVLink (memory mapped with CUDA IPC; no multicast, no TMA to or from peer memory); the
//                 last CTA publishes {row count, epoch} to every destination
//   ep_gate       waits (bounded) for every source's count, marks the unused rows of the dispatch buffer "no route"
//   (experts)     zq_moe_forward on the received rows: a token's routes on this rank are weighted and summed HERE, so one
//                 row per (token, rank) travels back; the forward's combine kernel stores those rows straight into the
//                 sources' return buffers (PeerRowSink) and its last CTA publishes the epoch
//   ep_combine    waits (bounded) for every owner rank, then y = residual + shared + sum over ranks in ascending order
// Every wait has a limit in nanoseconds; a wait that runs out sets the device status word and the kernel goes on, so
// nothing hangs (zq_ctx_sync reports it).  A rank finishes a call only after every peer has sent its part of the same
// call, so a rank is never more than one call ahead and a single set of buffers is enough.
#include "zq_dist.cuh"
#include "zq_moe.cuh"

namespace zq {

constexpr int kEpThreads = 256;

__device__ __forceinline__ uint2 ep_ld_flag(const uint2 *p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ep_st_flag(uint2 *p, uint2 v) { asm volatile("st.release.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory"); }
__device__ __forceinline__ uint64_t ep_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Layout of a rank's exchange buffer (the same on every rank):
//   [0, 4 KB)              flags: dispatch[src] at 16 * src, return[owner] at 2048 + 16 * owner  ({count, epoch} words)
//   dispatch rows          [W][C][row_bytes]      rows received from source rank s, in the activation dtype
//   dispatch ids           [W][C][K] u32          local expert ids (ZQ_MOE_NO_ROUTE = none)
//   dispatch weights       [W][C][K] f32
//   return rows            [W][C][H] f32          rows received back from owner rank d, indexed like this rank's sends
struct EpLayout {
    size_t cap, hidden, top_k, row_bytes, world;
    size_t off_rows, off_ids, off_w, off_ret, total;
};
static EpLayout ep_layout(size_t cap, size_t hidden, size_t top_k, size_t esz, size_t world) {
    EpLayout l;
    l.cap = cap; l.hidden = hidden; l.top_k = top_k; l.row_bytes = hidden * esz; l.world = world;
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    l.off_rows = 4096;
    l.off_ids = l.off_rows + al(world * cap * l.row_bytes);
    l.off_w = l.off_ids + al(world * cap * top_k * 4);
    l.off_ret = l.off_w + al(world * cap * top_k * 4);
    l.total = l.off_ret + al(world * cap * hidden * 4);
    return l;
}

struct EpArgs {
    uint8_t *peers[kDistMaxWorld];
    int rank, world, m, top_k, hidden, cap;
    int experts_total;
    int row_vec;              // 16-byte vectors per activation row
    size_t off_rows, off_ids, off_w, off_ret, row_bytes;
    uint32_t epoch;           // this call's tag (never 0)
    uint64_t wait_ns;
    uint32_t *status;
    const void *x;            // [m, hidden] local tokens
    const uint32_t *ids;      // [m, top_k] global expert ids
    const float *weights;     // [m, top_k]
    int *send_idx;            // [world][m]: position of token t among the rows sent to rank d, or -1
    int *send_cnt;            // [world]
    uint32_t *done;           // arrival counter of the pushing kernels
};

__device__ __forceinline__ int ep_owner(uint32_t e, int experts_total, int world) {
    // contiguous blocks whose sizes differ by at most one: the first (E % W) ranks hold one more
    const int base = experts_total / world, extra = experts_total % world, cut = extra * (base + 1);
    return (int)e < cut ? (int)e / (base + 1) : extra + ((int)e - cut) / (base > 0 ? base : 1);
}
__device__ __forceinline__ int ep_first_expert(int r, int experts_total, int world) {
    const int base = experts_total / world, extra = experts_total % world;
    return r * base + (r < extra ? r : extra);
}

// One CTA: for every destination rank, number the tokens that route there in token order.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const EpArgs a) {
    __shared__ int warp_sum[32];
    __shared__ int running;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    for (int d = 0; d < a.world; ++d) {
        if (tid == 0) running = 0;
        __syncthreads();
        for (int t0 = 0; t0 < a.m; t0 += 1024) {
            const int t = t0 + tid;
            int has = 0;
            if (t < a.m)
                for (int j = 0; j < a.top_k; ++j) {
                    const uint32_t e = a.ids[(size_t)t * a.top_k + j];
                    if (e < (uint32_t)a.experts_total && ep_owner(e, a.experts_total, a.world) == d) has = 1;
                }
            int incl = has;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (lane == 31) warp_sum[wid] = incl;
            __syncthreads();
            int before = running;
            for (int w = 0; w < wid; ++w) before += warp_sum[w];
            if (t < a.m) a.send_idx[(size_t)d * a.m + t] = has ? before + incl - 1 : -1;
            __syncthreads();
            if (tid == 1023) running = before + incl;
            __syncthreads();
        }
        if (tid == 0) a.send_cnt[d] = running;
        __syncthreads();
    }
}

// grid (chunks, world): rows and route lists of this rank's tokens into the destination's dispatch buffer.
__global__ void __launch_bounds__(kEpThreads) ep_push_kernel(const EpArgs a) {
    const int d = blockIdx.y;
    uint8_t *dst = a.peers[d];
    uint4 *rows = reinterpret_cast<uint4 *>(dst + a.off_rows + ((size_t)a.rank * a.cap) * a.row_bytes);
    uint32_t *ids = reinterpret_cast<uint32_t *>(dst + a.off_ids) + ((size_t)a.rank * a.cap) * a.top_k;
    float *wts = reinterpret_cast<float *>(dst + a.off_w) + ((size_t)a.rank * a.cap) * a.top_k;
    const int first = ep_first_expert(d, a.experts_total, a.world);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = kEpThreads / 32;
    for (int t = blockIdx.x * warps + warp; t < a.m; t += gridDim.x * warps) {  // one warp per token
        const int i = a.send_idx[(size_t)d * a.m + t];
        if (i < 0 || i >= a.cap) continue;
        const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(a.x) + (size_t)t * a.row_bytes);
        uint4 *out = rows + (size_t)i * a.row_vec;
        for (int v = lane; v < a.row_vec; v += 32) out[v] = src[v];
        if (lane < a.top_k) {
            const uint32_t e = a.ids[(size_t)t * a.top_k + lane];
            const bool mine = e < (uint32_t)a.experts_total && ep_owner(e, a.experts_total, a.world) == d;
            ids[(size_t)i * a.top_k + lane] = mine ? e - (uint32_t)first : ZQ_MOE_NO_ROUTE;
            wts[(size_t)i * a.top_k + lane] = mine ? a.weights[(size_t)t * a.top_k + lane] : 0.f;
        }
    }
    // the last CTA to finish publishes {count, epoch} to every destination
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) s_last = atomicAdd(a.done, 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        if (threadIdx.x < a.world) {
            int n = a.send_cnt[threadIdx.x];
            if (n > a.cap) n = a.cap;
            ep_st_flag(reinterpret_cast<uint2 *>(a.peers[threadIdx.x] + 16 * a.rank), make_uint2((uint32_t)n, a.epoch));
        }
        if (threadIdx.x == 0) *a.done = 0;
    }
}

// One CTA: wait for every source's count, then mark the unused rows of the dispatch buffer as "no route".
__global__ void __launch_bounds__(1024) ep_gate_kernel(const EpArgs a, int *recv_cnt) {
    uint8_t *local = a.peers[a.rank];
    __shared__ int s_cnt[kDistMaxWorld];
    if (threadIdx.x < a.world) {
        const uint2 *flag = reinterpret_cast<const uint2 *>(local + 16 * threadIdx.x);
        const uint64_t t0 = ep_timer_ns();
        uint2 got = ep_ld_flag(flag);
        while (got.y != a.epoch) {
            if (ep_timer_ns() - t0 > a.wait_ns) {  // give up: treat the source as having sent nothing
                atomicMax(a.status, (uint32_t)kStatusPeerTimeout);
                got.x = 0;
                break;
            }
            __nanosleep(100);
            got = ep_ld_flag(flag);
        }
        s_cnt[threadIdx.x] = (int)got.x < a.cap ? (int)got.x : a.cap;
        recv_cnt[threadIdx.x] = s_cnt[threadIdx.x];
    }
    __syncthreads();
    __threadfence_system();  // the rows the flags announce are read by the kernels that follow
    uint32_t *ids = reinterpret_cast<uint32_t *>(local + a.off_ids);
    float *wts = reinterpret_cast<float *>(local + a.off_w);
    const size_t per_src = (size_t)a.cap * a.top_k;
    for (size_t i = threadIdx.x; i < per_src * a.world; i += 1024) {
        const int s = (int)(i / per_src);
        const size_t row = (i - (size_t)s * per_src) / a.top_k;
        if ((int)row >= s_cnt[s]) {
            ids[i] = ZQ_MOE_NO_ROUTE;
            wts[i] = 0.f;
        }
    }
}

// y[t] = residual[t] + shared[t] + sum over owner ranks (ascending) of the row that rank returned for token t.
__global__ void __launch_bounds__(kEpThreads) ep_combine_kernel(const EpArgs a, const float *shared, const void *residual, void *y, int y_dtype) {
    uint8_t *local = a.peers[a.rank];
    if (threadIdx.x < a.world) {
        const uint2 *flag = reinterpret_cast<const uint2 *>(local + 2048 + 16 * threadIdx.x);
        const uint64_t t0 = ep_timer_ns();
        while (ep_ld_flag(flag).y != a.epoch) {
            if (ep_timer_ns() - t0 > a.wait_ns) {
                atomicMax(a.status, (uint32_t)kStatusPeerTimeout);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    __threadfence_system();
    const float4 *ret = reinterpret_cast<const float4 *>(local + a.off_ret);
    const int hv = a.hidden / 4;
    const size_t total = (size_t)a.m * hv;
    for (size_t i = (size_t)blockIdx.x * kEpThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kEpThreads) {
        const int t = (int)(i / hv), c = (int)(i - (size_t)t * hv);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int d = 0; d < a.world; ++d) {
            const int k = a.send_idx[(size_t)d * a.m + t];
            if (k < 0 || k >= a.cap) continue;
            const float4 v = __ldcg(ret + ((size_t)d * a.cap + k) * hv + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float vv[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const size_t o = (size_t)t * a.hidden + 4 * c + q;
            float v = vv[q];
            if (shared) v += shared[o];
            if (residual) v += load_as_f32(residual, y_dtype, o);
            store_from_f32(y, y_dtype, o, v);
        }
    }
}

}  // namespace zq

using namespace zq;

struct zq_ep_state {
    EpLayout layout;
    size_t esz = 0, experts_total = 0;
    uint8_t *exchange = nullptr;
    uint8_t *peers[kDistMaxWorld] = {};
    cudaIpcMemHandle_t handle;
    int *send_idx = nullptr;     // [world][cap]
    int *send_cnt = nullptr;     // [world] + recv_cnt [world]
    uint32_t *done = nullptr;
    float *out_rows = nullptr;   // [world * cap, hidden] f32: this rank's expert outputs for the received rows
    float *shared_out = nullptr; // [cap, hidden] f32
    uint32_t epoch = 0;
    bool mapped = false;
};

extern "C" {

int zq_moe_ep_export(zq_ctx *ctx, size_t max_tokens_per_rank, size_t hidden, size_t top_k, size_t num_experts_total, int x_dtype, void *out_handle, zq_error *err) {
    if (!ctx || !out_handle) return set_error(err, ZQ_ERR_ARG, "zq_moe_ep_export: null argument");
    if (!ctx->dist || ctx->dist->world < 1) return set_error(err, ZQ_ERR_DIST, "zq_moe_ep_export: set up the peer group first (zq_dist_export, zq_dist_init)");
    if (ctx->ep) return set_error(err, ZQ_ERR_DIST, "zq_moe_ep_export: the context already has expert-parallel buffers");
    if (x_dtype != ZQ_F32 && x_dtype != ZQ_F16 && x_dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_moe_ep_export: unknown dtype %d", x_dtype);
    if (max_tokens_per_rank == 0 || hidden == 0 || hidden % 32 || top_k == 0 || top_k > 32 || num_experts_total == 0) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_ep_export: tokens=%zu hidden=%zu (multiple of 32) top_k=%zu (<= 32) experts=%zu", max_tokens_per_rank, hidden, top_k, num_experts_total);
    int rc = use_device(ctx, err);
    if (rc) return rc;
    zq_ep_state *s = new zq_ep_state();
    const size_t world = (size_t)ctx->dist->world;
    s->esz = dtype_size(x_dtype);
    s->experts_total = num_experts_total;
    s->layout = ep_layout(max_tokens_per_rank, hidden, top_k, s->esz, world);
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&s->exchange), s->layout.total);
    if (e == cudaSuccess) e = cudaMemset(s->exchange, 0, 4096);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&s->send_idx), world * max_tokens_per_rank * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&s->send_cnt), 256);
    if (e == cudaSuccess) e = cudaMemset(s->send_cnt, 0, 256);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&s->out_rows), world * max_tokens_per_rank * hidden * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&s->shared_out), max_tokens_per_rank * hidden * sizeof(float));
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&s->handle, s->exchange);
    if (e != cudaSuccess) {
        if (s->exchange) cudaFree(s->exchange);
        if (s->send_idx) cudaFree(s->send_idx);
        if (s->send_cnt) cudaFree(s->send_cnt);
        if (s->out_rows) cudaFree(s->out_rows);
        if (s->shared_out) cudaFree(s->shared_out);
        delete s;
        return set_error(err, ZQ_ERR_CUDA, "zq_moe_ep_export: %s", cudaGetErrorString(e));
    }
    s->done = reinterpret_cast<uint32_t *>(s->send_cnt) + 32;
    memset(out_handle, 0, ZQ_DIST_HANDLE_BYTES);
    memcpy(out_handle, &s->handle, sizeof(cudaIpcMemHandle_t));
    const uint64_t sig = (uint64_t)s->layout.total;  // every rank must have asked for the same sizes
    memcpy(reinterpret_cast<uint8_t *>(out_handle) + sizeof(cudaIpcMemHandle_t), &sig, sizeof(sig));
    ctx->ep = s;
    return ZQ_OK;
}

int zq_moe_ep_init(zq_ctx *ctx, const void *all_handles, zq_error *err) {
    if (!ctx || !all_handles) return set_error(err, ZQ_ERR_ARG, "zq_moe_ep_init: null argument");
    zq_ep_state *s = ctx->ep;
    if (!s || !ctx->dist) return set_error(err, ZQ_ERR_DIST, "zq_moe_ep_init: call zq_moe_ep_export first");
    if (s->mapped) return set_error(err, ZQ_ERR_DIST, "zq_moe_ep_init: the buffers are already mapped");
    int rc = use_device(ctx, err);
    if (rc) return rc;
    const int world = ctx->dist->world, rank = ctx->dist->rank;
    const uint8_t *blobs = reinterpret_cast<const uint8_t *>(all_handles);
    for (int r = 0; r < world; ++r) {
        uint64_t sig = 0;
        memcpy(&sig, blobs + (size_t)r * ZQ_DIST_HANDLE_BYTES + sizeof(cudaIpcMemHandle_t), sizeof(sig));
        if (sig != (uint64_t)s->layout.total) return set_error(err, ZQ_ERR_DIST, "zq_moe_ep_init: rank %d exported buffers of another size", r);
    }
    for (int r = 0; r < world; ++r) {
        cudaIpcMemHandle_t h;
        memcpy(&h, blobs + (size_t)r * ZQ_DIST_HANDLE_BYTES, sizeof(h));
        if (r == rank || !memcmp(&h, &s->handle, sizeof(h))) {
            s->peers[r] = s->exchange;
            continue;
        }
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return set_error(err, ZQ_ERR_DIST, "zq_moe_ep_init: mapping the buffers of rank %d failed: %s", r, cudaGetErrorString(e));
        s->peers[r] = reinterpret_cast<uint8_t *>(p);
    }
    s->mapped = true;
    return ZQ_OK;
}

void zq_moe_ep_shutdown(zq_ctx *ctx) {
    if (!ctx || !ctx->ep) return;
    zq_ep_state *s = ctx->ep;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < kDistMaxWorld; ++r)
        if (s->peers[r] && s->peers[r] != s->exchange) cudaIpcCloseMemHandle(s->peers[r]);
    cudaFree(s->exchange);
    cudaFree(s->send_idx);
    cudaFree(s->send_cnt);
    cudaFree(s->out_rows);
    cudaFree(s->shared_out);
    delete s;
    ctx->ep = nullptr;
}

int zq_moe_forward_ep(zq_ctx *ctx, const zq_moe_experts *local_experts, const zq_weight *shared_gate, const zq_weight *shared_up, const zq_weight *shared_down, const void *dev_x, int x_dtype, size_t m, size_t m_cap,
                      const uint32_t *dev_ids, const float *dev_weights, size_t top_k, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err) {
    if (!ctx || !local_experts || !dev_x || !dev_ids || !dev_weights || !dev_y) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward_ep: null argument");
    zq_ep_state *s = ctx->ep;
    if (!s || !s->mapped || !ctx->dist) return set_error(err, ZQ_ERR_DIST, "zq_moe_forward_ep: expert-parallel buffers are not set up (zq_moe_ep_export, zq_moe_ep_init)");
    const int world = ctx->dist->world, rank = ctx->dist->rank;
    if (m_cap == 0) m_cap = m;
    if (m == 0 || m > m_cap || m_cap > s->layout.cap) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_forward_ep: %zu tokens under a per-rank bound of %zu; the buffers hold up to %zu per rank", m, m_cap, s->layout.cap);
    // this call's layout: the regions are sized by the call's own bound (the same on every rank), inside the allocation
    // made for the largest one, so a decode-sized call does not drag the empty rows of a prefill-sized buffer along
    const EpLayout l = ep_layout(m_cap, s->layout.hidden, s->layout.top_k, s->esz, (size_t)world);
    if (top_k != l.top_k || local_experts->hidden != l.hidden || dtype_size(x_dtype) != s->esz) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_forward_ep: top_k, hidden or dtype differ from what the buffers were made for");
    if (y_dtype != ZQ_F32 && y_dtype != ZQ_F16 && y_dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward_ep: unknown output dtype %d", y_dtype);
    const size_t base = s->experts_total / world, extra = s->experts_total % world;
    const size_t mine = base + ((size_t)rank < extra ? 1 : 0);
    if (local_experts->num_experts != mine) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_forward_ep: rank %d owns %zu of %zu experts, the table holds %zu", rank, mine, s->experts_total, local_experts->num_experts);
    if ((reinterpret_cast<uintptr_t>(dev_x) & 15) || (reinterpret_cast<uintptr_t>(dev_y) & 15) || (reinterpret_cast<uintptr_t>(dev_residual) & 15)) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward_ep: x, y and residual must be 16-byte aligned");
    const bool has_shared = shared_gate || shared_up || shared_down;
    if (has_shared && !(shared_gate && shared_up && shared_down)) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward_ep: shared expert needs gate, up and down");
    int rc = use_device(ctx, err);
    if (rc) return rc;

    EpArgs a;
    for (int r = 0; r < kDistMaxWorld; ++r) a.peers[r] = r < world ? s->peers[r] : nullptr;
    a.rank = rank; a.world = world; a.m = (int)m; a.top_k = (int)top_k; a.hidden = (int)l.hidden; a.cap = (int)l.cap;
    a.experts_total = (int)s->experts_total;
    a.row_vec = (int)(l.row_bytes / 16);
    a.off_rows = l.off_rows; a.off_ids = l.off_ids; a.off_w = l.off_w; a.off_ret = l.off_ret; a.row_bytes = l.row_bytes;
    a.epoch = ++s->epoch;
    if (a.epoch == 0) a.epoch = ++s->epoch;
    a.wait_ns = ctx->dist->wait_ns ? ctx->dist->wait_ns : 2000000000ull;
    a.status = ctx->status_dev;
    a.x = dev_x; a.ids = dev_ids; a.weights = dev_weights;
    a.send_idx = s->send_idx; a.send_cnt = s->send_cnt; a.done = s->done;
    int *recv_cnt = s->send_cnt + 16;

    ep_plan_kernel<<<1, 1024, 0, ctx->stream>>>(a);
    const unsigned chunks = (unsigned)((m + 7) / 8 < 64 ? (m + 7) / 8 : 64);
    ep_push_kernel<<<dim3(chunks, (unsigned)world), kEpThreads, 0, ctx->stream>>>(a);
    ctx->launches += 2;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    // the shared expert works on the rank's own tokens while the rows travel
    if (has_shared) {
        rc = zq_gated_mlp(ctx, shared_gate, shared_up, shared_down, dev_x, x_dtype, m, s->shared_out, ZQ_F32, nullptr, err);
        if (rc) return rc;
    }
    ep_gate_kernel<<<1, 1024, 0, ctx->stream>>>(a, recv_cnt);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    // this rank's experts on everything it received: one output row per received row = the weighted sum of that token's
    // routes on this rank
    // The combine of the local forward writes each summed row straight into its source rank's return buffer and its last
    // CTA sets the return flags: no local copy of the rows, no separate return pass.
    uint8_t *local = s->exchange;
    PeerRowSink sink;
    for (int r = 0; r < world; ++r) {
        sink.base[r] = reinterpret_cast<float *>(s->peers[r] + l.off_ret) + ((size_t)rank * l.cap) * l.hidden;
        sink.flag[r] = reinterpret_cast<uint2 *>(s->peers[r] + 2048 + 16 * rank);
    }
    sink.counts = recv_cnt;
    sink.done = a.done;
    sink.epoch = a.epoch;
    sink.cap = (int)l.cap;
    sink.world = world;
    ctx->moe_row_sink = &sink;
    rc = zq_moe_forward(ctx, local_experts, nullptr, nullptr, nullptr, local + l.off_rows, x_dtype, (size_t)world * l.cap, reinterpret_cast<const uint32_t *>(local + l.off_ids),
                        reinterpret_cast<const float *>(local + l.off_w), top_k, s->out_rows, ZQ_F32, nullptr, err);
    ctx->moe_row_sink = nullptr;
    if (rc) return rc;
    const size_t tot = m * l.hidden / 4;
    size_t cblocks = (tot + kEpThreads - 1) / kEpThreads;
    if (cblocks > (size_t)ctx->sm_count * 8) cblocks = (size_t)ctx->sm_count * 8;
    ep_combine_kernel<<<(unsigned)cblocks, kEpThreads, 0, ctx->stream>>>(a, has_shared ? s->shared_out : nullptr, dev_residual, dev_y, y_dtype);
    ctx->launches += 1;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

}  // extern "C"
