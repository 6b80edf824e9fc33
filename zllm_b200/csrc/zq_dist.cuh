// Peer group of one node for the tensor-parallel row split (zq_dist.cu): one exchange buffer per rank, mapped by all.
#pragma once
#include "zq_common.cuh"

namespace zq {
constexpr int kDistMaxWorld = 8;     // GPUs of one NVSwitch node
constexpr int kDistMaxSlices = 64;   // CTAs of one reduce call (one flag per peer, parity and slice)
constexpr int kDistMaxJobs = 32;     // row-parallel jobs summed by one reduce call

struct DistReduceJob {
    void *y;               // [count] in the output dtype
    const void *residual;  // or null
    size_t count;          // f32 elements of the partial result (rows * m)
};

size_t dist_exchange_bytes(size_t slot_bytes, int world);
int launch_tp_allreduce(zq_ctx *ctx, const DistReduceJob *jobs, size_t n_jobs, int y_dtype, zq_error *err);
}  // namespace zq

struct zq_dist_state {
    int rank = 0, world = 0, max_world = 0;
    size_t slot_bytes = 0;       // bytes one rank may contribute to one call
    size_t exchange_bytes = 0;
    uint8_t *exchange = nullptr; // [2 parities][world][slot_bytes] received partials, then [2][world][slices] u32 flags
    uint8_t *staging = nullptr;  // this rank's partial vector of the current call (f32)
    uint32_t *epoch = nullptr;   // device: reduce calls completed
    uint32_t *done = nullptr;    // device: CTAs of the running reduce call that have finished
    uint8_t *peers[zq::kDistMaxWorld] = {};
    cudaIpcMemHandle_t handle;
    uint64_t wait_ns = 0;        // 0 = default
};
