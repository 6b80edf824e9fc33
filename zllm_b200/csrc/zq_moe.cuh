// Resident expert table of a MoE layer and the entry points of the grouped decode path (zq_moe_grouped.cu).
#pragma once
#include <vector>

#include "zq_common.cuh"

struct zq_moe_experts {
    zq_ctx *ctx = nullptr;
    size_t num_experts = 0, hidden = 0, inter = 0;
    std::vector<const zq_weight *> gate, up, down;
    // grouped decode path: the experts' tensor maps as device arrays (gate/up: 64-row boxes, down: 128-row boxes);
    // null when the experts do not all share one gate/up type and one down type
    CUtensorMap *d_gate_maps = nullptr, *d_up_maps = nullptr, *d_down_maps = nullptr;
    // fused prefill GEMM: one-unit boxes of the same tensors
    CUtensorMap *d_gate_qmaps = nullptr, *d_up_qmaps = nullptr, *d_down_qmaps = nullptr;
    uint32_t gate_type = 0, down_type = 0;
};

namespace zq {

// Where the combine of zq_moe_forward puts its rows when the caller is the expert-parallel forward: row r = s * cap + i
// (row i of what source rank s sent) goes, as f32, straight into rank s's return buffer over NVLink, rows beyond the
// count that s sent are skipped, and the last CTA to finish announces the rows to every source ({0, epoch} flags, as the
// separate return kernel did).  Unused (world = 0) everywhere else.
struct PeerRowSink {
    float *base[8] = {};        // per source rank: first row of this rank's block in that rank's return buffer
    uint2 *flag[8] = {};        // per source rank: this rank's return flag in that rank's buffer
    const int *counts = nullptr;  // rows each source sent
    uint32_t *done = nullptr;   // arrival counter of the CTAs (zero between uses)
    uint32_t epoch = 0;
    int cap = 0, world = 0;
};

bool moe_grouped_supported(const zq_moe_experts *t, size_t m, size_t top_k);
size_t moe_grouped_ws_bytes(const zq_moe_experts *t, size_t m, size_t top_k, bool has_shared);
bool moe_shared_rides_along(const zq_moe_experts *t, const zq_weight *sg, const zq_weight *su, const zq_weight *sd);
int moe_grouped_forward(zq_ctx *ctx, const zq_moe_experts *t, const zq_weight *shared_gate, const zq_weight *shared_up, const zq_weight *shared_down, const void *dev_x, int x_dtype, size_t m, const uint32_t *dev_ids,
                        const float *dev_weights, size_t top_k, uint8_t *ws, float **routed_out, uint32_t **token_slots_out, float **token_w_out, float **shared_buf, bool has_shared, zq_error *err);

}  // namespace zq
