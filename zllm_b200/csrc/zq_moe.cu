// MoE entry points (router, resident expert table, routed forward).
#include "zq_common.cuh"

using namespace zq;

struct zq_moe_experts {
    zq_ctx *ctx = nullptr;
    size_t num_experts = 0;
    std::vector<const zq_weight *> gate, up, down;
};

extern "C" {
int zq_moe_route_softmax_topk(zq_ctx *, const void *, int, size_t, size_t, const float *, const float *, size_t, size_t, float, int, uint32_t *, float *, zq_error *err) {
    return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_moe_route_softmax_topk: not built yet");
}
int zq_moe_experts_create(zq_ctx *, const zq_weight *const *, const zq_weight *const *, const zq_weight *const *, size_t, zq_moe_experts **, zq_error *err) {
    return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_moe_experts_create: not built yet");
}
void zq_moe_experts_destroy(zq_moe_experts *experts) { delete experts; }
int zq_moe_forward(zq_ctx *, const zq_moe_experts *, const zq_weight *, const zq_weight *, const zq_weight *, const void *, int, size_t, const uint32_t *, const float *, size_t, void *, int, const void *, zq_error *err) {
    return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_moe_forward: not built yet");
}
}
