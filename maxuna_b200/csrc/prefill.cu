// Prefill path: expert-sorted grouped GEMM (placeholder until the tensor-core kernel lands).
#include "fused.cuh"

#define NOT_YET(name) return lmoe_fail(LMOE_ERR_UNSUPPORTED, name " is not built yet")

size_t prefill_workspace_bytes(const lmoe_layer *, int64_t) { return 65536; }
lmoe_status launch_moe_prefill(const lmoe_layer *, const float *, int64_t, float *, uint32_t *, float *, void *, size_t,
                               cudaStream_t) { NOT_YET("moe_forward_prefill"); }
extern "C" lmoe_status lmoe_experts_forward_rows(const lmoe_layer *, const float *, const uint32_t *, const float *,
                                                 int64_t, float *, void *, size_t, void *) { NOT_YET("experts_forward_rows"); }
extern "C" lmoe_status lmoe_shared_forward(const lmoe_layer *, const float *, int64_t, float *, void *, size_t,
                                           void *) { NOT_YET("shared_forward"); }
extern "C" int32_t lmoe_mm_id_supported(int32_t, int64_t) { return 0; }
extern "C" size_t lmoe_mm_id_workspace_bytes(int64_t, int64_t, int64_t, int64_t) { return 0; }
extern "C" lmoe_status lmoe_mul_mm_id_shared(const lmoe_expert_stack *, const float *, int64_t, int64_t, int64_t,
                                             const uint32_t *, int64_t, int64_t, const void *, int64_t, int64_t,
                                             int64_t, float *, void *, size_t, void *) { NOT_YET("mul_mm_id_shared"); }
extern "C" lmoe_status lmoe_mul_mm_id(const lmoe_expert_stack *, const float *, int64_t, int64_t, int64_t,
                                      const uint32_t *, int64_t, int64_t, float *, void *, size_t, void *) { NOT_YET("mul_mm_id"); }
