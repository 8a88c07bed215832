// Header-only C++ host layer over the C ABI of include/lmoe.h, mirroring the names of the
// reference's Rust items for the MoE path:
//   laguna::ExpertStack            src/gguf.rs:247-276
//   laguna::ops::mul_mv_id ...     src/ops/mv_id.rs:37, src/ops/mm_id.rs:16-50,
//                                  src/ops/silu_mul.rs:14, src/ops/combine.rs:16
//   laguna::MoeBlock               src/moe.rs:28-79 (route / forward)
// Tensors are plain device pointers with explicit shapes (the reference passes candle
// tensors); every call returns laguna::Result: ok() or the message of the failed check,
// like the reference's anyhow::Result -- never a GPU fault.  Outputs are caller-allocated.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <utility>

#include "../../include/lmoe.h"

namespace laguna {

struct Result {
    lmoe_status status = LMOE_OK;
    std::string message;
    bool ok() const { return status == LMOE_OK; }
    explicit operator bool() const { return ok(); }
    static Result from(lmoe_status st) {
        Result r;
        r.status = st;
        if (st != LMOE_OK) r.message = lmoe_last_error();
        return r;
    }
};

enum class GgmlDType : int32_t { Q4K = LMOE_Q4_K, Q6K = LMOE_Q6_K };

// Stacked per-expert weights kept in their quantized GGUF layout.
class ExpertStack {
public:
    ExpertStack() = default;
    ExpertStack(const ExpertStack &) = delete;
    ExpertStack &operator=(const ExpertStack &) = delete;
    ExpertStack(ExpertStack &&o) noexcept { *this = std::move(o); }
    ExpertStack &operator=(ExpertStack &&o) noexcept {
        reset();
        h_ = o.h_; dtype = o.dtype; n_expert = o.n_expert; n_out = o.n_out; k = o.k; base_off = o.base_off;
        o.h_ = nullptr;
        return *this;
    }
    ~ExpertStack() { reset(); }

    // `Weights::expert_stack` (classic load): one upload of the raw super-blocks.
    static Result upload(GgmlDType dt, int64_t n_expert, int64_t n_out, int64_t k, const void *host_bytes, size_t nbytes,
                         ExpertStack &out, size_t base_off = 0) {
        lmoe_expert_stack *h = nullptr;
        Result r = Result::from(lmoe_expert_stack_create((int32_t)dt, n_expert, n_out, k, host_bytes, nbytes, base_off, &h));
        if (r) out.adopt(h, dt, n_expert, n_out, k, base_off);
        return r;
    }
    // Zero-copy view over bytes already in device memory (the mmap-alias load's counterpart).
    static Result view(GgmlDType dt, int64_t n_expert, int64_t n_out, int64_t k, const void *device_base, size_t nbytes,
                       size_t base_off, ExpertStack &out) {
        lmoe_expert_stack *h = nullptr;
        Result r = Result::from(lmoe_expert_stack_wrap((int32_t)dt, n_expert, n_out, k, device_base, nbytes, base_off, &h));
        if (r) out.adopt(h, dt, n_expert, n_out, k, base_off);
        return r;
    }
    const lmoe_expert_stack *handle() const { return h_; }

    GgmlDType dtype = GgmlDType::Q4K;
    int64_t n_expert = 0, n_out = 0, k = 0;
    size_t base_off = 0;

private:
    void adopt(lmoe_expert_stack *h, GgmlDType dt, int64_t ne, int64_t no, int64_t kk, size_t off) {
        reset();
        h_ = h; dtype = dt; n_expert = ne; n_out = no; k = kk; base_off = off;
    }
    void reset() {
        if (h_) lmoe_expert_stack_destroy(h_);
        h_ = nullptr;
    }
    lmoe_expert_stack *h_ = nullptr;
};

// The geometry a map0 scratch was laid out for (`Map0Scratch`, src/ops/dispatch.rs:752-757).
struct Map0Scratch {
    void *buffer = nullptr; // device, lmoe_map0_scratch_bytes(n_expert, t)
    int64_t n_expert = 0, t = 0, top_k = 0;
};

namespace ops {

inline Result mul_mv_id(const ExpertStack &stack, const float *x, int64_t t, int64_t x_per_row, int64_t k,
                        const uint32_t *ids, int64_t t_ids, int64_t top_k, float *out, void *stream) {
    return Result::from(lmoe_mul_mv_id(stack.handle(), x, t, x_per_row, k, ids, t_ids, top_k, out, stream));
}
inline Result mul_mv(const void *weight, GgmlDType dt, int64_t n_out, int64_t k, const float *x, int64_t t, float *out,
                     void *stream) {
    return Result::from(lmoe_mul_mv(weight, (int32_t)dt, n_out, k, x, t, out, stream));
}
inline Result prepare_map0(int64_t n_expert, const uint32_t *ids, int64_t t, int64_t top_k, void *scratch,
                           size_t scratch_bytes, void *stream, Map0Scratch &out) {
    Result r = Result::from(lmoe_prepare_map0(ids, t, top_k, n_expert, scratch, scratch_bytes, stream));
    if (r) out = Map0Scratch{scratch, n_expert, t, top_k};
    return r;
}
inline bool supported(GgmlDType dt, int64_t top_k) { return lmoe_mm_id_supported((int32_t)dt, top_k) != 0; }
inline Result mul_mm_id_shared(const ExpertStack &stack, const float *x, int64_t t, int64_t x_per_row, int64_t k,
                               const uint32_t *ids, int64_t t_ids, int64_t top_k, const Map0Scratch &scratch, float *out,
                               void *workspace, size_t workspace_bytes, void *stream) {
    return Result::from(lmoe_mul_mm_id_shared(stack.handle(), x, t, x_per_row, k, ids, t_ids, top_k, scratch.buffer,
                                              scratch.n_expert, scratch.t, scratch.top_k, out, workspace, workspace_bytes,
                                              stream));
}
inline Result mul_mm_id(const ExpertStack &stack, const float *x, int64_t t, int64_t x_per_row, int64_t k,
                        const uint32_t *ids, int64_t t_ids, int64_t top_k, float *out, void *workspace,
                        size_t workspace_bytes, void *stream) {
    return Result::from(lmoe_mul_mm_id(stack.handle(), x, t, x_per_row, k, ids, t_ids, top_k, out, workspace,
                                       workspace_bytes, stream));
}
inline Result silu_mul(const float *gate, const float *up, int64_t n, float *out, void *stream) {
    return Result::from(lmoe_silu_mul(gate, up, n, out, stream));
}
inline Result combine(const float *down, const float *col_l2, const float *weights, int64_t seq, int64_t top_k,
                      int64_t n_out, float *out, void *stream) {
    return Result::from(lmoe_combine(down, col_l2, weights, seq, top_k, n_out, out, stream));
}

} // namespace ops

// One MoE FFN block: route -> routed experts -> + shared expert.
class MoeBlock {
public:
    MoeBlock() = default;
    MoeBlock(const MoeBlock &) = delete;
    MoeBlock &operator=(const MoeBlock &) = delete;
    ~MoeBlock() { if (h_) lmoe_layer_destroy(h_); }

    // `MoeBlock::new`: the stacks, router [n_expert, hidden] and bias stay owned by the caller.
    Result init(int64_t hidden, int64_t expert_ff, int64_t n_expert, int64_t n_expert_used, float weights_scale,
                bool weights_norm, const float *router, const float *exp_probs_b, const ExpertStack &gate,
                const ExpertStack &up, const ExpertStack &down, const ExpertStack *sh_gate = nullptr,
                const ExpertStack *sh_up = nullptr, const ExpertStack *sh_down = nullptr) {
        hidden_ = hidden; n_expert_ = n_expert; top_k_ = n_expert_used; scale_ = weights_scale; norm_ = weights_norm;
        router_ = router; bias_ = exp_probs_b;
        return Result::from(lmoe_layer_create(hidden, expert_ff, n_expert, n_expert_used, weights_scale, weights_norm ? 1 : 0,
                                              router, exp_probs_b, gate.handle(), up.handle(), down.handle(),
                                              sh_gate ? sh_gate->handle() : nullptr, sh_up ? sh_up->handle() : nullptr,
                                              sh_down ? sh_down->handle() : nullptr, &h_));
    }
    size_t workspace_bytes(int64_t max_tokens) const { return lmoe_layer_workspace_bytes(h_, max_tokens); }

    // `MoeBlock::route`: (ids [seq, top_k] u32, weights [seq, top_k] f32), both on the device.
    Result route(const float *x_normed, int64_t seq, uint32_t *ids, float *weights, void *workspace, size_t workspace_bytes,
                 void *stream) const {
        return Result::from(lmoe_route(router_, bias_, x_normed, seq, hidden_, n_expert_, top_k_, scale_, norm_ ? 1 : 0, ids,
                                       weights, workspace, workspace_bytes, stream));
    }
    // `MoeBlock::forward`: the mat-vec path below lmoe_mm_id_min_seq() tokens, the grouped GEMM from there on
    // (the same rule as lmoe_moe_forward_host and lmoe_moe_layer_forward).
    Result forward(const float *x_normed, int64_t seq, float *out, void *workspace, size_t workspace_bytes, void *stream,
                   uint32_t *ids_out = nullptr, float *weights_out = nullptr) const {
        if (seq >= lmoe_mm_id_min_seq())
            return Result::from(lmoe_moe_forward_prefill(h_, x_normed, seq, out, ids_out, weights_out, workspace,
                                                         workspace_bytes, stream));
        return Result::from(lmoe_moe_forward_decode(h_, x_normed, seq, out, ids_out, weights_out, workspace, workspace_bytes,
                                                    stream));
    }
    // `ExpertFfn::forward` (src/moe.rs:19-21): the routed experts on the caller's routing decision.
    size_t experts_workspace_bytes(int64_t max_tokens) const { return lmoe_experts_workspace_bytes(h_, max_tokens); }
    Result experts_forward(const float *x, const uint32_t *ids, const float *weights, int64_t seq, float *out, void *workspace,
                           size_t workspace_bytes, void *stream, bool add_shared = false) const {
        return Result::from(lmoe_experts_forward(h_, x, ids, weights, seq, add_shared ? 1 : 0, out, workspace, workspace_bytes,
                                                 stream));
    }
    // The FFN half of a layer (src/model.rs:340-350): out = ffn_inp + forward(ffn_norm(ffn_inp)).
    size_t layer_workspace_bytes(int64_t max_tokens) const { return lmoe_moe_layer_workspace_bytes(h_, max_tokens); }
    Result layer_forward(const float *ffn_inp, const float *ffn_norm_weight, float rms_eps, int64_t seq, float *out,
                         void *workspace, size_t workspace_bytes, void *stream, uint32_t *ids_out = nullptr,
                         float *weights_out = nullptr) const {
        return Result::from(lmoe_moe_layer_forward(h_, ffn_inp, ffn_norm_weight, rms_eps, seq, out, ids_out, weights_out,
                                                   workspace, workspace_bytes, stream));
    }
    const lmoe_layer *handle() const { return h_; }

private:
    lmoe_layer *h_ = nullptr;
    int64_t hidden_ = 0, n_expert_ = 0, top_k_ = 0;
    float scale_ = 1.f;
    bool norm_ = true;
    const float *router_ = nullptr, *bias_ = nullptr;
};

} // namespace laguna
